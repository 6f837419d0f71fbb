"""The Gupizen design in the engine against the plain implementation (tests/plain/gupizen.py).

The tests make their own small configurations and their own weights (tests/gupizen_models.py): each mechanism alone,
whole prompts against token-by-token decoding, pieces down to two tokens, unequal batches against each request alone,
slots and pages used again, keys just inside and just outside every window in prompts and in decoding (with weights
under which ONE key holds the attention's weight, and controls that a window one token off would show), the sink, the
first tokens, long decoding (recurrent states and the windows' freed pages carried for hundreds of steps), sizes that
are no multiple of 8, one head, one expert, one tap, a window of one token, loops from the first layer on, and greedy
generation through the package's entry point.

Tolerances. 32-bit: ||ref - got|| / ||ref|| of every row of logits within 1e-4 (the recurrent layers carry rounding
along a sequence). bfloat16: a row's ||ref - got|| is set against the request's typical row norm (the root mean square
of ||ref|| over its rows); the mean over a request's rows within 5e-2, and every row within 2e-1 but for at most one
row in fifty: the router picks by comparing logits, and a token whose last chosen and first unchosen logits lie closer
than bfloat16 resolves may take the other expert, which moves that row (and, through the recurrent states, a few
after it) by a visible amount; no row may be off by more than 1. What the schedule changes is held separately against
the engine's own whole run, the same way with 2e-2 and 1e-1. A lost state, a wrong edge or a stale page moves rows by
their whole size, and the 32-bit runs of the same tests hold every row to 1e-4.
"""
import json
import os

import numpy as np
import pytest

import gupizen_models as gm
from helpers import assert_close, rel_err
from plain import gupizen as plain

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_MEAN_TOL, BF16_ROW_TOL, BF16_SCHEDULE_MEAN_TOL, BF16_SCHEDULE_ROW_TOL = 5e-2, 2e-1, 2e-2, 1e-1
DTYPES = ["float32", "bfloat16"]


def _bf16_rows(rows, mean_tol, row_tol, what):
    assert rows.mean() <= mean_tol, f"{what}: mean rel error {rows.mean():.3e}"
    over = int((rows > row_tol).sum())
    assert over <= max(1, len(rows) // 50), f"{what}: {over} of {len(rows)} rows over {row_tol}, the first at {int(np.argmax(rows > row_tol))}"
    assert rows.max() <= 1.0, f"{what}: row {int(rows.argmax())} has rel error {rows.max():.3e}"


def close(ref, got, dtype, what, whole=None):
    """`got` against the plain implementation's `ref`; in bfloat16 also against the engine's own whole run."""
    if dtype == "float32":
        return assert_close(ref, got, FP32_TOL, what)
    ref, got = np.asarray(ref, dtype=np.float64), np.asarray(got, dtype=np.float64)
    assert ref.shape == got.shape and np.all(np.isfinite(got)), what
    scale = max(float(np.sqrt((np.linalg.norm(ref, axis=-1) ** 2).mean())), 1e-30)
    _bf16_rows(np.linalg.norm(ref - got, axis=-1) / scale, BF16_MEAN_TOL, BF16_ROW_TOL, what)
    if whole is not None:
        _bf16_rows(np.linalg.norm(np.asarray(whole, dtype=np.float64) - got, axis=-1) / scale, BF16_SCHEDULE_MEAN_TOL,
                   BF16_SCHEDULE_ROW_TOL, what + " against the whole run")


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return gm.write_models(tmp_path_factory.mktemp("gupizen"))


_ENGINES = {}
_PLAIN = {}


def engine(models, name, dtype, max_tokens=2048, **kw):
    from mynah_slm_b200.engine.engine import Engine
    key = (name, dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _ENGINES:
        _ENGINES[key] = Engine.from_folder(models[name][0], dtype=dtype, max_tokens=max_tokens, **kw)
    return _ENGINES[key]


def reference(models, name, toks):
    key = (name, tuple(toks))
    if key not in _PLAIN:
        _PLAIN[key] = plain.forward(models[name][1], models[name][2], toks)
    return _PLAIN[key]


def entry(slot, tokens, want):
    from mynah_slm_b200.engine.engine import StepEntry
    return StepEntry(slot, list(tokens), tuple(want))


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def run_pieces(eng, toks, cuts):
    """One sequence alone, cut at `cuts`; logits of every position."""
    slot = eng.open_sequence()
    rows, lo = [], 0
    for hi in list(cuts) + [len(toks)]:
        if hi > lo:
            rows.append(eng.step([entry(slot, toks[lo:hi], range(hi - lo))]).cpu().numpy())
            lo = hi
    eng.check_status()
    eng.close_sequence(slot)
    return np.concatenate(rows, 0)


# ------------------------------------------------------------------ each mechanism alone, whole prompts
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["parallel", "delta", "moe", "hybrid", "odd", "once", "ragged"])
def test_whole_prompts(models, name, dtype):
    cfg = models[name][1]
    eng = engine(models, name, dtype)
    for n in (1, 2, 3, 7, 64, 65, 150):
        toks = tokens_for(cfg, n, n)
        close(reference(models, name, toks), run_pieces(eng, toks, []), dtype, f"{name} {dtype} whole {n}")


def test_layers_one_by_one(models):
    """The residual stream behind every run of a layer (a looped layer counts each time), 32-bit."""
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", "float32")
    toks = tokens_for(cfg, 90, 5)
    _, ref = plain.forward(cfg, W, toks, return_layers=True)
    slot = eng.open_sequence()
    taps = {}
    eng.step([entry(slot, toks, (0,))], taps=taps)
    eng.close_sequence(slot)
    assert len(ref) == 9
    for i, r in enumerate(ref):
        assert_close(r, taps[f"layer{i}"].cpu().numpy(), FP32_TOL, f"layer run {i}")


# ------------------------------------------------------------------ prefill against decoding, pieces
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["hybrid", "odd", "ragged"])
def test_token_by_token(models, name, dtype):
    cfg = models[name][1]
    eng = engine(models, name, dtype)
    toks = tokens_for(cfg, 75, 11)
    close(reference(models, name, toks), run_pieces(eng, toks, range(1, 75)), dtype, f"{name} {dtype} one by one",
          whole=run_pieces(eng, toks, []))


@pytest.mark.parametrize("dtype", DTYPES)
def test_pieces_of_several_sizes(models, dtype):
    cfg = models["hybrid"][1]
    eng = engine(models, "hybrid", dtype)
    toks = tokens_for(cfg, 200, 12)
    ref = reference(models, "hybrid", toks)
    whole = run_pieces(eng, toks, [])
    for cuts in ([2, 4, 6, 8, 10], [1, 3, 4, 64, 66, 128, 129, 131], [31, 32, 33, 96, 100, 140], [63, 64, 65, 70, 192]):
        close(ref, run_pieces(eng, toks, cuts), dtype, f"{dtype} cuts {cuts}", whole=whole)
    if dtype == "float32":      # pieces and the whole agree far more closely than either with float64
        assert_close(whole, run_pieces(eng, toks, [2, 4, 5, 64, 100, 101, 103]), 2e-5, "whole against pieces")


# ------------------------------------------------------------------ batches
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["hybrid", "odd"])
def test_unequal_batch_then_decode_together(models, name, dtype):
    cfg = models[name][1]
    eng = engine(models, name, dtype)
    lens, extra = [5, 130, 1, 66, 31], [20, 3, 12, 20, 7]
    seqs = [tokens_for(cfg, n + e, 40 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    refs = [reference(models, name, s) for s in seqs]
    wholes = [run_pieces(eng, s, []) for s in seqs]
    slots = [eng.open_sequence() for _ in seqs]
    got = [[] for _ in seqs]
    out = eng.step([entry(s, t[:n], range(n)) for s, t, n in zip(slots, seqs, lens)]).cpu().numpy()
    at = 0
    for i, n in enumerate(lens):
        got[i].append(out[at:at + n])
        at += n
    live = list(range(len(seqs)))
    step = 0
    while live:
        out = eng.step([entry(slots[i], [seqs[i][lens[i] + step]], (0,)) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
        step += 1
        for i in [i for i in live if step >= extra[i]]:       # shorter requests end earlier
            eng.close_sequence(slots[i])
            live.remove(i)
    eng.check_status()
    for i, ref in enumerate(refs):
        close(ref, np.concatenate(got[i], 0), dtype, f"{name} {dtype} request {i}", whole=wholes[i])


def test_batch_equals_alone_in_32_bit(models):
    cfg = models["hybrid"][1]
    eng = engine(models, "hybrid", "float32")
    seqs = [tokens_for(cfg, n, 60 + n) for n in (3, 77, 140)]
    alone = [run_pieces(eng, s, []) for s in seqs]
    slots = [eng.open_sequence() for _ in seqs]
    out = eng.step([entry(s, t, range(len(t))) for s, t in zip(slots, seqs)]).cpu().numpy()
    for s in slots:
        eng.close_sequence(s)
    at = 0
    for a in alone:
        assert_close(a, out[at:at + len(a)], 2e-5, "batched against alone")
        at += len(a)


# ------------------------------------------------------------------ slots and pages used again
@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(models, dtype):
    """Two slots and few pages, four times over: states must start from zero and freed pages must not show."""
    cfg = models["hybrid"][1]
    eng = engine(models, "hybrid", dtype, max_tokens=512, max_seqs=2)
    seen = set()
    for turn in range(4):
        toks_a, toks_b = tokens_for(cfg, 100 + turn, 70 + turn), tokens_for(cfg, 30 + turn, 80 + turn)
        sa, sb = eng.open_sequence(), eng.open_sequence()
        seen.update((sa, sb))
        out = eng.step([entry(sa, toks_a[:90], range(90)), entry(sb, toks_b[:20], range(20))]).cpu().numpy()
        rows_a, rows_b = [out[:90]], [out[90:]]
        for t in range(10):
            out = eng.step([entry(sa, [toks_a[90 + t]], (0,)), entry(sb, [toks_b[20 + t]], (0,))]).cpu().numpy()
            rows_a.append(out[:1])
            rows_b.append(out[1:])
        eng.check_status()
        eng.close_sequence(sa)
        eng.close_sequence(sb)
        close(reference(models, "hybrid", toks_a[:100]), np.concatenate(rows_a, 0), dtype, f"turn {turn} a")
        close(reference(models, "hybrid", toks_b[:30]), np.concatenate(rows_b, 0), dtype, f"turn {turn} b")
    assert len(seen) <= 2


# ------------------------------------------------------------------ windows, page borders, far positions
def test_every_position_with_sharp_attention(models):
    """Sharp attention and no recurrent branch, 32-bit: every position of a prompt that spans several pages and several
    windows, run whole, in pieces around the page borders and the windows' edges, and with its last 150 tokens decoded
    one by one. The controls show that a window one token longer or shorter would be seen at this tolerance."""
    _, cfg, W = models["sharp"]
    eng = engine(models, "sharp", "float32")
    toks = tokens_for(cfg, 420, 21)
    ref = reference(models, "sharp", toks)
    assert_close(ref, run_pieces(eng, toks, []), FP32_TOL, "sharp whole")
    assert_close(ref, run_pieces(eng, toks, range(270, 420)), FP32_TOL, "sharp decoded")
    assert_close(ref, run_pieces(eng, toks, [63, 64, 65, 96, 97, 98, 127, 128, 129, 191, 192, 200, 201, 256, 257, 320]), FP32_TOL,
                 "sharp pieces")
    for delta in (-1, 1):
        other = json.loads(json.dumps(cfg))
        for L in other["layers"]:
            L["mixer"]["left"]["mask"]["size"] += delta
        assert rel_err(ref[250:], plain.forward(other, W, toks)[250:]) > 100 * FP32_TOL, "control: a window one token off goes unseen"


def _standout_model(models, window):
    """One parallel layer in which the query of token 0 finds the key of token 1 and nothing else: token 0's embedding
    lives on coordinates 0..7 and the queries read those, token 1's lives on coordinates 8..15 and the keys read those,
    all other tokens are zero there (their scores are 0), and only dimensions that no rotation reaches get weight. The
    recurrent branch is silent and the input convolution is off. A token 1 placed w positions before a token 0 holds
    that position's whole weight if and only if w < window."""
    import torch
    folder, cfg, _ = models["sharp"]
    cfg = json.loads(json.dumps(cfg))
    cfg["layers"] = cfg["layers"][:1]
    left = cfg["layers"][0]["mixer"]["left"]
    left["mask"]["size"] = window
    left["rot"]["dims"] = 8
    Wt = gm.make_weights(cfg, 77, sharp=True)
    H, dim, D = left["heads"], left["dim"], cfg["width"]
    emb = torch.randn((cfg["vocab"], D), generator=torch.Generator().manual_seed(5), dtype=torch.float64)
    emb[:, :16] = 0.0
    emb[0], emb[1] = 0.0, 0.0
    emb[0, :8], emb[1, 8:16] = 1.0, 1.0
    q = torch.zeros((H, dim, D), dtype=torch.float64)
    k = torch.zeros((H, dim, D), dtype=torch.float64)
    for d in range(8):
        q[:, 8 + d, d] = 1.0
        k[:, 8 + d, 8 + d] = 1.0
    Wt["l0.mix.left.q"] = q.reshape(H * dim, D).to(torch.bfloat16)
    Wt["l0.mix.left.k"] = k.reshape(H * dim, D).to(torch.bfloat16)
    Wt["embed"] = emb.to(torch.bfloat16)
    Wt["l0.canon1"] = torch.zeros_like(Wt["l0.canon1"])
    out = os.path.join(os.path.dirname(folder), f"standout_{window}")
    gm.write_model(out, cfg, Wt)
    return out, cfg, gm.as_numpy(Wt)


@pytest.mark.parametrize("window", [37, 64, 65, 130])
def test_keys_just_inside_and_outside_the_window(models, window):
    """The key that the last position asks for at distance window - 1 (seen) and window (not seen), among random
    others, at several places along the sequence, in a prompt, in pieces and decoded; in both precisions."""
    from mynah_slm_b200.engine.engine import Engine
    folder, cfg, W = _standout_model(models, window)
    rng = np.random.default_rng(window)
    engines = {dtype: Engine.from_folder(folder, dtype=dtype, max_tokens=1024) for dtype in DTYPES}
    for end in (window + 3, 199, 321):
        for dist in (window - 1, window):
            toks = rng.integers(2, cfg["vocab"], size=end + 1).tolist()
            toks[end], toks[end - dist] = 0, 1
            ref = plain.forward(cfg, W, toks)
            moved = list(toks)
            moved[end - dist] = 2
            seen = rel_err(ref[-1:], plain.forward(cfg, W, moved)[-1:]) > 1e-2
            assert seen == (dist < window), "control: the key at the window's edge does not decide the last row"
            for dtype in DTYPES:
                eng = engines[dtype]
                close(ref, run_pieces(eng, toks, []), dtype, f"window {window} end {end} dist {dist} whole")
                close(ref, run_pieces(eng, toks, range(max(end - dist - 2, 1), end + 1)), dtype,
                      f"window {window} end {end} dist {dist} decoded")
                close(ref, run_pieces(eng, toks, [end - dist, end - 1]), dtype, f"window {window} end {end} dist {dist} pieces")


def test_the_sink_takes_its_share(models):
    """The plain implementation without the sink's term differs visibly, so a sink left out would show."""
    _, cfg, W = models["parallel"]
    toks = tokens_for(cfg, 60, 3)
    ref = reference(models, "parallel", toks)
    no_sink = dict(W)
    no_sink["l0.mix.left.sink"] = np.full_like(W["l0.mix.left.sink"], -1e9)
    assert rel_err(ref, plain.forward(cfg, no_sink, toks)) > 1e-2, "control: the sink does not matter"
    assert_close(ref, run_pieces(engine(models, "parallel", "float32"), toks, [1, 2, 30]), FP32_TOL, "sink")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(models, dtype):
    cfg = models["hybrid"][1]
    eng = engine(models, "hybrid", dtype)
    toks = tokens_for(cfg, 330, 31)
    close(reference(models, "hybrid", toks), run_pieces(eng, toks, range(10, 330)), dtype, f"{dtype} long decoding",
          whole=run_pieces(eng, toks, []))


def test_first_tokens(models):
    """Positions 0..5 of several sequences, as prompts of one to six tokens and decoded from the first token on."""
    for name in ("hybrid", "once"):
        cfg = models[name][1]
        eng = engine(models, name, "float32")
        for n in range(1, 7):
            toks = tokens_for(cfg, n, 90 + n)
            ref = reference(models, name, toks)
            assert_close(ref, run_pieces(eng, toks, []), FP32_TOL, f"prompt of {n}")
            assert_close(ref, run_pieces(eng, toks, range(1, n)), FP32_TOL, f"decoded from the first of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["wide", "large"])
def test_other_sizes(models, name, dtype):
    cfg = models[name][1]
    eng = engine(models, name, dtype, max_tokens=1024)
    toks = tokens_for(cfg, 200, 61)
    ref = reference(models, name, toks)
    whole = run_pieces(eng, toks, [])
    close(ref, whole, dtype, f"{name} {dtype} whole")
    close(ref, run_pieces(eng, toks, [3, 5, 64, 89, 90, 91, 150] + list(range(180, 200))), dtype, f"{name} {dtype} pieces",
          whole=whole)


def test_without_graphs_equals_with(models):
    cfg = models["hybrid"][1]
    toks = tokens_for(cfg, 120, 33)
    a = run_pieces(engine(models, "hybrid", "float32"), toks, range(100, 120))
    b = run_pieces(engine(models, "hybrid", "float32", use_graphs=False), toks, range(100, 120))
    assert_close(a, b, 1e-6, "captured steps against launched ones")


def test_random_weights_on_the_device_equal_a_written_folder(tmp_path):
    """`Engine.random` (weights made in place, the narrow sizes chosen by the parts) against the folder
    `write_random_model` writes."""
    import torch
    from mynah_slm_b200.engine.engine import Engine
    from mynah_slm_b200.registry import parse_config
    from mynah_slm_b200.weights.random_init import write_random_model
    cfg = gm.HYBRID
    folder = write_random_model(str(tmp_path / "m"), parse_config(cfg), 3, torch.bfloat16)
    a = Engine.from_folder(folder, dtype="float32", max_tokens=256)
    b = Engine.random(cfg, seed=3, dtype="float32", stored_dtype="bfloat16", max_tokens=256)
    toks = tokens_for(cfg, 50, 1)
    assert np.array_equal(run_pieces(a, toks, [20]), run_pieces(b, toks, [20]))


# ------------------------------------------------------------------ generation through the entry point
@pytest.mark.parametrize("name", ["hybrid", "odd"])
def test_greedy_generation(models, name):
    from mynah_slm_b200 import LLM
    folder, cfg, W = models[name]
    llm = LLM(folder, dtype="float32", max_tokens=1024)
    prompts = [tokens_for(cfg, n, 200 + n) for n in (4, 70, 1, 33, 129)]
    n_new = 24
    results = llm.generate(prompts, max_new=n_new, temp=0.0, ignore_eos=True, max_batch=3)
    for p, r in zip(prompts, results):
        seq = list(p)
        for t in range(n_new):
            logits = plain.forward(cfg, W, seq)[-1]
            top2 = np.sort(logits)[-2:]
            if top2[1] - top2[0] < 1e-3 * max(1.0, abs(top2[1])):
                break                                   # a near tie: either choice is right, stop comparing
            assert r.tokens[t] == int(np.argmax(logits)), f"{name}: token {t} of the prompt of {len(p)}"
            seq.append(r.tokens[t])


def test_command_line_and_trace_runner(models, tmp_path):
    """`mynah-slm run` on a folder (greedy tokens against the plain implementation) and bin/trace_run as a process: a
    batch of two prompts, decoding together, one ends early."""
    import subprocess
    import sys
    folder, cfg, W = models["hybrid"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a, b = tokens_for(cfg, 70, 301), tokens_for(cfg, 9, 302)
    ids = lambda t: ",".join(str(x) for x in t)
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "mynah-slm"), "run", "-m", folder, "--tokens", ids(a[:40]), "-n", "5",
                        "--temp", "0", "--dtype", "float32", "--ignore-eos", "--quiet"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    got = [int(x) for x in p.stdout.split()]
    assert len(got) == 5
    seq = list(a[:40])
    for t in range(5):
        logits = plain.forward(cfg, W, seq)[-1]
        top2 = np.sort(logits)[-2:]
        if top2[1] - top2[0] < 1e-3 * max(1.0, abs(top2[1])):
            break
        assert got[t] == int(np.argmax(logits))
        seq.append(got[t])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]}, {"id": "b", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[67:68], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[68:69], "want": [0]}], "end": ["a"]}]
    out = str(tmp_path / "out")
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out, "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain.forward(cfg, W, a), plain.forward(cfg, W, b)
    read = lambda i: np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
    assert_close(np.stack([ra[0], ra[65], rb[6]]), read(0), FP32_TOL, "step 0")
    assert_close(ra[66:67], read(1), FP32_TOL, "step 1")
    assert_close(np.stack([ra[67], rb[8]]), read(2), FP32_TOL, "step 2")
    assert_close(ra[68:69], read(3), FP32_TOL, "step 3")
