"""The Gomuzen design in the engine against the plain implementation (tests/plain/gomuzen.py).

The tests make their own small configurations and their own weights (tests/gomuzen_models.py): each mechanism alone,
whole prompts against token-by-token decoding, pieces down to two tokens, unequal batches against each request alone,
slots and pages used again, every position across page borders and across the edges of the windows and of the kept
first tokens with sharpened attention (with controls that a window or a kept count one token off, or one lost far key,
would show), the first tokens, long decoding, sizes that are no multiple of 8, constants of 1, one head, one expert,
heads of the tensor-core sizes, and greedy generation through the package's entry point.

Tolerances. 32-bit: ||ref - got|| / ||ref|| of every row of logits within 1e-4. bfloat16: a row's ||ref - got|| is set
against the request's typical row norm (the root mean square of ||ref|| over its rows); the mean over a request's rows
within 5e-2 and every row within 2e-1, and what the schedule changes is held separately against the engine's own whole
run: mean within 2e-2, every row within 1e-1. A wrong edge or a stale page moves rows by their whole size, and the
32-bit runs of the same tests hold every row to 1e-4.
"""
import copy
import json
import os

import numpy as np
import pytest

import gomuzen_models as gm
from helpers import assert_close, rel_err
from plain import gomuzen as plain

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_MEAN_TOL, BF16_ROW_TOL, BF16_SCHEDULE_MEAN_TOL, BF16_SCHEDULE_ROW_TOL = 5e-2, 2e-1, 2e-2, 1e-1
DTYPES = ["float32", "bfloat16"]


CLOSE_CALL = 0.01      # a router's gap between the last chosen and the first left out below which bfloat16 may choose otherwise


def close_calls(cfg, W, toks):
    """Rows at which some routed feed-forward of the plain implementation chose by a narrow gap: a bfloat16 run may
    rightly pick another expert there, which moves the row by more than rounding does."""
    margins = []
    plain.forward(cfg, W, toks, margins=margins)
    return np.min(margins, axis=0) < CLOSE_CALL if margins else np.zeros(len(toks), dtype=bool)


def close(ref, got, dtype, what, whole=None, model=None):
    """`got` against the plain implementation's `ref`; in bfloat16 also against the engine's own whole run. `model`
    = (cfg, W, tokens): in bfloat16, rows that a router chose by a narrow gap are left out of the per-row limit."""
    if dtype == "float32":
        return assert_close(ref, got, FP32_TOL, what)
    ref, got = np.asarray(ref, dtype=np.float64), np.asarray(got, dtype=np.float64)
    assert ref.shape == got.shape and np.all(np.isfinite(got)), what
    scale = max(float(np.sqrt((np.linalg.norm(ref, axis=-1) ** 2).mean())), 1e-30)
    rows = np.linalg.norm(ref - got, axis=-1) / scale
    if model is not None and rows.max() > BF16_ROW_TOL:
        narrow = close_calls(*model)[-len(rows):]
        assert narrow.mean() < 0.5, f"{what}: the test's weights make too many close calls"
        rows = np.where(narrow, 0.0, rows)
    assert rows.mean() <= BF16_MEAN_TOL, f"{what}: mean rel error {rows.mean():.3e}"
    assert rows.max() <= BF16_ROW_TOL, f"{what}: row {int(rows.argmax())} has rel error {rows.max():.3e}"
    if whole is not None:
        rows = np.linalg.norm(np.asarray(whole, dtype=np.float64) - got, axis=-1) / scale
        assert rows.mean() <= BF16_SCHEDULE_MEAN_TOL, f"{what}: mean rel error {rows.mean():.3e} against the whole run"
        assert rows.max() <= BF16_SCHEDULE_ROW_TOL, f"{what}: row {int(rows.argmax())} is {rows.max():.3e} off the whole run"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return gm.write_models(tmp_path_factory.mktemp("gomuzen"))


_ENGINES = {}


def engine(models, name, dtype, max_tokens=2048, **kw):
    from mynah_slm_b200.engine.engine import Engine
    key = (name, dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _ENGINES:
        _ENGINES[key] = Engine.from_folder(models[name][0], dtype=dtype, max_tokens=max_tokens, **kw)
    return _ENGINES[key]


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
@pytest.mark.parametrize("name", ["latent", "diff", "window", "moe", "plain", "hybrid", "odd"])
def test_whole_prompts(models, name, dtype):
    _, cfg, W = models[name]
    eng = engine(models, name, dtype)
    for n in (1, 2, 3, 7, 64, 65, 150):
        toks = tokens_for(cfg, n, n)
        close(plain.forward(cfg, W, toks), run_pieces(eng, toks, []), dtype, f"{name} {dtype} whole {n}", model=(cfg, W, toks))


def test_layers_one_by_one(models):
    """The residual stream behind every run of the schedule (a looped layer counts each time), 32-bit."""
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", "float32")
    toks = tokens_for(cfg, 90, 5)
    ref = []
    plain.forward(cfg, W, toks, layers_out=ref)
    assert len(ref) == 1 + 3 * 3 + 3
    slot = eng.open_sequence()
    taps = {}
    eng.step([entry(slot, toks, (0,))], taps=taps)
    eng.close_sequence(slot)
    for i, r in enumerate(ref):
        assert_close(r, taps[f"layer{i}"].cpu().numpy(), FP32_TOL, f"run {i}")


# ------------------------------------------------------------------ prefill against decoding, pieces
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["hybrid", "odd", "plain"])
def test_token_by_token(models, name, dtype):
    _, cfg, W = models[name]
    eng = engine(models, name, dtype)
    toks = tokens_for(cfg, 90, 11)
    close(plain.forward(cfg, W, toks), run_pieces(eng, toks, range(1, 90)), dtype, f"{name} {dtype} one by one",
          whole=run_pieces(eng, toks, []), model=(cfg, W, toks))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["hybrid", "odd"])
def test_pieces_of_several_sizes(models, name, dtype):
    _, cfg, W = models[name]
    eng = engine(models, name, dtype)
    toks = tokens_for(cfg, 200, 12)
    ref = plain.forward(cfg, W, toks)
    whole = run_pieces(eng, toks, [])
    for cuts in ([2, 4, 6, 8, 10], [1, 3, 4, 64, 66, 128, 129, 131], [31, 32, 33, 96, 100, 140], [63, 64, 65, 70, 192]):
        close(ref, run_pieces(eng, toks, cuts), dtype, f"{dtype} cuts {cuts}", whole=whole, model=(cfg, W, toks))
    if dtype == "float32":      # pieces and the whole agree far more closely than either with float64
        assert_close(whole, run_pieces(eng, toks, [2, 4, 5, 64, 100, 101, 103]), 2e-5, "whole against pieces")


# ------------------------------------------------------------------ batches
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["hybrid", "odd"])
def test_unequal_batch_then_decode_together(models, name, dtype):
    _, cfg, W = models[name]
    eng = engine(models, name, dtype)
    lens, extra = [5, 130, 1, 66, 31], [20, 3, 12, 20, 7]
    seqs = [tokens_for(cfg, n + e, 40 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    refs = [plain.forward(cfg, W, s) for s in seqs]
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
        close(ref, np.concatenate(got[i], 0), dtype, f"{name} {dtype} request {i}", whole=wholes[i], model=(cfg, W, seqs[i]))


def test_batch_equals_alone_in_32_bit(models):
    _, cfg, _ = models["hybrid"]
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
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", dtype, max_tokens=256, max_seqs=2)      # 4 pages, 2 slots
    seen = set()
    for round_ in range(4):
        toks_a, toks_b = tokens_for(cfg, 100 + round_, 70 + round_), tokens_for(cfg, 30 + round_, 80 + round_)
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
        close(plain.forward(cfg, W, toks_a[:100]), np.concatenate(rows_a, 0), dtype, f"round {round_} a", model=(cfg, W, toks_a[:100]))
        close(plain.forward(cfg, W, toks_b[:30]), np.concatenate(rows_b, 0), dtype, f"round {round_} b", model=(cfg, W, toks_b[:30]))
    assert len(seen) <= 2


# ------------------------------------------------------------------ windows, kept first tokens, far keys, page borders
def test_every_position_with_sharp_attention(models):
    """Sharp attention, 32-bit: every position of a prompt that spans several pages, run whole, in pieces around the
    page borders and the windows' edges, and with its last 200 tokens decoded one by one (the windows of 76 and 130
    pass over decoded tokens and over page borders). The controls show that a window one position longer or shorter, a
    kept count one token off, or another key at ONE far place would be seen at this tolerance."""
    _, cfg, W = models["sharp"]
    eng = engine(models, "sharp", "float32")
    toks = tokens_for(cfg, 420, 21)
    ref = plain.forward(cfg, W, toks)
    assert_close(ref, run_pieces(eng, toks, []), FP32_TOL, "sharp whole")
    assert_close(ref, run_pieces(eng, toks, range(220, 420)), FP32_TOL, "sharp decoded")
    assert_close(ref, run_pieces(eng, toks, [9, 10, 11, 63, 64, 65, 75, 76, 77, 85, 86, 127, 128, 129, 130, 131, 191, 192, 193, 194,
                                             256, 257, 320]), FP32_TOL, "sharp pieces")
    for layer, key, by in ((0, "size", 1), (0, "size", -1), (0, "keep_first", 1), (0, "keep_first", -1), (3, "size", 1),
                           (3, "size", -1), (3, "keep_first", 1), (3, "keep_first", -1)):
        other = copy.deepcopy(cfg)
        other["layers"][layer]["mixer"]["mask"][key] += by
        assert rel_err(ref[300:], plain.forward(other, W, toks)[300:]) > 100 * FP32_TOL, f"control: layer {layer} {key} {by:+d} goes unseen"
    moved = [(toks[0] + 1) % cfg["vocab"]] + toks[1:]
    assert rel_err(ref[300:], plain.forward(cfg, W, moved)[300:]) > 100 * FP32_TOL, "control: the first position's key goes unseen"


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_in_decoding_and_in_prompts(models, dtype):
    """One windowed layer alone (window 50, 7 kept first tokens): positions 40 to 140 as the ends of prompts and decoded one
    by one, so that the first position outside the window, the last kept token and the page border are each met both ways."""
    _, cfg, W = models["window"]
    eng = engine(models, "window", dtype)
    toks = tokens_for(cfg, 140, 77)
    ref = plain.forward(cfg, W, toks)
    whole = run_pieces(eng, toks, [])
    close(ref, whole, dtype, f"window {dtype} whole")
    close(ref, run_pieces(eng, toks, range(40, 140)), dtype, f"window {dtype} decoded", whole=whole)
    close(ref, run_pieces(eng, toks, [49, 50, 51, 56, 57, 58, 64, 100, 113, 114, 115]), dtype, f"window {dtype} pieces", whole=whole)
    if dtype == "float32":
        for key, by in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
            other = copy.deepcopy(cfg)
            other["layers"][0]["mixer"]["mask"][key] += by
            assert rel_err(ref[60:], plain.forward(other, W, toks)[60:]) > 100 * FP32_TOL, f"control: {key} {by:+d} goes unseen"


def test_tensor_core_attention_sizes(models):
    """bfloat16 with heads of 64 and 128 and cache rows of 128: whichever attention kernels the dispatch picks, against
    the plain implementation and against the general kernels on the same cache, whole, in pieces and decoded."""
    from mynah_slm_b200.ops import attention_dispatch
    _, cfg, W = models["wide"]
    toks = tokens_for(cfg, 520, 41)
    ref = plain.forward(cfg, W, toks)
    eng = engine(models, "wide", "bfloat16")
    runs = {}
    for use_tc in (True, False):
        attention_dispatch.USE_TC_MASKED = use_tc
        try:
            eng_k = eng if use_tc else engine(models, "wide", "bfloat16", use_graphs=False)
            runs[use_tc] = [run_pieces(eng_k, toks, cuts) for cuts in ([], [99, 100, 101, 128, 150, 200, 201, 300, 399, 400],
                                                                       range(380, 520))]
        finally:
            attention_dispatch.USE_TC_MASKED = True
    for got_tc, got_general in zip(runs[True], runs[False]):
        close(ref, got_tc, "bfloat16", "tensor-core attention", whole=got_general, model=(cfg, W, toks))
        close(ref, got_general, "bfloat16", "general attention", model=(cfg, W, toks))
    close(ref, run_pieces(engine(models, "wide", "float32"), toks, [150, 151, 400]), "float32", "wide in 32-bit")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(models, dtype):
    _, cfg, W = models["hybrid"]
    eng = engine(models, "hybrid", dtype)
    toks = tokens_for(cfg, 330, 31)
    close(plain.forward(cfg, W, toks), run_pieces(eng, toks, range(10, 330)), dtype, f"{dtype} long decoding",
          whole=run_pieces(eng, toks, []), model=(cfg, W, toks))


def test_first_tokens(models):
    """Positions 0..5 of several sequences, as prompts of one to six tokens and decoded from the first token on."""
    for name in ("hybrid", "odd"):
        _, cfg, W = models[name]
        eng = engine(models, name, "float32")
        for n in range(1, 7):
            toks = tokens_for(cfg, n, 90 + n)
            ref = plain.forward(cfg, W, toks)
            assert_close(ref, run_pieces(eng, toks, []), FP32_TOL, f"{name}: prompt of {n}")
            assert_close(ref, run_pieces(eng, toks, range(1, n)), FP32_TOL, f"{name}: decoded from the first of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_large_sizes(models, dtype):
    _, cfg, W = models["large"]
    eng = engine(models, "large", dtype, max_tokens=1024)
    toks = tokens_for(cfg, 200, 61)
    ref = plain.forward(cfg, W, toks)
    whole = run_pieces(eng, toks, [])
    close(ref, whole, dtype, f"large {dtype} whole", model=(cfg, W, toks))
    close(ref, run_pieces(eng, toks, [3, 5, 64, 89, 90, 91, 150] + list(range(180, 200))), dtype, f"large {dtype} pieces",
          whole=whole, model=(cfg, W, toks))


def test_without_graphs_equals_with(models):
    _, cfg, _ = models["hybrid"]
    toks = tokens_for(cfg, 120, 33)
    a = run_pieces(engine(models, "hybrid", "float32"), toks, range(100, 120))
    b = run_pieces(engine(models, "hybrid", "float32", use_graphs=False), toks, range(100, 120))
    assert_close(a, b, 1e-6, "captured steps against launched ones")


def test_a_window_alone_gives_pages_back(models):
    """A windowed layer without kept first tokens frees the pages behind its window: a long sequence, run piece by
    piece and token by token, never holds more pages than its window and a piece span, and equals the plain
    implementation. A window that keeps first tokens holds every page."""
    _, cfg, W = models["slide"]
    eng = engine(models, "slide", "float32")
    assert [g.window for g in eng.cache.plan.groups] == [70]
    toks = tokens_for(cfg, 1000, 19)
    slot = eng.open_sequence()
    rows, lo, most = [], 0, 0
    for hi in list(range(50, 900, 50)) + list(range(900, 1001)):
        rows.append(eng.step([entry(slot, toks[lo:hi], range(hi - lo))]).cpu().numpy())
        most = max(most, eng.cache.pages.n_held(slot, 0))
        lo = hi
    eng.check_status()
    eng.close_sequence(slot)
    assert most <= 3, f"the sequence held {most} pages at once"
    assert_close(plain.forward(cfg, W, toks), np.concatenate(rows, 0), FP32_TOL, "a long sequence under a window")
    assert not any(g.window == 40 for g in engine(models, "hybrid", "float32").cache.plan.groups)


def test_random_weights_on_the_device_equal_a_written_folder(tmp_path):
    """`Engine.random` (weights made in place) against the folder `write_random_model` writes."""
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


def test_command_line(models, tmp_path):
    """`mynah-slm run` on a folder: greedy tokens against the plain implementation, the prompts' logits written beside."""
    import subprocess
    import sys
    folder, cfg, W = models["plain"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli = [sys.executable, os.path.join(root, "bin", "mynah-slm")]
    a, b = tokens_for(cfg, 40, 401), tokens_for(cfg, 3, 402)
    ids = lambda t: ",".join(str(x) for x in t)
    npy = tmp_path / "logits.npy"
    p = subprocess.run(cli + ["run", "-m", folder, "--tokens", ids(a), "--tokens", ids(b), "-n", "5", "--temp", "0", "--dtype", "float32",
                              "--ignore-eos", "--quiet", "--logits-out", str(npy)], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [[int(x) for x in l.split()] for l in p.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(l) == 5 for l in lines)
    assert_close(np.concatenate([plain.forward(cfg, W, a), plain.forward(cfg, W, b)]), np.load(npy), FP32_TOL, "--logits-out")


def test_trace_runner_process(models, tmp_path):
    """bin/trace_run as a process: a batch of two prompts, decoding together, one ends early."""
    import subprocess
    import sys
    folder, cfg, W = models["hybrid"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a, b = tokens_for(cfg, 70, 301), tokens_for(cfg, 9, 302)
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


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_looped_latent_layer_decodes_with_a_cache_a_pass(models, dtype):
    """One latent layer run twice: each pass keeps latent rows of its own, and decoding reads both."""
    _, cfg, W = models["latent"]
    eng = engine(models, "latent", dtype)
    assert len(eng.cache.plan.groups) == 1 and len(eng.cache.plan.groups[0].entries) == 2
    toks = tokens_for(cfg, 150, 5)
    close(plain.forward(cfg, W, toks), run_pieces(eng, toks, [3, 70] + list(range(100, 150))), dtype, f"looped latent {dtype}",
          whole=run_pieces(eng, toks, []))
