"""The mechanisms of the Gupizen design, each alone as a part on the device, against the plain functions of
tests/plain/gupizen.py (float64): rotation frequencies scaled by wavelength, the windowed attention with a sink, mixed
heads and rotated values (whole, in pieces over scrambled pages, a window longer than the kernel's chunk of keys,
grouped heads, odd sizes), the gated linear recurrent unit (pieces, two sequences with padding rows, states in other
slots), the delta rule with a decay per key channel, the learned router with its experts, and the mean of two normed
branches."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import gupizen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(v):
    return torch.tensor(np.asarray(v), dtype=torch.int32, device=DEV)


def rel(ref, got):
    ref, got = np.asarray(ref, dtype=np.float64), np.asarray(got, dtype=np.float64)
    return float(np.abs(ref - got).max() / max(np.abs(ref).max(), 1e-30))


def ctx_for(q_lens, slots, starts=None, pad_rows=0, page_lists=None, n_pages=0, bases=None, decode_splits=1):
    """The fields of a step's context that the parts read: rows packed sequence by sequence, then padding rows."""
    from mynah_slm_b200.ops.kernels import PageTableView
    starts = starts or [0] * len(q_lens)
    tok_seq, tok_pos, cu = [], [], [0]
    for b, (n, s) in enumerate(zip(q_lens, starts)):
        tok_seq += [b] * n
        tok_pos += list(range(s, s + n))
        cu.append(cu[-1] + n)
    tok_seq += [-1] * pad_rows
    tok_pos += [0] * pad_rows
    pages = []
    if page_lists is not None:
        indptr = np.cumsum([0] + [len(p) for p in page_lists])
        pages = [PageTableView(i32(indptr), i32([p for l in page_lists for p in l]), i32(bases or [0] * len(q_lens)), n_pages)]
    return SimpleNamespace(tok_seq=i32(tok_seq), tok_pos=i32(tok_pos), cu_q=i32(cu), slots=i32(slots), B=len(q_lens),
                           kv_len=i32([s + n for n, s in zip(q_lens, starts)]), decode_splits=decode_splits,
                           T=len(tok_seq), status=torch.zeros((1,), dtype=torch.int32, device=DEV), pages=pages,
                           is_decode=all(n == 1 for n in q_lens) and pad_rows == 0, max_q_len=max(q_lens))


def runtime(dtype=torch.float32, max_positions=2048):
    from mynah_slm_b200.engine.engine import Runtime
    return Runtime(torch.device(DEV), dtype, max_positions)


def bound(family, spec, W, dtype=torch.float32, **kw):
    """The part built from `spec` and bound to the float64 arrays of W (by the part's own tensor names)."""
    from mynah_slm_b200.parts import build_part
    part = build_part(family, spec)
    tensors = {ts.name: torch.tensor(W[ts.name], dtype=torch.float32).to(dtype if ts.role != "table" else torch.int32).to(DEV)
               for ts in part.tensor_specs()}
    part.bind(tensors, runtime(dtype, **kw))
    return part


def rows(a, dtype=torch.float32, pad=0):
    t = torch.tensor(np.asarray(a), dtype=torch.float32).to(dtype).to(DEV)
    if pad:
        t = torch.cat([t, torch.zeros((pad, t.shape[1]), dtype=dtype, device=DEV)], 0)
    return t.contiguous()


@pytest.mark.parametrize("dims,base,scaling", [(16, 5000.0, (4.0, 1.0, 4.0, 64)), (6, 20.0, None), (64, 10000.0, (8.0, 1.0, 4.0, 512)),
                                               (10, 33.0, (3.0, 2.0, 5.0, 40))])
def test_frequencies_scaled_by_wavelength(dims, base, scaling):
    from mynah_slm_b200.ops import kernels
    from mynah_slm_b200.parts.position import rotary_frequencies
    sc = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
    f, mult = rotary_frequencies(dims, base, dict(sc, kind="wavelength") if sc else None)
    ref = plain.rotary_freqs(dims, base, sc)
    assert mult == 1.0 and np.allclose(f, ref, rtol=1e-14)
    if sc:      # all three bands of the scaling occur in at least one of the cases
        plain_f = plain.rotary_freqs(dims, base, None)
        kinds = {("kept" if a == b else "divided" if np.isclose(a, b / sc["factor"]) else "blended") for a, b in zip(ref, plain_f)}
        assert len(kinds) >= 2
    cos, sin = kernels.rope_table_freqs(1000, f, mult, DEV)
    ang = np.arange(1000)[:, None] * ref[None, :]
    assert np.abs(cos.cpu().numpy() - np.cos(ang)).max() < 1e-6 and np.abs(sin.cpu().numpy() - np.sin(ang)).max() < 1e-6


def _attention_case(H, G, dim, vd, window, rot_dims, D, seed, scaling=None):
    from mynah_slm_b200.config.spec import PartSpec
    rng = np.random.default_rng(seed)
    rot = {"dims": rot_dims, "base": 300.0}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vd, "scale": 1.3 / np.sqrt(dim), "mask": {"size": window}, "rot": rot}
    W = {"q": rng.normal(size=(H * dim, D)) / np.sqrt(D) * 2, "k": rng.normal(size=(G * dim, D)) / np.sqrt(D) * 2,
         "v": rng.normal(size=(G * vd, D)) / np.sqrt(D), "o": rng.normal(size=(D, H * vd)) / np.sqrt(H * vd),
         "talk": 0.6 * np.eye(H) + 0.4 * rng.normal(size=(H, H)), "sink": rng.normal(size=(H,))}
    W = {k: torch.tensor(v).to(torch.bfloat16).to(torch.float64).numpy() for k, v in W.items()}
    spec = PartSpec("sink_talk_attention", {
        "hidden_size": D, "heads": H, "kv_heads": G, "dim": dim, "vdim": vd, "scale": m["scale"], "window": window,
        "rot": {"dims": rot_dims, "base": 300.0, "pairing": "interleaved",
                "scaling": dict(rot["scaling"], kind="wavelength") if scaling else None},
        "value_rot": {"dims": vd, "base": 300.0, "pairing": "interleaved", "scaling": None},
        **{k: k for k in ("q", "k", "v", "o", "talk", "sink")}})
    return m, W, spec


@pytest.mark.parametrize("H,G,dim,vd,window,rot_dims", [(4, 2, 16, 24, 40, 8), (1, 1, 6, 10, 1, 6), (3, 1, 14, 10, 64, 10), (6, 6, 8, 16, 65, 4),
                                                        (2, 1, 256, 200, 150, 64), (5, 5, 12, 6, 1000, 12)])
def test_sink_attention_part(H, G, dim, vd, window, rot_dims):
    """A prompt of 150 tokens whole, then the same in three pieces (the middle one of two tokens) over pages in
    another order, then 30 more tokens one by one; fp32."""
    from mynah_slm_b200.parts import CacheView
    D, T = 40, 180
    m, W, spec = _attention_case(H, G, dim, vd, window, rot_dims, D, seed=H * 10 + G, scaling=(4.0, 1.0, 4.0, 64))
    part = bound("mixer", spec, W)
    h = np.random.default_rng(1).normal(size=(T, D))
    ref = plain.sink_talk_attention(h, W, m, np.arange(T))
    n_pages = 8
    for pages, cuts in (([0, 1, 2], [0, 150]), ([5, 2, 7], [0, 64, 66, 150])):
        kc = torch.full((n_pages, G, 64, dim), 9.0, device=DEV)
        vc = torch.full((n_pages, G, 64, vd), 9.0, device=DEV)
        cache = CacheView(group=0, k=kc, v=vc, writes=True)
        got = []
        for lo, hi in list(zip(cuts[:-1], cuts[1:])) + [(t, t + 1) for t in range(150, T)]:
            ctx = ctx_for([hi - lo], [0], starts=[lo], pad_rows=1 if hi - lo > 1 else 0, page_lists=[pages], n_pages=n_pages)
            out = part.forward(rows(h[lo:hi], pad=1 if hi - lo > 1 else 0), ctx, cache)
            assert int(ctx.status.item()) == 0
            got.append(out[:hi - lo].cpu().numpy())
        assert rel(ref, np.concatenate(got, 0)) < 2e-5, (pages, cuts)


def test_sink_attention_window_longer_than_a_chunk_of_keys():
    """Sixteen heads of 128 leave the kernel room for about 1,100 keys at a time; a window of 1,400 makes it walk the
    keys in two chunks (scores formed twice). Two sequences in one step, the second one short."""
    from mynah_slm_b200.parts import CacheView
    H, G, dim, vd, window, D = 16, 4, 128, 128, 1400, 32
    m, W, spec = _attention_case(H, G, dim, vd, window, 32, D, seed=3)
    part = bound("mixer", spec, W, max_positions=2048)
    T1, T2 = 1500, 70
    rng = np.random.default_rng(2)
    h1, h2 = rng.normal(size=(T1, D)), rng.normal(size=(T2, D))
    n_pages = 32
    cache = CacheView(group=0, k=torch.zeros((n_pages, G, 64, dim), device=DEV), v=torch.zeros((n_pages, G, 64, vd), device=DEV), writes=True)
    ctx = ctx_for([T1, T2], [0, 1], page_lists=[list(range(24)), [30, 29]], n_pages=n_pages)
    out = part.forward(rows(np.concatenate([h1, h2], 0)), ctx, cache).cpu().numpy()
    assert int(ctx.status.item()) == 0
    sel = list(range(0, 40)) + list(range(1380, 1500))       # the plain loop is slow: the first rows and those past the window
    ref1 = plain.sink_talk_attention(h1, W, m, np.arange(T1))
    assert rel(ref1[sel], out[:T1][sel]) < 2e-5
    assert rel(plain.sink_talk_attention(h2, W, m, np.arange(T2)), out[T1:]) < 2e-5


def test_sink_attention_in_bfloat16():
    from mynah_slm_b200.parts import CacheView
    H, G, dim, vd, window, D, T = 4, 2, 32, 16, 50, 64, 130
    m, W, spec = _attention_case(H, G, dim, vd, window, 16, D, seed=9)
    part = bound("mixer", spec, W, dtype=torch.bfloat16)
    h = torch.tensor(np.random.default_rng(4).normal(size=(T, D))).to(torch.bfloat16)
    ref = plain.sink_talk_attention(h.to(torch.float64).numpy(), W, m, np.arange(T))
    cache = CacheView(group=0, k=torch.zeros((4, G, 64, dim), dtype=torch.bfloat16, device=DEV),
                      v=torch.zeros((4, G, 64, vd), dtype=torch.bfloat16, device=DEV), writes=True)
    ctx = ctx_for([T], [0], page_lists=[[3, 0, 1]], n_pages=4)
    out = part.forward(h.to(DEV), ctx, cache).cpu().numpy()
    assert rel(ref, out) < 3e-2


@pytest.mark.parametrize("H,G,dim,vd,window,splits", [(4, 2, 64, 128, 40, 3), (16, 8, 128, 128, 100, 2), (3, 3, 128, 64, None, 5),
                                                       (20, 5, 64, 64, 65, 1), (2, 1, 128, 128, 32, 4)])
def test_sink_attention_on_tensor_cores(monkeypatch, H, G, dim, vd, window, splits):
    """bfloat16 with heads of 64 or 128 takes the tensor-core kernels: two unequal prompts in one step (with padding
    rows), a portion of two tokens each, then twenty tokens one by one with the keys in `splits` shares, over pages
    in no order. Against the general kernel on the same rows (they differ by the output's rounding at most) and
    against the plain implementation."""
    from mynah_slm_b200.ops import kernels
    from mynah_slm_b200.parts import CacheView
    D, LA, LB, ND = 48, 150, 37, 20
    m, W, spec = _attention_case(H, G, dim, vd, window or 4096, 32, D, seed=H + dim)
    if window is None:
        spec = type(spec)(spec.kind, {**dict(spec.params), "window": None})
    hA = torch.tensor(np.random.default_rng(5).normal(size=(LA + 2 + ND, D))).to(torch.bfloat16)
    hB = torch.tensor(np.random.default_rng(6).normal(size=(LB + 2 + ND, D))).to(torch.bfloat16)
    steps = [((0, LA), (0, LB), 2), ((LA, LA + 2), (LB, LB + 2), 0)] + [((LA + 2 + i, LA + 3 + i), (LB + 2 + i, LB + 3 + i), 0) for i in range(ND)]
    used = []

    def run(tc):
        if not tc:
            monkeypatch.setattr(kernels, "sink_attn_tc_supported", lambda *a: False)
        else:
            real = kernels.sink_attn_tc
            monkeypatch.setattr(kernels, "sink_attn_tc", lambda *a, **k: (used.append(1), real(*a, **k))[1])
        part = bound("mixer", spec, W, dtype=torch.bfloat16)
        cache = CacheView(group=0, k=torch.full((9, G, 64, dim), 3.0, dtype=torch.bfloat16, device=DEV),
                          v=torch.full((9, G, 64, vd), 3.0, dtype=torch.bfloat16, device=DEV), writes=True)
        outA, outB = [], []
        for (a0, a1), (b0, b1), pad in steps:
            ctx = ctx_for([a1 - a0, b1 - b0], [0, 1], starts=[a0, b0], pad_rows=pad, page_lists=[[7, 2, 5], [8, 0]], n_pages=9,
                          decode_splits=splits)
            x = torch.cat([hA[a0:a1], hB[b0:b1], torch.zeros((pad, D), dtype=torch.bfloat16)], 0).to(DEV).contiguous()
            out = part.forward(x, ctx, cache).float().cpu().numpy()
            assert int(ctx.status.item()) == 0
            outA.append(out[:a1 - a0])
            outB.append(out[a1 - a0:a1 - a0 + b1 - b0])
        monkeypatch.undo()
        return np.concatenate(outA, 0), np.concatenate(outB, 0)

    tcA, tcB = run(True)
    assert len(used) == len(steps)
    gA, gB = run(False)
    assert rel(gA, tcA) < 6e-3 and rel(gB, tcB) < 6e-3
    mm = dict(m, mask={"size": window or 10 ** 6})
    assert rel(plain.sink_talk_attention(hA.to(torch.float64).numpy(), W, mm, np.arange(len(hA))), tcA) < 3e-2
    assert rel(plain.sink_talk_attention(hB.to(torch.float64).numpy(), W, mm, np.arange(len(hB))), tcB) < 3e-2


@pytest.mark.parametrize("window,star", [(70, 60), (64, 64), (33, 127), (200, 3)])
def test_tensor_core_attention_sees_a_key_up_to_the_window_edge_and_not_beyond(window, star):
    """One key stands out (its score is 40 above the others'): every query that sees it returns that key's value,
    mixed over the heads; the query one position beyond the window does not. In a prompt, and with single queries
    whose keys are cut in shares, at page borders; the general kernel on the same rows says the same."""
    from mynah_slm_b200.ops import kernels
    H, G, dim, vd, T = 4, 2, 64, 64, 330
    rng = np.random.default_rng(window)
    bf = lambda a: torch.tensor(a, dtype=torch.float32).to(torch.bfloat16).to(DEV).contiguous()
    q = np.zeros((T, H, dim))
    q[:, :, 5] = 8.0
    k = 0.05 * rng.normal(size=(T, G, dim))
    k[star, :, 5] = 5.0                                             # 8 * 5 * scale(1.0) = 40
    v = rng.normal(size=(T, G, vd))
    talk = 0.5 * np.eye(H) + 0.3 * rng.normal(size=(H, H))
    talk = torch.tensor(talk).to(torch.bfloat16).to(torch.float64).numpy()
    n_pages = (T + 63) // 64
    pages = list(rng.permutation(n_pages))
    kc = torch.zeros((n_pages, G, 64, dim), dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros((n_pages, G, 64, vd), dtype=torch.bfloat16, device=DEV)
    for t in range(T):
        kc[pages[t // 64], :, t % 64] = bf(k[t])
        vc[pages[t // 64], :, t % 64] = bf(v[t])
    v_star = vc[pages[star // 64], :, star % 64].float().cpu().numpy()                  # [G, vd]
    want = np.stack([talk[h].sum() * v_star[h // (H // G)] for h in range(H)]).reshape(-1)
    cos_v = torch.ones((T, vd // 2), device=DEV)
    sin_v = torch.zeros((T, vd // 2), device=DEV)
    tk, sk = bf(talk), bf(np.full((H,), -30.0))
    last_in, first_out = min(star + window - 1, T - 1), star + window

    def both(ctx, rows_q, splits):
        outs = []
        for tc in (True, False):
            out = torch.zeros((rows_q.shape[0], H * vd), dtype=torch.bfloat16, device=DEV)
            if tc:
                scratch = torch.empty((kernels.sink_attn_tc_scratch(rows_q.shape[0], H, vd, splits),), dtype=torch.float32, device=DEV)
                kernels.sink_attn_tc(rows_q, out, scratch, kc, vc, tk, sk, cos_v, sin_v, ctx, ctx.pages[0], H, G, dim, vd, window, 1.0, True, splits)
            else:
                kernels.sink_attn(rows_q, out, kc, vc, tk, sk, cos_v, sin_v, ctx, ctx.pages[0], H, G, dim, vd, window, 1.0, True)
            assert int(ctx.status.item()) == 0
            outs.append(out.float().cpu().numpy())
        assert rel(outs[1], outs[0]) < 6e-3
        return outs[0]

    whole = both(ctx_for([T], [0], page_lists=[pages], n_pages=n_pages), bf(q.reshape(T, -1)), 1)
    for i in range(star, last_in + 1):
        assert rel(want, whole[i]) < 2e-2, i
    for i in [star - 1] * (star > 0) + [first_out] * (first_out < T):
        assert rel(want, whole[i]) > 0.3, i
    for i in [last_in] + [first_out] * (first_out < T):
        one = both(ctx_for([1], [0], starts=[i], page_lists=[pages], n_pages=n_pages, decode_splits=3), bf(q[i].reshape(1, -1)), 3)
        assert (rel(want, one[0]) < 2e-2) == (i == last_in), i


def _states(req, n_slots):
    return {k: torch.zeros((n_slots + 1, *r.shape), dtype=r.dtype, device=DEV) for k, r in req.items()}


@pytest.mark.parametrize("width,blocks,taps", [(48, 3, 4), (13, 1, 1), (21, 7, 2), (128, 2, 4), (320, 5, 3)])
def test_recurrent_unit_part(width, blocks, taps):
    """Two sequences of unequal length in one step with a padding row, then each carried on (one in two further pieces,
    the other token by token) from states that sit in other slots than the rows' order suggests; fp32."""
    from mynah_slm_b200.config.spec import PartSpec
    from mynah_slm_b200.parts import CacheView
    D = 40
    rng = np.random.default_rng(width)
    bw = width // blocks
    W = {"y": rng.normal(size=(width, D)) / np.sqrt(D), "y.b": 0.3 * rng.normal(size=width), "x": rng.normal(size=(width, D)) / np.sqrt(D),
         "x.b": 0.3 * rng.normal(size=width), "conv": 0.4 * rng.normal(size=(width, taps)), "conv.b": 0.2 * rng.normal(size=width),
         "ra": rng.normal(size=(blocks, bw, bw)) / np.sqrt(bw), "ra.b": 0.3 * rng.normal(size=(blocks, bw)),
         "ri": rng.normal(size=(blocks, bw, bw)) / np.sqrt(bw), "ri.b": 0.3 * rng.normal(size=(blocks, bw)),
         "lam": -2.5 + 1.5 * rng.normal(size=width), "o": rng.normal(size=(D, width)) / np.sqrt(width)}
    names = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv_name": "conv", "conv_bias": "conv.b", "ra": "ra",
             "ra_bias": "ra.b", "ri": "ri", "ri_bias": "ri.b", "lam": "lam", "o": "o"}
    part = bound("mixer", PartSpec("rglru", {"hidden_size": D, "width": width, "blocks": blocks, "conv": taps, "decay_scale": 8.0, **names}), W)
    m = {"width": width, "blocks": blocks, "conv": taps}
    ha, hb = rng.normal(size=(150, D)), rng.normal(size=(40, D))
    ref_a, ref_b = plain.rglru(ha, W, m), plain.rglru(hb, W, m)
    cache = CacheView(state=_states(part.state_request(), 4))
    out = part.forward(rows(np.concatenate([ha[:90], hb[:7]], 0), pad=1), ctx_for([90, 7], [3, 1], pad_rows=1), cache).cpu().numpy()
    got_a, got_b = [out[:90]], [out[90:97]]
    out = part.forward(rows(np.concatenate([hb[7:8], ha[90:92]], 0)), ctx_for([1, 2], [1, 3], starts=[7, 90]), cache).cpu().numpy()
    got_b.append(out[:1])
    got_a.append(out[1:3])
    for t in range(8, 40):
        got_b.append(part.forward(rows(hb[t:t + 1]), ctx_for([1], [1], starts=[t]), cache).cpu().numpy())
    got_a.append(part.forward(rows(ha[92:]), ctx_for([58], [3], starts=[92]), cache).cpu().numpy())
    assert rel(ref_a, np.concatenate(got_a, 0)) < 2e-5 and rel(ref_b, np.concatenate(got_b, 0)) < 2e-5
    assert float(cache.state["S"][0].abs().max()) == 0.0 and float(cache.state["S"][2].abs().max()) == 0.0


def test_recurrent_unit_cuts_long_sequences_into_pieces():
    """A sequence of 128 rows or more is scanned in 32 pieces that are joined through the linear recurrence: 301 rows
    beside a short sequence (which goes the ordinary way), then 130 more rows onto the state that was left."""
    from mynah_slm_b200.config.spec import PartSpec
    from mynah_slm_b200.parts import CacheView
    D, width, blocks, taps = 24, 40, 2, 3
    rng = np.random.default_rng(77)
    bw = width // blocks
    W = {"y": rng.normal(size=(width, D)) / np.sqrt(D), "y.b": 0.3 * rng.normal(size=width), "x": rng.normal(size=(width, D)) / np.sqrt(D),
         "x.b": 0.3 * rng.normal(size=width), "conv": 0.4 * rng.normal(size=(width, taps)), "conv.b": 0.2 * rng.normal(size=width),
         "ra": rng.normal(size=(blocks, bw, bw)) / np.sqrt(bw), "ra.b": 0.3 * rng.normal(size=(blocks, bw)),
         "ri": rng.normal(size=(blocks, bw, bw)) / np.sqrt(bw), "ri.b": 0.3 * rng.normal(size=(blocks, bw)),
         "lam": -4.0 + 1.5 * rng.normal(size=width), "o": rng.normal(size=(D, width)) / np.sqrt(width)}     # slow decays: far rows count
    names = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv_name": "conv", "conv_bias": "conv.b", "ra": "ra",
             "ra_bias": "ra.b", "ri": "ri", "ri_bias": "ri.b", "lam": "lam", "o": "o"}
    part = bound("mixer", PartSpec("rglru", {"hidden_size": D, "width": width, "blocks": blocks, "conv": taps, "decay_scale": 8.0, **names}), W)
    m = {"width": width, "blocks": blocks, "conv": taps}
    ha, hb = rng.normal(size=(431, D)), rng.normal(size=(50, D))
    ref_a, ref_b = plain.rglru(ha, W, m), plain.rglru(hb, W, m)
    cache = CacheView(state=_states(part.state_request(), 3))
    out = part.forward(rows(np.concatenate([hb, ha[:301]], 0)), ctx_for([50, 301], [2, 0]), cache).cpu().numpy()
    more = part.forward(rows(ha[301:]), ctx_for([130], [0], starts=[301]), cache).cpu().numpy()
    assert rel(ref_b, out[:50]) < 2e-5
    assert rel(ref_a, np.concatenate([out[50:], more], 0)) < 2e-5


def test_recurrent_unit_keeps_what_it_is_told_to():
    """A decay parameter far below zero keeps the state for hundreds of tokens: the first token still shows at the end
    (control), and the part carries it there whole and token by token."""
    from mynah_slm_b200.config.spec import PartSpec
    from mynah_slm_b200.parts import CacheView
    D, width = 16, 8
    rng = np.random.default_rng(0)
    W = {"y": rng.normal(size=(width, D)), "y.b": np.zeros(width), "x": rng.normal(size=(width, D)), "x.b": np.zeros(width),
         "conv": np.ones((width, 1)), "conv.b": np.zeros(width), "ra": np.zeros((1, width, width)), "ra.b": np.zeros((1, width)),
         "ri": np.zeros((1, width, width)), "ri.b": np.full((1, width), 3.0), "lam": np.full(width, -9.0), "o": np.eye(D, width)}
    names = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv_name": "conv", "conv_bias": "conv.b", "ra": "ra",
             "ra_bias": "ra.b", "ri": "ri", "ri_bias": "ri.b", "lam": "lam", "o": "o"}
    part = bound("mixer", PartSpec("rglru", {"hidden_size": D, "width": width, "blocks": 1, "conv": 1, "decay_scale": 8.0, **names}), W)
    m = {"width": width, "blocks": 1, "conv": 1}
    h = 0.01 * rng.normal(size=(600, D))
    h[0] = 5.0 * rng.normal(size=D)
    ref = plain.rglru(h, W, m)
    other = h.copy()
    other[0] = 0.0
    assert rel(ref[-1:], plain.rglru(other, W, m)[-1:]) > 0.3, "control: the first token is forgotten"
    cache = CacheView(state=_states(part.state_request(), 1))
    assert rel(ref, part.forward(rows(h), ctx_for([600], [0]), cache).cpu().numpy()) < 2e-5
    cache = CacheView(state=_states(part.state_request(), 1))
    got = [part.forward(rows(h[:300]), ctx_for([300], [0]), cache).cpu().numpy()]
    got += [part.forward(rows(h[t:t + 1]), ctx_for([1], [0], starts=[t]), cache).cpu().numpy() for t in range(300, 600)]
    assert rel(ref, np.concatenate(got, 0)) < 2e-5


@pytest.mark.parametrize("H,G,dim,vd,taps,ra,rg", [(4, 2, 16, 8, 3, 12, 10), (3, 1, 10, 6, 1, 5, 7), (2, 2, 24, 12, 4, 8, 16), (2, 1, 300, 20, 4, 24, 24),
                                                   (8, 4, 64, 32, 4, 16, 16)])
def test_channel_delta_part(H, G, dim, vd, taps, ra, rg):
    """The delta rule with one decay a head and key channel, the narrow sizes read off the tensors: whole, then in
    pieces (one of two tokens), then token by token; fp32."""
    from mynah_slm_b200.config.spec import PartSpec
    from mynah_slm_b200.parts import CacheView
    D, T = 40, 120
    rng = np.random.default_rng(H * 7 + dim)
    lin = lambda o, i: rng.normal(size=(o, i)) / np.sqrt(i)
    W = {"q": lin(G * dim, D), "k": lin(G * dim, D), "v": lin(H * vd, D), "q.conv": 0.4 * rng.normal(size=(G * dim, taps)),
         "k.conv": 0.4 * rng.normal(size=(G * dim, taps)), "v.conv": 0.4 * rng.normal(size=(H * vd, taps)), "b": lin(H, D),
         "A_log": -1.0 + 0.7 * rng.normal(size=H), "dt_bias": 0.5 * rng.normal(size=H * dim), "a1": lin(ra, D), "a2": lin(H * dim, ra),
         "g1": lin(rg, D), "g2": lin(H * vd, rg), "norm": 1.0 + 0.1 * rng.normal(size=vd), "o": lin(D, H * vd)}
    names = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b", "a": "a2", "a_in": "a1",
             "A_log": "A_log", "dt_bias": "dt_bias", "g": "g2", "g_in": "g1", "norm": "norm", "o": "o"}
    part = bound("mixer", PartSpec("gated_delta", {"hidden_size": D, "heads": H, "kv_heads": G, "dim": dim, "vdim": vd, "conv": taps, "eps": 1e-5,
                                                   "decay": "channel", "gate_act": "sigmoid", **names}), W)
    m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vd, "conv": taps}
    h = rng.normal(size=(T, D))
    ref = plain.channel_delta(h, W, m, 1e-5)
    for cuts in ([0, T], [0, 64, 66, 100] + list(range(101, T + 1))):
        cache = CacheView(state=_states(part.state_request(), 2))
        got = [part.forward(rows(h[lo:hi]), ctx_for([hi - lo], [1], starts=[lo]), cache).cpu().numpy() for lo, hi in zip(cuts[:-1], cuts[1:])]
        assert rel(ref, np.concatenate(got, 0)) < 5e-5, cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,F,E,top", [(70, 40, 12, 1, 1), (150, 48, 56, 9, 2), (1, 52, 18, 3, 2), (33, 40, 20, 7, 7), (300, 256, 128, 8, 2),
                                         (700, 128, 64, 16, 4)])
def test_router_experts_part(dtype, T, D, F, E, top):
    """The inputs and the weights are values that bfloat16 holds, so the router's logits are the same in both
    precisions up to the order of the sums; in bfloat16 the rows whose last chosen and first unchosen logits lie within
    a thousandth of the logits' spread are left out of the comparison all the same."""
    from mynah_slm_b200.config.spec import PartSpec
    rng = np.random.default_rng(T + E)
    W = {"router": 2.0 * rng.normal(size=(E, D)) / np.sqrt(D), "router.b": 0.3 * rng.normal(size=E)}
    for e in range(E):
        W[f"e{e}.up"], W[f"e{e}.down"] = rng.normal(size=(F, D)) / np.sqrt(D), rng.normal(size=(D, F)) / np.sqrt(F)
    W = {k: torch.tensor(v).to(torch.bfloat16).to(torch.float64).numpy() for k, v in W.items()}
    part = bound("ffn", PartSpec("router_experts", {"hidden_size": D, "intermediate_size": F, "experts": E, "top": top,
                                                    "router": "router", "router_bias": "router.b", "expert_prefix": "e"}), W, dtype=dtype)
    h = torch.tensor(rng.normal(size=(T, D))).to(torch.bfloat16).to(torch.float64).numpy()
    ref = plain.routed_experts(h, W, {"router": {"experts": E, "top": top}})
    ctx = ctx_for([T], [0], pad_rows=3)
    out = part.forward(rows(h, dtype=dtype, pad=3), ctx, ).cpu().numpy()[:T]
    assert int(ctx.status.item()) == 0
    if dtype == torch.float32:
        assert rel(ref, out) < 2e-5
        return
    z = np.sort(h @ W["router"].T + W["router.b"], axis=1)[:, ::-1]
    sure = np.ones(T, bool) if top == E else (z[:, top - 1] - z[:, top]) > 1e-3 * (z[:, 0] - z[:, -1])
    assert sure.sum() >= 0.95 * T and rel(ref[sure], out[sure]) < 3e-2


def test_mean_of_two_normed_branches_and_norm_behind_a_sublayer():
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(5)
    for T, D in ((1, 40), (70, 52), (9, 2500)):
        a, b, x, e = (rng.normal(size=(T, D)) * s for s in (3.0, 0.2, 1.0, 1.0))
        ga, gb, g1, g2 = (1.0 + 0.1 * rng.normal(size=D) for _ in range(4))
        t = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
        got = kernels.rms_pair_mean(t(a), t(b), t(ga), t(gb), 1e-5, 0.5).cpu().numpy()
        assert rel(0.5 * (plain.rms_norm(a, ga, 1e-5, False) + plain.rms_norm(b, gb, 1e-5, False)), got) < 1e-5
        xt = t(x)
        h = kernels.rmsnorm_add(xt, t(a), t(g1), 1e-5, extra=t(e), gain2=t(g2), eps2=1e-3).cpu().numpy()
        new = x + e + plain.rms_norm(a, g1, 1e-5, False)
        assert rel(new, xt.cpu().numpy()) < 1e-5 and rel(plain.rms_norm(new, g2, 1e-3, False), h) < 1e-5
        xt = t(x)
        assert kernels.rmsnorm_add(xt, t(b), t(g1), 1e-5) is None and rel(x + plain.rms_norm(b, g1, 1e-5, False), xt.cpu().numpy()) < 1e-5
