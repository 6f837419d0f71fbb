"""The kernels behind the Gomuzen parts, each alone, against the plain functions of tests/plain/gomuzen.py (float64):
the preparation of capped / differential attention with its cache write, the attention kernels under a cap, a window
that keeps first tokens and key heads that share value heads (general and tensor-core forms, prompts and single
queries, ONE key made to stand out just inside and just outside every edge), the combination of two score maps, the
head gate, the vector added to the stream, and the group-limited router with its experts."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import gomuzen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def i32(v):
    return torch.tensor(np.asarray(v), dtype=torch.int32, device=DEV)


def t32(a):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV)


def rel(ref, got):
    ref, got = np.asarray(ref, dtype=np.float64), np.asarray(got, dtype=np.float64)
    return float(np.abs(ref - got).max() / max(np.abs(ref).max(), 1e-30))


def step_ctx(q_lens, starts, pad_rows=0):
    """What the kernels read of a step: rows packed sequence by sequence (then padding rows), every sequence's pages
    handed out in a shuffled order from one pool."""
    from mynah_slm_b200.ops import kernels
    tok_seq, tok_pos, cu, kv_len, indptr, ids = [], [], [0], [], [0], []
    total = sum((s + n + PAGE - 1) // PAGE for n, s in zip(q_lens, starts))
    pool = list(np.random.default_rng(total).permutation(total + 3))
    for b, (n, s) in enumerate(zip(q_lens, starts)):
        tok_seq += [b] * n
        tok_pos += list(range(s, s + n))
        cu.append(cu[-1] + n)
        kv_len.append(s + n)
        ids += [int(pool.pop()) for _ in range((s + n + PAGE - 1) // PAGE)]
        indptr.append(len(ids))
    tok_seq += [-1] * pad_rows
    tok_pos += [0] * pad_rows
    B = len(q_lens)
    pages = kernels.PageTableView(i32(indptr), i32(ids), i32([0] * B), total + 3)
    ctx = SimpleNamespace(tok_seq=i32(tok_seq), tok_pos=i32(tok_pos), cu_q=i32(cu), kv_len=i32(kv_len), B=B, T=len(tok_seq),
                          status=torch.zeros((1,), dtype=torch.int32, device=DEV), is_decode=all(n == 1 for n in q_lens),
                          max_q_len=max(q_lens), decode_splits=max((k + PAGE - 1) // PAGE for k in kv_len), pages=[pages])
    return ctx, pages, total + 3


def place(cache, pages_ids, indptr, b, rows):
    """rows [n, heads, d] of sequence b from position 0 into its pages."""
    for p in range(rows.shape[0]):
        cache[pages_ids[indptr[b] + p // PAGE], :, p % PAGE] = rows[p]


# ------------------------------------------------------------------ preparation
@pytest.mark.parametrize("H,G,M,dim,vd,rot,interleaved,norm,bias", [
    (4, 2, 2, 16, 24, 8, False, True, False), (6, 2, 1, 16, 8, 16, False, False, True), (1, 1, 2, 10, 6, 6, False, True, True),
    (3, 1, 1, 10, 7, 4, True, False, False), (5, 5, 2, 5, 9, 0, False, True, False),
    # units that move 16 bytes at a time (the vector form): whole and partial rotations in both pairings, every width
    (4, 2, 2, 64, 64, 32, False, True, False), (2, 1, 1, 128, 128, 128, False, False, True), (3, 3, 1, 32, 8, 32, True, True, True),
    (2, 2, 2, 256, 40, 64, False, True, False), (8, 4, 1, 8, 8, 0, False, True, True), (6, 3, 1, 16, 24, 6, True, False, True),
    (16, 8, 1, 128, 128, 64, False, True, True)])
def test_capped_prep_and_cache_rows(H, G, M, dim, vd, rot, interleaved, norm, bias):
    from mynah_slm_b200.ops import kernels
    from mynah_slm_b200.parts.position import rotary_frequencies
    rng = np.random.default_rng(H * 100 + dim)
    dimp, vdp, R = (dim + 7) // 8 * 8, (vd + 7) // 8 * 8, H // G
    T, start = 70, 60                                            # positions 60..129: three pages, two partly written
    nq, nk, nv = H * M * dim, G * M * dim, G * vd
    x = rng.normal(size=(T, nq + nk + nv))
    b_all = rng.normal(size=(nq + nk + nv,)) if bias else np.zeros(nq + nk + nv)
    gq, gk = 1.0 + 0.1 * rng.normal(size=(dim,)), 1.0 + 0.1 * rng.normal(size=(dim,))
    cos = sin = None
    if rot:
        f, mult = rotary_frequencies(rot, 300.0, None)
        cos, sin = kernels.rope_table_freqs(256, f, mult, DEV)
    ctx, pages, n_pages = step_ctx([T], [start], pad_rows=2)
    xin = torch.cat([t32(x), torch.zeros((2, x.shape[1]), device=DEV)], 0).contiguous()
    k_cache = torch.full((n_pages, G * M, PAGE, dimp), 9.0, dtype=torch.float32, device=DEV)
    v_cache = torch.full((n_pages, G, PAGE, vdp), 9.0, dtype=torch.float32, device=DEV)
    q_out = torch.full((T + 2, H * M * dimp), 9.0, dtype=torch.float32, device=DEV)
    kernels.capped_attn_prep(xin, q_out, H * M, G * M, G, dim, vd, dimp, vdp, M, R, t32(b_all) if bias else None,
                             t32(gq) if norm else None, t32(gk) if norm else None, 1e-5, cos, sin, rot, interleaved, ctx, pages,
                             k_cache, v_cache)
    assert int(ctx.status.item()) == 0
    pos = np.arange(start, start + T)
    y = x + b_all
    q, k, v = y[:, :nq].reshape(T, H, M, dim), y[:, nq:nq + nk].reshape(T, G, M, dim), y[:, nq + nk:].reshape(T, G, vd)
    if norm:
        q, k = plain.rms_unit(q, 1e-5) * gq, plain.rms_unit(k, 1e-5) * gk
    if rot:
        pairing = "interleaved" if interleaved else "half"
        q, k = plain.turn(q, pos, {"dims": rot, "base": 300.0}, pairing), plain.turn(k, pos, {"dims": rot, "base": 300.0}, pairing)
    ids = pages.ids.cpu().numpy()
    got_k = torch.stack([k_cache[ids[p // PAGE], :, p % PAGE] for p in pos]).cpu().numpy()          # [T, G*M, dimp]
    got_v = torch.stack([v_cache[ids[p // PAGE], :, p % PAGE] for p in pos]).cpu().numpy()
    assert rel(k.reshape(T, G * M, dim), got_k[..., :dim]) < 1e-5 and np.all(got_k[..., dim:] == 0)
    assert rel(v, got_v[..., :vd]) < 1e-5 and np.all(got_v[..., vd:] == 0)
    # nothing else was written: the rows before position 60 of the first page, those after 129 of the last, other pages
    assert float(k_cache[ids[0], :, :60].min()) == 9.0 and float(k_cache[ids[2], :, 2:].min()) == 9.0
    assert float(v_cache[ids[0], :, :60].min()) == 9.0 and float(v_cache[ids[2], :, 2:].min()) == 9.0
    others = [p for p in range(n_pages) if p not in ids[:3]]
    assert float(k_cache[others].min()) == 9.0 and float(v_cache[others].min()) == 9.0
    # the packed queries: slot (kv head, map, query head of the group)
    qo = q_out[:T].view(T, G, M, R, dimp).cpu().numpy()
    want = q.reshape(T, G, R, M, dim).transpose(0, 1, 3, 2, 4)
    assert rel(want, qo[..., :dim]) < 1e-5 and np.all(qo[..., dim:] == 0) and np.all(q_out[T:].cpu().numpy() == 9.0)


# ------------------------------------------------------------------ the attention kernels under cap, window, kept tokens
def attention_reference(q, k, v, starts, q_lens, R, vdiv, scale, cap, window, keep):
    """q [T, H, d] packed over the sequences' new rows; k, v: per sequence [n, KV, d] / [n, KV / vdiv, vd] from position 0."""
    out, at = [], 0
    for b, (n, s) in enumerate(zip(q_lens, starts)):
        pos = np.arange(s + n)
        vis = plain.visible(pos, window, keep)[s:]
        o = np.zeros((n, q.shape[1], v[b].shape[-1]))
        for h in range(q.shape[1]):
            g = h // R
            sc = q[at:at + n, h] @ k[b][:, g].T * scale
            if cap:
                sc = plain.capped(sc, cap)
            o[:, h] = plain.softmax_rows(sc, vis) @ v[b][:, g // vdiv]
        out.append(o)
        at += n
    return np.concatenate(out, 0)


def run_attention(dtype, H, KV, vdiv, d, vd, q_lens, starts, scale, cap, window, keep, seed, tc=True, sharp=None):
    """Random q, k, v (or `sharp`: one query direction and one key made large) through the dispatch, and the reference."""
    from mynah_slm_b200.ops import attention_dispatch
    rng = np.random.default_rng(seed)
    ctx, pages, n_pages = step_ctx(q_lens, starts)
    ids, indptr = pages.ids.cpu().numpy(), pages.indptr.cpu().numpy()
    T = sum(q_lens)
    rnd = lambda *shape: torch.tensor(rng.normal(size=shape), dtype=dtype).double().numpy()      # values the type holds
    q = rnd(T, H, d)
    k = [rnd(s + n, KV, d) for n, s in zip(q_lens, starts)]
    v = [rnd(s + n, KV // vdiv, vd) for n, s in zip(q_lens, starts)]
    if sharp is not None:                     # every query looks along e_0; the key at `sharp` of sequence 0 lies there
        q[..., 0] = 12.0
        for kb in k:
            kb[..., 0] = 0.0
        k[0][sharp, :, 0] = 12.0
    k_cache = torch.zeros((n_pages, KV, PAGE, d), dtype=dtype, device=DEV)
    v_cache = torch.zeros((n_pages, KV // vdiv, PAGE, vd), dtype=dtype, device=DEV)
    for b in range(len(q_lens)):
        place(k_cache, ids, indptr, b, torch.tensor(k[b], dtype=dtype, device=DEV))
        place(v_cache, ids, indptr, b, torch.tensor(v[b], dtype=dtype, device=DEV))
    qt = torch.tensor(q.reshape(T, H * d), dtype=dtype, device=DEV)
    out = torch.zeros((T, H * vd), dtype=dtype, device=DEV)
    before = attention_dispatch.USE_TC_MASKED
    attention_dispatch.USE_TC_MASKED = tc
    try:
        if ctx.is_decode:
            scratch = torch.empty((ctx.B * H * ctx.decode_splits * (max(d, vd) + 2),), dtype=torch.float32, device=DEV)
            attention_dispatch.decode_capped(qt, out, ctx, H, KV, d, vd, k_cache, v_cache, pages, window or 0, scale, cap,
                                             keep, vdiv, scratch)
        else:
            attention_dispatch.prefill_capped(qt, out, ctx, H, KV, d, vd, k_cache, v_cache, pages, window or 0, scale, cap,
                                              keep, vdiv)
    finally:
        attention_dispatch.USE_TC_MASKED = before
    assert int(ctx.status.item()) == 0
    ref = attention_reference(q, k, v, starts, q_lens, H // KV, vdiv, scale, cap, window, keep)
    return ref, out.double().cpu().numpy().reshape(T, H, vd), v


CASES = [  # H, KV, vdiv, d, vd, cap, window, keep
    (4, 2, 1, 16, 8, 10.0, 40, 5), (8, 4, 2, 16, 24, 30.0, None, 0), (3, 1, 1, 24, 16, 0.0, 70, 0), (2, 2, 2, 8, 8, 1.0, 1, 0),
    (4, 2, 1, 8, 16, 50.0, 9, 70), (6, 2, 1, 40, 40, 12.0, 90, 17), (2, 2, 1, 256, 40, 5.0, 150, 130)]


@pytest.mark.parametrize("case", CASES)
def test_general_attention_prompts_and_single_queries(case):
    H, KV, vdiv, d, vd, cap, window, keep = case
    for q_lens, starts in (([150], [0]), ([1, 70, 33], [0, 0, 0]), ([40, 2], [100, 63]), ([1, 1, 1], [0, 200, 64])):
        ref, got, _ = run_attention(torch.float32, H, KV, vdiv, d, vd, q_lens, starts, 0.3, cap, window, keep, sum(q_lens) + H)
        assert rel(ref, got) < 2e-5, (case, q_lens, starts)


@pytest.mark.parametrize("d,H,KV,vdiv,cap,window,keep", [(64, 4, 2, 1, 20.0, 100, 12), (64, 4, 2, 2, 30.0, None, 0), (128, 2, 1, 1, 50.0, 200, 70),
                                                         (128, 8, 4, 2, 30.0, None, 0), (64, 4, 1, 1, 15.0, None, 0), (128, 4, 2, 1, 25.0, 130, 64),
                                                         (64, 2, 2, 1, 20.0, 300, 129)])
def test_tensor_core_attention_against_the_general_kernels(d, H, KV, vdiv, cap, window, keep):
    """bfloat16 heads of 64 and 128: the tensor-core forms (tcgen05 for prompts, mma.sync for single queries) against the
    plain reference and against the general kernels on the same cache."""
    for q_lens, starts in (([300], [0]), ([129, 70, 1], [0, 0, 0]), ([50, 140], [200, 63]), ([1, 1, 1, 1], [0, 400, 64, 191])):
        ref, tc, _ = run_attention(torch.bfloat16, H, KV, vdiv, d, d, q_lens, starts, d ** -0.5, cap, window, keep, d + H, tc=True)
        _, gen, _ = run_attention(torch.bfloat16, H, KV, vdiv, d, d, q_lens, starts, d ** -0.5, cap, window, keep, d + H, tc=False)
        assert rel(ref, tc) < 2e-2 and rel(ref, gen) < 2e-2 and rel(gen, tc) < 2e-2, (q_lens, starts)


@pytest.mark.parametrize("dtype,d", [(torch.float32, 16), (torch.bfloat16, 64), (torch.bfloat16, 128)])
def test_one_key_stands_out_at_every_edge(dtype, d):
    """ONE key of sequence 0 is large along the direction every query looks in, so that a query that sees it returns its
    value and one that does not returns something else: the key sits on the last kept first token and on the first
    token that is not kept, on the window's last position and just behind it, at page borders, far back among
    hundreds; queries come as a prompt's rows and as single queries."""
    window, keep, n = 76, 66, 345
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    for key in (0, 63, 64, 65, 66, 67, 127, 128, 200, 256, 257):
        for q_lens, starts in (([n], [0]), ([n - 250], [250])) + tuple(([1], [p]) for p in (key, key + 1, key + 75, key + 76, 300, 344) if key <= p < n):
            ref, got, v = run_attention(dtype, 2, 2, 1, d, d, q_lens, starts, 1.0, 200.0, window, keep, key, sharp=key)
            assert rel(ref, got) < tol, (key, q_lens, starts)
            for r, p in enumerate(range(starts[0], starts[0] + q_lens[0])):
                sees = key <= p and (p - key < window or key < keep)
                hit = rel(v[0][key], got[r]) < 0.05
                assert hit == sees or p == key, f"key {key}, query at {p}: sees {sees}, returned its value {hit}"


# ------------------------------------------------------------------ maps, gate, stream vector
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,vd", [(4, 2, 24), (1, 1, 6), (6, 3, 64), (5, 5, 9), (2, 1, 256)])
def test_diff_combine(dtype, H, R, vd):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(H + vd)
    vdp, T, G = (vd + 7) // 8 * 8, 37, H // R
    a = torch.tensor(rng.normal(size=(T, G, 2, R, vdp)), dtype=dtype, device=DEV)
    ctx = SimpleNamespace(tok_seq=i32([0] * (T - 2) + [-1, -1]))
    out = kernels.diff_combine(a.view(T, -1).contiguous(), H, R, vd, vdp, 0.37, 0.6, 1e-5, ctx)
    an = a.double().cpu().numpy()[..., :vd]
    ref = (plain.rms_unit(an[:, :, 0] - 0.37 * an[:, :, 1], 1e-5) * 0.6).reshape(T, H * vd)
    assert rel(ref[:T - 2], out[:T - 2].double().cpu().numpy()) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,vd,off", [(4, 24, 8), (1, 5, 3), (16, 128, 0)])
def test_head_gate(dtype, H, vd, off):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(H + vd)
    T = 50
    x = torch.tensor(rng.normal(size=(T, H * vd)), dtype=dtype, device=DEV)
    p = torch.tensor(3.0 * rng.normal(size=(T, off + H + 5)), dtype=dtype, device=DEV)
    ref = (x.double().cpu().numpy().reshape(T, H, vd) * plain.sigmoid(p.double().cpu().numpy()[:, off:off + H])[..., None]).reshape(T, -1)
    kernels.head_gate(x, p[:, off:off + H], H, vd)
    assert rel(ref, x.double().cpu().numpy()) < (1e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,n_in,n_out", [(70, 3, 16, 40), (1, 1, 6, 13), (200, 16, 96, 128), (9, 2, 64, 24)])
def test_head_linear_with_the_gate_on_its_accumulators(dtype, T, H, n_in, n_out):
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(T + n_in)
    x = torch.tensor(rng.normal(size=(T, H * n_in)), dtype=dtype, device=DEV)
    W = torch.tensor(rng.normal(size=(H, n_out, n_in)) / np.sqrt(n_in), dtype=dtype, device=DEV)
    p = torch.tensor(2.0 * rng.normal(size=(T, 8 + H + 3)), dtype=dtype, device=DEV)
    out = torch.zeros((T, H * n_out), dtype=dtype, device=DEV)
    kernels.head_linear(x, n_in, 0, W, out, n_out, 0, gate=p[:, 8:8 + H])
    ref = np.einsum("thi,hji->thj", x.double().cpu().numpy().reshape(T, H, n_in), W.double().cpu().numpy())
    ref = ref * plain.sigmoid(p.double().cpu().numpy()[:, 8:8 + H])[..., None]
    assert rel(ref.reshape(T, -1), out.double().cpu().numpy()) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_residual_add_row():
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(3)
    x, v = rng.normal(size=(33, 44)), rng.normal(size=(44,))
    xt = t32(x)
    kernels.residual_add_row(xt, t32(v))
    assert np.array_equal(xt.cpu().numpy(), (x.astype(np.float32) + v.astype(np.float32)))


# ------------------------------------------------------------------ the router and its experts
@pytest.mark.parametrize("D,F,E,top,groups,keep", [(48, 24, 10, 3, 2, 1), (64, 40, 12, 3, 4, 2), (44, 12, 1, 1, 1, 1), (40, 10, 7, 7, 7, 7),
                                                   (48, 16, 6, 2, 3, 3), (96, 200, 72, 4, 12, 5), (52, 18, 9, 2, 3, 1), (64, 64, 16, 2, 16, 4)])
def test_group_router_and_experts(D, F, E, top, groups, keep):
    """32-bit: choices inside the kept groups, weights without the correction, clamped-gate experts; padding rows stay out."""
    from mynah_slm_b200.ops import kernels
    rng = np.random.default_rng(D + E)
    for T in (1, 5, 300):
        h = rng.normal(size=(T, D))
        W = {"router": rng.normal(size=(E, D)) / np.sqrt(D) * 2.0, "correction": 0.3 * rng.normal(size=(E,))}
        for e in range(E):
            W[f"e{e}.gate"], W[f"e{e}.up"] = rng.normal(size=(F, D)) / np.sqrt(D) * 2, rng.normal(size=(F, D)) / np.sqrt(D) * 2
            W[f"e{e}.down"] = rng.normal(size=(D, F)) / np.sqrt(F)
        W = {n: np.asarray(t32(w).cpu().numpy(), dtype=np.float64) for n, w in W.items()}
        mlp = {"expert": {"ff": F, "limit": 1.25}, "router": {"experts": E, "top": top, "scale": 2.25, "groups": {"count": groups, "keep": keep}}}
        h = np.asarray(t32(h).cpu().numpy(), dtype=np.float64)
        margins = []
        ref = plain.grouped_moe(h, W, "", mlp, margins)
        steady = margins[0] > 1e-5                                  # rows whose choice does not hang on rounding
        ctx = SimpleNamespace(tok_seq=i32([0] * T + [-1]), status=torch.zeros((1,), dtype=torch.int32, device=DEV))
        w_gu = torch.stack([torch.stack([t32(W[f"e{e}.gate"]), t32(W[f"e{e}.up"])]) for e in range(E)]).contiguous()
        w_down = torch.stack([t32(W[f"e{e}.down"]) for e in range(E)]).contiguous()
        hp = torch.cat([t32(h), torch.full((1, D), 1e9, device=DEV)], 0).contiguous()       # a padding row of huge values
        out = kernels.moe_group_router_ffn(hp, t32(W["router"]), t32(W["correction"]), w_gu, w_down, ctx, top, groups, keep, 2.25,
                                           1.25, 1.702)
        assert int(ctx.status.item()) == 0
        got = out[:T].cpu().numpy()
        assert steady.mean() > 0.9 and rel(ref[steady], got[steady]) < 2e-5, (T, rel(ref[steady], got[steady]))
