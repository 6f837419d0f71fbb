"""Plain Gomuzen forward pass: whole sequences, no cache, numpy float64.

One function per mechanism, written from the design's equations. Notation: T tokens, x the residual stream
[T, width], W the dictionary of weights by tensor name, p a tensor-name prefix, m a mixer's entry of the
configuration. Linear weights are [out, in] and applied as x @ W.T. No code is shared with the product package.

  rms_unit            x / sqrt(mean(x^2) + eps)
  rotary_tables       cos and sin of every (position, pair), with the optional long-context interpolation
  turn                pairs (2i, 2i+1) or (i, i + dims/2) of a head's first `dims` dimensions turned
  visible             the mask: causal, optionally a window that also keeps the sequence's first tokens
  softmax_rows        softmax over the visible keys of every query
  gated_latent_attention   attention over one latent per position, every head's output gated by a sigmoid
  differential_attention   two attention maps a head over the same values, a1 - lambda a2, unit RMS, (1 - diff)
  capped_window_attention  biased projections, capped scores, window with kept first tokens
  pick_experts        sigmoid scores, correction for the choice, best groups, `top` of them
  expert, grouped_moe the clamped-gate expert and the weighted sum of a token's experts
  forward             embedding, layers (a range of them several times, a learned vector added before every
                      pass), norm, head
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rotary_tables(positions, rot):
    """cos, sin [T, dims/2]. rot: {dims, base, scaling?: {factor, original, fast, slow}}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, original = float(sc["factor"]), float(sc["original"])

        def dim_of(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    return np.cos(a) * mult, np.sin(a) * mult


def turn(x, positions, rot, pairing):
    """x [T, ..., d]: the first rot.dims of the last axis are turned, the rest pass."""
    dims = int(rot["dims"])
    c, s = rotary_tables(positions, rot)
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = c.reshape(shape), s.reshape(shape)
    out = x.copy()
    if pairing == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        half = dims // 2
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    return out


def visible(positions, window=None, keep_first=0):
    """[T, T] bool: query i sees key j."""
    p = np.asarray(positions)
    i, j = p[:, None], p[None, :]
    vis = j <= i
    if window is not None:
        vis &= (i - j < window) | (j < keep_first)
    return vis


def softmax_rows(s, vis):
    s = np.where(vis, s, -np.inf)
    w = np.exp(s - s.max(-1, keepdims=True))
    return w / w.sum(-1, keepdims=True)


def gated_latent_attention(h, W, p, m, eps, positions):
    T = h.shape[0]
    H, dim, rd, vd, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = (h @ W[p + "q"].T).reshape(T, H, dim + rd)
    d = h @ W[p + "dkv"].T
    c = rms_unit(d[:, :r], eps) * W[p + "dkv.norm"]
    kr = turn(d[:, r:], positions, m["rot"], "interleaved")
    qr = turn(q[..., dim:], positions, m["rot"], "interleaved")
    ku = (c @ W[p + "uk"].T).reshape(T, H, dim)
    v = (c @ W[p + "uv"].T).reshape(T, H, vd)
    gate = sigmoid(h @ W[p + "g"].T)                                   # [T, H]
    vis = visible(positions)
    out = np.zeros((T, H, vd))
    for hd in range(H):
        s = (q[:, hd, :dim] @ ku[:, hd].T + qr[:, hd] @ kr.T) * float(m["scale"])
        out[:, hd] = (softmax_rows(s, vis) @ v[:, hd]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def capped(s, cap):
    return cap * np.tanh(s / cap)


def differential_attention(h, W, p, m, eps, positions):
    T = h.shape[0]
    H, G, dim, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    q = (h @ W[p + "q"].T).reshape(T, H, 2, dim)
    k = (h @ W[p + "k"].T).reshape(T, G, 2, dim)
    v = (h @ W[p + "v"].T).reshape(T, G, vd)
    q = turn(rms_unit(q, eps) * W[p + "q.norm"], positions, m["rot"], "half")
    k = turn(rms_unit(k, eps) * W[p + "k.norm"], positions, m["rot"], "half")
    lam = (math.exp(float(np.sum(W[p + "lq1"] * W[p + "lk1"]))) - math.exp(float(np.sum(W[p + "lq2"] * W[p + "lk2"])))
           + diff)
    vis = visible(positions)
    out = np.zeros((T, H, vd))
    for hd in range(H):
        g = hd // (H // G)
        a = [softmax_rows(capped(q[:, hd, j] @ k[:, g, j].T * float(m["scale"]), float(m["softcap"])), vis) @ v[:, g]
             for j in range(2)]
        out[:, hd] = rms_unit(a[0] - lam * a[1], eps) * (1.0 - diff)
    return out.reshape(T, H * vd) @ W[p + "o"].T


def capped_window_attention(h, W, p, m, eps, positions):
    T = h.shape[0]
    H, G, dim, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, dim)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, dim)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, vd)
    q, k = turn(q, positions, m["rot"], "half"), turn(k, positions, m["rot"], "half")
    mask = m.get("mask") or {}
    vis = visible(positions, mask.get("size"), int(mask.get("keep_first", 0)))
    out = np.zeros((T, H, vd))
    for hd in range(H):
        g = hd // (H // G)
        s = capped(q[:, hd] @ k[:, g].T * float(m["scale"]), float(m["softcap"]))
        out[:, hd] = softmax_rows(s, vis) @ v[:, g]
    return out.reshape(T, H * vd) @ W[p + "o"].T


def pick_experts(h, W, p, router, margins=None):
    """(experts [T, top], weights [T, top]) in the order of the choice. `margins`, a list, receives per token the
    smallest gap by which a group or an expert made it into the choice (inf where nothing was left out)."""
    E, top = int(router["experts"]), int(router["top"])
    s = sigmoid(h @ W[p + "router"].T)
    choice = s + W[p + "correction"]
    groups = router.get("groups")
    gap = np.full(h.shape[0], np.inf)
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        g = choice.reshape(-1, n, per)
        score = np.sort(g, axis=-1)[..., -2:].sum(-1)                     # a group's two largest
        best = np.argsort(-score, axis=-1, kind="stable")[:, :keep]
        if keep < n:
            ordered = -np.sort(-score, axis=-1)
            gap = np.minimum(gap, ordered[:, keep - 1] - ordered[:, keep])
        allowed = np.zeros((h.shape[0], n), dtype=bool)
        np.put_along_axis(allowed, best, True, axis=1)
        choice = np.where(np.repeat(allowed, per, axis=1), choice, -np.inf)
    picked = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    if margins is not None:
        ordered = -np.sort(-choice, axis=-1)
        if top < E:
            with np.errstate(invalid="ignore"):
                d = ordered[:, top - 1] - ordered[:, top]
            gap = np.minimum(gap, np.where(np.isnan(d), np.inf, d))
        margins.append(gap)
    return picked, np.take_along_axis(s, picked, axis=1) * float(router["scale"])


def expert(h, W, p, limit):
    g = np.minimum(h @ W[p + "gate"].T, limit)
    u = np.clip(h @ W[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def grouped_moe(h, W, p, mlp, margins=None):
    picked, weights = pick_experts(h, W, p, mlp["router"], margins)
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, w in zip(picked[t], weights[t]):
            out[t] += w * expert(h[t:t + 1], W, f"{p}e{int(e)}.", float(mlp["expert"]["limit"]))[0]
    return out


MIXERS = {"latent_attention": gated_latent_attention, "attention": differential_attention,
          "attention_2": capped_window_attention}


def layer_runs(cfg):
    """(layer, number of the pass whose first layer it is or None) in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(cfg, W, tokens, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence from position 0; `layers_out`, a list, receives the stream behind every run,
    `margins`, a list, every routed feed-forward's per-token gap between chosen and not chosen (see pick_experts)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = np.arange(len(tokens))
    eps = float(cfg["norm"]["eps"])
    x = np.asarray(W["embed"], dtype=np.float64)[tokens]
    for i, first_of_pass in layer_runs(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if first_of_pass is not None:
            x = x + W["loop.step"][first_of_pass]
        h = rms_unit(x, eps) * W[p + "norm1"]
        x = x + MIXERS[L["type"]](h, W, p + "mix.", L["mixer"], eps, positions)
        if L.get("mlp") is not None:
            h = rms_unit(x, eps) * W[p + "norm2"]
            x = x + grouped_moe(h, W, p + "mlp.", L["mlp"], margins)
        if layers_out is not None:
            layers_out.append(x.copy())
    return (rms_unit(x, eps) * W["final.norm"]) @ np.asarray(W["head"], dtype=np.float64).T
