"""The Gupizen design in plain numpy (float64), one function per mechanism, whole
sequences, no cache. It shares no code with the package; the tests compare the
engine with it.

A layer:  x <- x + post1(mixer(cin1(pre1(x)))),  x <- x + post2(ff(cin2(pre2(x))))
with pre/post RMS norms whose gains are stored around zero (1 + w) and
cin(h) = h + causal per-channel convolution of h. Two mixers: "parallel" (a
windowed softmax attention with a sink, mixed heads and rotated values, beside
a gated linear recurrent unit; the mean of their RMS-normed outputs) and
"channel_delta" (a gated delta rule with one decay per key channel). The
feed-forward is a set of small GELU experts with a softmax-over-the-chosen
router. A range of layers may run several times, the embedding output being
added again before every pass but the first.
"""
from __future__ import annotations

import math

import numpy as np


def rms_norm(x, w, eps, offset):
    """x / sqrt(mean(x^2) + eps) * (w, or 1 + w)."""
    x = np.asarray(x, np.float64)
    r = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return r * ((1.0 + w) if offset else w)


def causal_conv(x, w, bias=None):
    """y_t[c] = sum_j w[c, j] x_(t - taps + 1 + j)[c] (+ bias), zeros before the start. x [T, C], w [C, taps]."""
    T, C = x.shape
    taps = w.shape[1]
    y = np.zeros((T, C))
    for j in range(taps):
        shift = taps - 1 - j
        if shift < T:
            y[shift:] += x[: T - shift] * w[:, j]
    if bias is not None:
        y = y + bias
    return y


def input_conv(h, w):
    return h + causal_conv(h, w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    from math import erf
    return 0.5 * z * (1.0 + np.vectorize(erf)(z / math.sqrt(2.0)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def rotary_freqs(dims, base, scaling=None):
    """f_i = base^(-2i/dims); with scaling {factor, low, high, original}: short wavelengths keep f, long ones use
    f / factor, the band between is blended linearly in original / wavelength."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.copy()
    for i, fi in enumerate(f):
        wl = 2.0 * math.pi / fi
        if wl < orig / high:
            continue
        if wl > orig / low:
            out[i] = fi / factor
        else:
            s = (orig / wl - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_pairs(x, pos, freqs, sign=1.0):
    """Turn the pairs (2i, 2i+1) of the first 2*len(freqs) dimensions of x [T, heads, d] by sign * pos * f_i."""
    x = np.array(x, np.float64)
    n = len(freqs)
    ang = sign * np.asarray(pos, np.float64)[:, None] * freqs[None, :]          # [T, n]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:2 * n:2].copy(), x[..., 1:2 * n:2].copy()
    x[..., 0:2 * n:2] = u * c - v * s
    x[..., 1:2 * n:2] = v * c + u * s
    return x


def sink_talk_attention(h, W, m, pos):
    """The left mixer. W: its tensors by short name (q, k, v, o, talk, sink); m: its sizes and constants."""
    T = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W["q"].T).reshape(T, H, dim)
    k = (h @ W["k"].T).reshape(T, G, dim)
    v = (h @ W["v"].T).reshape(T, G, vd)
    rot = m["rot"]
    fk = rotary_freqs(rot["dims"], rot["base"], rot.get("scaling"))
    fv = rotary_freqs(vd, rot["base"], None)
    q, k = rotate_pairs(q, pos, fk), rotate_pairs(k, pos, fk)
    v = rotate_pairs(v, pos, fv)
    window = m["mask"]["size"]
    out = np.zeros((T, H, vd))
    rep = H // G
    for i in range(T):
        lo = max(0, i - window + 1)
        w = np.zeros((H, i + 1 - lo))
        for hh in range(H):
            s = (k[lo:i + 1, hh // rep] @ q[i, hh]) * m["scale"]
            mx = max(s.max(), W["sink"][hh])
            e = np.exp(s - mx)
            w[hh] = e / (e.sum() + math.exp(W["sink"][hh] - mx))
        wm = W["talk"] @ w                                                       # [H, keys]
        for hh in range(H):
            out[i, hh] = wm[hh] @ v[lo:i + 1, hh // rep]
    out = rotate_pairs(out, pos, fv, sign=-1.0)
    return out.reshape(T, H * vd) @ W["o"].T


def rglru(h, W, m):
    """The right mixer: a real-gated linear recurrent unit between two branches."""
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ W["y"].T + W["y.b"])
    u = causal_conv(h @ W["x"].T + W["x.b"], W["conv"], W["conv.b"])
    bw = width // blocks
    r = np.zeros((T, width))
    i = np.zeros((T, width))
    for b in range(blocks):
        ub = u[:, b * bw:(b + 1) * bw]
        r[:, b * bw:(b + 1) * bw] = sigmoid(ub @ W["ra"][b].T + W["ra.b"][b])
        i[:, b * bw:(b + 1) * bw] = sigmoid(ub @ W["ri"][b].T + W["ri.b"][b])
    log_a = -8.0 * r * softplus(W["lam"])
    a = np.exp(log_a)
    S = np.zeros(width)
    out = np.zeros((T, width))
    for t in range(T):
        S = a[t] * S + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ W["o"].T


def parallel_mixer(h, W, m, pos, eps):
    left = {k[len("left."):]: v for k, v in W.items() if k.startswith("left.") and k != "left.out"}
    right = {k[len("right."):]: v for k, v in W.items() if k.startswith("right.") and k != "right.out"}
    a = sink_talk_attention(h, left, m["left"], pos)
    b = rglru(h, right, m["right"])
    return 0.5 * (rms_norm(a, W["left.out"], eps, False) + rms_norm(b, W["right.out"], eps, False))


def channel_delta(h, W, m, eps):
    """Gated delta rule with a decay per head and key channel."""
    T = h.shape[0]
    H, G, dim, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W["q"].T, W["q.conv"])).reshape(T, G, dim)
    k = silu(causal_conv(h @ W["k"].T, W["k.conv"])).reshape(T, G, dim)
    v = silu(causal_conv(h @ W["v"].T, W["v.conv"])).reshape(T, H, vd)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W["b"].T)                                                 # [T, H]
    dt = softplus((h @ W["a1"].T) @ W["a2"].T + W["dt_bias"]).reshape(T, H, dim)
    g = np.exp(-np.exp(W["A_log"])[None, :, None] * dt)                          # [T, H, dim]
    gate = sigmoid((h @ W["g1"].T) @ W["g2"].T).reshape(T, H, vd)
    rep = H // G
    S = np.zeros((H, dim, vd))
    o = np.zeros((T, H, vd))
    for t in range(T):
        for hh in range(H):
            kk, qq = k[t, hh // rep], q[t, hh // rep]
            S[hh] = g[t, hh][:, None] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ kk)
            S[hh] = S[hh] + np.outer(kk, u)
            o[t, hh] = S[hh].T @ qq
    o = o / np.sqrt(np.mean(o * o, axis=-1, keepdims=True) + eps) * W["norm"] * gate
    return o.reshape(T, H * vd) @ W["o"].T


def routed_experts(h, W, mlp):
    """Each token's `top` experts by router logit; weights: softmax over the chosen logits."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ W["router"].T + W["router.b"]
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-z[t, e], e))[:top]
        zz = np.array([z[t, e] for e in order])
        p = np.exp(zz - zz.max())
        p = p / p.sum()
        for e, pe in zip(order, p):
            out[t] += pe * (gelu_erf(h[t] @ W[f"e{e}.up"].T) @ W[f"e{e}.down"].T)
    return out


def schedule(cfg):
    """Layer indices in the order they run, with a flag: the embedding output is added before this run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(start)]
    for p in range(times):
        runs += [(i, p > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence; with return_layers also the residual stream behind every run."""
    w = {k: np.asarray(v, np.float64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x = x0.copy()
    pos = np.arange(len(tokens))
    layers = []
    for li, add in schedule(cfg):
        L = cfg["layers"][li]
        p = f"l{li}."
        if add:
            x = x + x0
        h = input_conv(rms_norm(x, w[p + "norm1"], eps, True), w[p + "canon1"])
        if L["type"] == "parallel":
            y = parallel_mixer(h, sub(w, p + "mix."), L["mixer"], pos, eps)
        elif L["type"] == "channel_delta":
            y = channel_delta(h, sub(w, p + "mix."), L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, w[p + "norm1b"], eps, True)
        if L.get("mlp") is not None:
            h = input_conv(rms_norm(x, w[p + "norm2"], eps, True), w[p + "canon2"])
            x = x + rms_norm(routed_experts(h, sub(w, p + "mlp."), L["mlp"]), w[p + "norm2b"], eps, True)
        layers.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps, True) @ w["embed"].T
    return (logits, np.stack(layers)) if return_layers else logits
