"""Small Gomuzen configurations and weights for the tests (numpy generator; values that bfloat16 holds exactly)."""
import json
import os
import zlib

import numpy as np
import torch


def _rot(dims, base, scaling):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, scaling=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "scale": scale, "rot": _rot(rot_dim, base, scaling)}}


def differential(heads, kv_heads, dim, vdim, scale, softcap, diff, rot_dims, base=10000.0, scaling=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "softcap": softcap, "diff": diff, "rot": _rot(rot_dims, base, scaling)}}


def windowed(heads, kv_heads, dim, vdim, scale, softcap, rot_dims, base=10000.0, scaling=None, window=None, keep_first=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
         "rot": _rot(rot_dims, base, scaling)}
    if window is not None:
        m["mask"] = {"size": window, "keep_first": keep_first}
    return {"type": "attention_2", "mixer": m}


def moe(layer, ff, limit, experts, top, scale, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return dict(layer, mlp={"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router})


def bare(layer):
    return dict(layer, mlp=None)


def config(width, vocab, layers, eps=1e-5, loop=None):
    c = {"architecture": "Gomuzen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# every mixer twice with different sizes, experts with and without groups, a layer without feed-forward, a window with
# kept first tokens and a window without, interpolated and plain rotations, a range of three layers run three times
HYBRID = config(64, 300, [
    moe(latent(4, 16, 8, 24, 40, 0.3, base=5000.0, scaling=(4.0, 64, 16.0, 1.0)), 40, 1.5, 6, 2, 1.7, groups=(3, 2)),
    moe(differential(4, 2, 16, 24, 0.25, 30.0, 0.3, 8), 24, 0.7, 8, 3, 2.0, groups=(4, 2)),
    moe(windowed(6, 2, 16, 8, 0.2, 10.0, 16, base=1000.0, scaling=(4.0, 64, 16.0, 1.0), window=40, keep_first=5), 32, 3.0, 4, 1, 1.0),
    bare(windowed(2, 1, 24, 16, 0.2, 25.0, 8, base=300.0)),
    moe(latent(3, 8, 16, 8, 24, 0.25, base=300.0), 24, 1.0, 5, 5, 0.5, groups=(1, 1)),
    moe(differential(3, 3, 8, 16, 0.35, 15.0, 0.8, 8, base=500.0, scaling=(2.0, 32, 8.0, 1.0)), 16, 2.0, 6, 2, 1.2, groups=(2, 1)),
    bare(windowed(4, 4, 8, 8, 0.3, 40.0, 4, window=70)),
], loop=(1, 4, 3))
# sizes that are no multiple of 8 or 4, one head, one expert, top 1, constants of 1, a window of one position, kept first
# tokens that fill more than a page, a kept count beyond the window's reach of short prompts, a loop that runs once
ODD = config(44, 131, [
    moe(latent(1, 6, 10, 5, 13, 1.0, base=77.0), 12, 1.0, 1, 1, 1.0),
    moe(differential(1, 1, 10, 6, 1.0, 1.0, 0.0, 6, base=20.0), 10, 2.5, 7, 7, 1.0, groups=(7, 7)),
    bare(windowed(3, 1, 10, 6, 0.5, 1.0, 10, base=33.0, window=1, keep_first=0)),
    moe(windowed(2, 2, 6, 7, 0.4, 50.0, 2, base=90.0, window=9, keep_first=70), 20, 0.9, 9, 2, 3.0, groups=(3, 1)),
    bare(differential(5, 1, 5, 9, 0.6, 8.0, 0.5, 4, base=90.0)),
], eps=1e-3, loop=(0, 2, 1))
# no loop at all
PLAIN = config(48, 200, [
    moe(windowed(4, 2, 8, 8, 0.3, 20.0, 8, window=33, keep_first=3), 24, 1.3, 4, 2, 2.2, groups=(2, 1)),
    bare(latent(2, 8, 8, 8, 16, 0.25, base=300.0)),
])
ONLY_LATENT = config(48, 200, [bare(latent(4, 16, 8, 8, 24, 0.25, base=300.0, scaling=(8.0, 32, 8.0, 2.0)))], loop=(0, 1, 2))      # the one layer twice
ONLY_DIFF = config(48, 200, [bare(differential(4, 2, 16, 12, 0.25, 12.0, 0.4, 12, base=1000.0))])
ONLY_WINDOW = config(48, 200, [bare(windowed(4, 2, 16, 12, 0.25, 12.0, 16, base=1000.0, scaling=(8.0, 32, 8.0, 2.0), window=50, keep_first=7))])
ONLY_SLIDE = config(48, 200, [bare(windowed(4, 2, 16, 12, 0.25, 12.0, 16, base=1000.0, window=70))])      # nothing kept: pages go back
ONLY_MOE = config(48, 200, [moe(windowed(1, 1, 8, 8, 0.3, 5.0, 8), 56, 1.2, 12, 3, 1.9, groups=(4, 2))])
# attention whose softmax is sharp (large query and key weights, a cap far above the scores): one key stands out
SHARP = config(64, 150, [
    bare(windowed(4, 2, 16, 16, 1.0, 200.0, 16, base=1000.0, window=76, keep_first=10)),
    bare(differential(2, 1, 16, 16, 1.0, 200.0, 0.3, 16, base=1000.0)),
    bare(latent(4, 16, 16, 16, 32, 1.0, base=1000.0)),
    bare(windowed(2, 2, 16, 8, 1.0, 200.0, 8, base=1000.0, window=130, keep_first=66)),
])
# heads of 64 and 128 with equal keys and values, cache rows of 128: the sizes the tensor-core attention kernels take
WIDE = config(128, 200, [
    moe(windowed(4, 2, 64, 64, 0.125, 18.0, 64, window=100, keep_first=12), 64, 2.0, 8, 2, 2.0, groups=(4, 2)),
    bare(differential(2, 1, 64, 64, 0.125, 30.0, 0.5, 32)),
    bare(latent(16, 16, 32, 8, 96, 0.2, base=500.0, scaling=(2.0, 128, 32.0, 1.0))),
    bare(windowed(2, 1, 128, 128, 0.09, 50.0, 128, window=200, keep_first=70)),
    bare(windowed(4, 1, 64, 64, 0.125, 15.0, 32)),
    bare(differential(4, 2, 128, 128, 0.09, 30.0, 0.2, 128)),
], loop=(0, 2, 2))
# the large ends: a cache row of 256 values, heads of 256, many experts in many groups
LARGE = config(96, 180, [
    bare(latent(8, 40, 64, 24, 192, 0.06, base=10000.0)),
    moe(windowed(2, 1, 256, 40, 0.06, 30.0, 64, window=150, keep_first=130), 200, 2.0, 72, 4, 1.5, groups=(12, 5)),
    bare(differential(2, 2, 200, 256, 0.07, 30.0, 0.6, 100)),
])

CONFIGS = {"hybrid": HYBRID, "odd": ODD, "plain": PLAIN, "latent": ONLY_LATENT, "diff": ONLY_DIFF, "window": ONLY_WINDOW,
           "slide": ONLY_SLIDE, "moe": ONLY_MOE, "sharp": SHARP, "wide": WIDE, "large": LARGE}


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    if cfg.get("loop"):
        s["loop.step"] = (cfg["loop"]["times"], D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = (D,)
        mlp = L.get("mlp")
        if mlp:
            s[p + "norm2"] = (D,)
            F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            for e in range(E):
                s[f"{p}mlp.e{e}.gate"] = s[f"{p}mlp.e{e}.up"] = (F, D)
                s[f"{p}mlp.e{e}.down"] = (D, F)
            s[p + "mlp.router"], s[p + "mlp.correction"] = (E, D), (E,)
        p += "mix."
        H = m["heads"]
        if L["type"] == "latent_attention":
            s.update({p + "q": (H * (m["dim"] + m["rot_dim"]), D), p + "dkv": (m["kv_rank"] + m["rot_dim"], D),
                      p + "dkv.norm": (m["kv_rank"],), p + "uk": (H * m["dim"], m["kv_rank"]),
                      p + "uv": (H * m["vdim"], m["kv_rank"]), p + "g": (H, D), p + "o": (D, H * m["vdim"])})
            continue
        G, M = m["kv_heads"], 2 if L["type"] == "attention" else 1
        s.update({p + "q": (H * M * m["dim"], D), p + "k": (G * M * m["dim"], D), p + "v": (G * m["vdim"], D),
                  p + "o": (D, H * m["vdim"])})
        if L["type"] == "attention":
            for n in ("q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2"):
                s[p + n] = (m["dim"],)
        else:
            s.update({p + "q.b": (H * m["dim"],), p + "k.b": (G * m["dim"],), p + "v.b": (G * m["vdim"],)})
    return s


def make_weights(cfg, seed, sharp=False, steady=False):
    """sharp: large query weights and gains, so that single keys stand out. steady: corrections far apart, so that a
    router's choice rarely hangs on a narrow gap (for runs in bfloat16, where a narrow gap may fall either way)."""
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name == "embed":
            w = rng.normal(0, 1.0, shape)
        elif last in ("norm", "norm1", "norm2"):
            w = (2.5 if sharp and name.endswith((".q.norm", ".dkv.norm")) else 1.0) * (1.0 + 0.1 * rng.normal(size=shape))
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            w = 0.3 * rng.normal(size=shape)
        elif last == "correction":
            w = (3.0 if steady else 0.2) * rng.normal(size=shape)
        elif last == "b":
            w = 0.3 * rng.normal(size=shape)
        elif name == "loop.step":
            w = 0.5 * rng.normal(size=shape)
        elif last == "g":
            w = rng.normal(0, 2.0 / np.sqrt(shape[1]), shape)
        elif len(shape) == 2:
            gain = 3.0 if sharp and last == "q" and ".mix." in name else 1.0
            w = rng.normal(0, gain / np.sqrt(shape[1]), shape)
        else:
            w = 0.1 * rng.normal(size=shape)
        W[name] = torch.tensor(np.asarray(w), dtype=torch.float32).to(torch.bfloat16)
    return W


def as_numpy(W):
    return {n: t.to(torch.float64).numpy() for n, t in W.items()}


def write_model(folder, cfg, W):
    from mynah_slm_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), W)
    return folder


def write_models(root, names=None):
    """name -> (folder, config, weights as float64 numpy)."""
    out = {}
    for name, cfg in CONFIGS.items():
        if names is not None and name not in names:
            continue
        W = make_weights(cfg, zlib.crc32(name.encode()) % 1000, sharp=name == "sharp",       # a seed that stays with the name
                         steady=name in ("hybrid", "wide", "large"))
        out[name] = (write_model(os.path.join(str(root), name), cfg, W), cfg, as_numpy(W))
    return out
