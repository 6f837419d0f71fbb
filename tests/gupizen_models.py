"""Small Gupizen configurations and weights for the tests (numpy generator; values that bfloat16 holds exactly)."""
import json
import os
import zlib

import numpy as np
import torch

# narrow sizes of the delta rule's two-step projections when the configuration leaves them to the checkpoint
FREE_RANKS = (12, 10)


def parallel(heads, kv, dim, vdim, window, rot_dims, base, scale, width, blocks, conv, scaling=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window}, "rot": rot, "scale": scale},
        "right": {"width": width, "blocks": blocks, "conv": conv}}}


def cdelta(heads, kv, dim, vdim, conv, ranks=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}
    if ranks is not None:
        m["decay_rank"], m["gate_rank"] = ranks
    return {"type": "channel_delta", "mixer": m}


def moe(layer, ff, experts, top):
    return dict(layer, mlp={"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}})


def bare(layer):
    return dict(layer, mlp=None)


def config(width, vocab, layers, taps=2, eps=1e-5, emb=3.0, loop=None):
    c = {"architecture": "Gupizen", "vocab": vocab, "width": width, "embedding": {"scale": emb}, "norm": {"eps": eps},
         "canon": {"taps": taps}, "layers": layers}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# both mixers, grouped heads in both, keys and values of different sizes, a loop over two layers in the middle, windows
# shorter and longer than a page, scaled and plain rotations, layers with and without a feed-forward
HYBRID = config(64, 300, [
    moe(parallel(4, 2, 16, 24, 40, 8, 10000.0, 0.25, 48, 3, 4, scaling=(4.0, 1.0, 4.0, 64)), 40, 6, 2),
    bare(cdelta(4, 2, 16, 8, 3)),
    moe(parallel(6, 3, 8, 16, 70, 8, 500.0, 0.4, 32, 2, 2), 24, 5, 3),
    moe(cdelta(2, 2, 24, 12, 4, ranks=(8, 16)), 32, 4, 1),
    bare(parallel(2, 1, 32, 8, 130, 16, 10000.0, 0.2, 40, 1, 3, scaling=(8.0, 1.0, 4.0, 32))),
], taps=4, loop=(1, 3, 3))
# sizes that are no multiple of 8 or 4, one head, one expert, top = experts, one block, one tap everywhere, a window
# of one token (a position sees itself alone), a loop from the first layer on and one that runs once, constants of 1
ODD = config(40, 131, [
    moe(parallel(1, 1, 6, 10, 1, 6, 77.0, 1.0, 13, 1, 1), 12, 1, 1),
    moe(cdelta(3, 1, 10, 6, 1), 20, 7, 7),
    bare(parallel(3, 3, 10, 6, 5, 4, 20.0, 0.5, 21, 7, 2)),
], taps=1, eps=1e-3, emb=1.0, loop=(0, 2, 2))
ONCE = config(40, 131, ODD["layers"][::-1], taps=3, eps=1e-3, emb=1.0, loop=(1, 3, 1))
ONLY_PARALLEL = config(48, 200, [bare(parallel(4, 2, 16, 8, 50, 12, 300.0, 0.25, 24, 2, 4, scaling=(8.0, 1.0, 4.0, 32)))])
ONLY_DELTA = config(48, 200, [bare(cdelta(4, 2, 12, 16, 4))], taps=3)
ONLY_MOE = config(48, 200, [moe(cdelta(1, 1, 8, 8, 2), 56, 9, 2)], taps=2)
# attention that decides the result: no recurrent help (the right branch's output matrix is zero), sharp queries
SHARP = config(64, 150, [
    bare(parallel(4, 4, 16, 16, 200, 16, 1000.0, 1.0, 8, 1, 2)),
    bare(parallel(2, 1, 32, 16, 97, 16, 1000.0, 0.8, 8, 1, 2)),
], taps=2)
# the sizes the bfloat16 matrix kernels tile: multiples of 128 in the products, 16 heads
WIDE = config(256, 512, [
    moe(parallel(8, 2, 64, 64, 100, 32, 10000.0, 0.125, 128, 4, 4), 128, 8, 2),
    moe(cdelta(8, 4, 64, 32, 4), 64, 16, 4),
    bare(parallel(16, 16, 32, 16, 64, 32, 500.0, 0.2, 256, 2, 4, scaling=(2.0, 1.0, 4.0, 128))),
], taps=3, loop=(0, 2, 2))
# the large ends: keys of 256, values of 200, many experts, a delta key of 300
LARGE = config(96, 180, [
    bare(parallel(2, 1, 256, 200, 150, 64, 10000.0, 0.06, 320, 5, 4)),
    moe(cdelta(2, 1, 300, 20, 4), 200, 70, 4),
], taps=2)
# a width, a vocabulary and inner sizes that are no multiple of 8 or of 4 anywhere
RAGGED = config(52, 97, [
    moe(parallel(3, 1, 14, 10, 33, 10, 33.0, 0.3, 18, 2, 3, scaling=(3.0, 2.0, 5.0, 40)), 18, 3, 2),
    moe(cdelta(2, 1, 7, 5, 3), 30, 5, 2),
    bare(parallel(2, 2, 6, 18, 64, 6, 90.0, 0.6, 9, 3, 2)),
], taps=2, eps=1e-4, emb=2.0, loop=(1, 2, 2))

CONFIGS = {"ragged": RAGGED, "hybrid": HYBRID, "odd": ODD, "once": ONCE, "parallel": ONLY_PARALLEL, "delta": ONLY_DELTA,
           "moe": ONLY_MOE, "sharp": SHARP, "wide": WIDE, "large": LARGE}


def tensor_shapes(cfg):
    D, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    s = {"embed": (V, D), "final.norm": (D,)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = s[p + "norm1b"] = (D,)
        s[p + "canon1"] = (D, taps)
        mlp = L.get("mlp")
        if mlp:
            s[p + "norm2"] = s[p + "norm2b"] = (D,)
            s[p + "canon2"] = (D, taps)
            F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            for e in range(E):
                s[f"{p}mlp.e{e}.up"], s[f"{p}mlp.e{e}.down"] = (F, D), (D, F)
            s[p + "mlp.router"], s[p + "mlp.router.b"] = (E, D), (E,)
        p += "mix."
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            H, G, dim, vd, W = a["heads"], a["kv_heads"], a["dim"], a["vdim"], r["width"]
            bw = W // r["blocks"]
            s.update({p + "left.q": (H * dim, D), p + "left.k": (G * dim, D), p + "left.v": (G * vd, D),
                      p + "left.o": (D, H * vd), p + "left.talk": (H, H), p + "left.sink": (H,), p + "left.out": (D,),
                      p + "right.y": (W, D), p + "right.y.b": (W,), p + "right.x": (W, D), p + "right.x.b": (W,),
                      p + "right.conv": (W, r["conv"]), p + "right.conv.b": (W,), p + "right.ra": (r["blocks"], bw, bw),
                      p + "right.ra.b": (r["blocks"], bw), p + "right.ri": (r["blocks"], bw, bw),
                      p + "right.ri.b": (r["blocks"], bw), p + "right.lam": (W,), p + "right.o": (D, W),
                      p + "right.out": (D,)})
        else:
            H, G, dim, vd, t = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = m.get("decay_rank", FREE_RANKS[0]), m.get("gate_rank", FREE_RANKS[1])
            s.update({p + "q": (G * dim, D), p + "k": (G * dim, D), p + "v": (H * vd, D), p + "q.conv": (G * dim, t),
                      p + "k.conv": (G * dim, t), p + "v.conv": (H * vd, t), p + "b": (H, D), p + "A_log": (H,),
                      p + "dt_bias": (H * dim,), p + "a1": (ra, D), p + "a2": (H * dim, ra), p + "g1": (rg, D),
                      p + "g2": (H * vd, rg), p + "norm": (vd,), p + "o": (D, H * vd)})
    return s


def make_weights(cfg, seed, sharp=False):
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        n = rng.normal(size=shape)
        if name == "embed":
            w = n
        elif last in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            w = 0.1 * n                                         # stored around zero
        elif last in ("out", "norm"):
            w = 1.0 + 0.1 * n                                   # plain gains
        elif last in ("canon1", "canon2"):
            w = 0.2 * n
        elif last == "conv":
            w = 0.4 * n
        elif last == "talk":
            w = 0.7 * np.eye(shape[0]) + 0.3 * n
        elif last == "sink":
            w = n
        elif last == "lam":
            w = -2.5 + 1.5 * n                                  # decays from almost nothing kept to almost everything
        elif last == "A_log":
            w = -1.0 + 0.7 * n
        elif last == "dt_bias":
            w = 0.5 * n
        elif name.endswith((".ra.b", ".ri.b", ".y.b", ".x.b", ".conv.b", ".router.b")):
            w = 0.3 * n
        elif last in ("ra", "ri"):
            w = n / np.sqrt(shape[-1])
        elif last == "router":
            w = 2.0 * n / np.sqrt(shape[1])
        elif sharp and name.endswith("right.o"):
            w = 0.0 * n
        elif len(shape) == 2:
            w = n * (3.0 if sharp and last == "q" else 1.0) / np.sqrt(shape[1])
        else:
            w = 0.1 * n
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
        W = make_weights(cfg, zlib.crc32(name.encode()) % 1000, sharp=name == "sharp")      # a seed that stays with the name
        out[name] = (write_model(os.path.join(str(root), name), cfg, W), cfg, as_numpy(W))
    return out
