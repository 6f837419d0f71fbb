"""Typed configuration of the Gomuzen design, read from its config.json.

A small decoder-only model whose layers are listed one by one: `layers[i]`
names the layer's mixer (`type`), the mixer's sizes (`mixer`) and its
feed-forward (`mlp`, or null for none). A range of layers may run several
times in a row with the same weights (`loop`), every pass with a cache of its
own; before every pass, the first too, row t of the tensor `loop.step`
[times, width] is added to the stream, t the number of the pass. Every size and
every constant that can differ between two models of the design is read from
the file; what the design fixes (which mixer pairs rotated dimensions how, the
constant in the experts' gate, two score maps a head in the differential
mixer) lives here and in the parts.

  architecture      "Gomuzen"
  vocab, width, max_positions (optional: the design has no limit, so 2^20 unless given)
  norm.eps          epsilon of every RMS norm (plain gains)
  loop              {start, stop, times} | absent
  layers[i]         {type, mixer: {...}, mlp: {...} | null}
    latent_attention  heads, dim, rot_dim, vdim, kv_rank, scale, rot: {dims, base, scaling?}
                      (one latent a position, an output gate a head; rotated pairs (2i, 2i+1))
    attention         heads, kv_heads, dim, vdim, scale, softcap, diff, rot: {dims, base, scaling?}
                      (two score maps a head over the same values, per-map q/k norm; pairs (i, i + dims/2))
    attention_2       heads, kv_heads, dim, vdim, scale, softcap, rot: {dims, base, scaling?},
                      mask: {size, keep_first} | absent  (biases on q, k, v; pairs (i, i + dims/2))
    mlp               {kind: "moe", expert: {ff, limit}, router: {experts, top, scale, groups: {count, keep} | absent}}

Layer i's tensors start with "l<i>."; the block is pre-norm with two norms
(`norm1`, `norm2`); a norm (`final.norm`) and an untied head (`head`) end the
model.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .keys import ConfigError, opt_int, req_float, req_int, req_str
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Gomuzen"
MIXERS = ("latent_attention", "attention", "attention_2")
GATE_ALPHA = 1.702          # the experts' gate is g * sigmoid(GATE_ALPHA g)


def _obj(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: missing config key: {key} (an object)")
    return v


def _check_rot(rot: Any, limit: int, where: str) -> None:
    if not isinstance(rot, dict):
        raise ConfigError(f"{where}: missing config key: rot (an object)")
    dims = req_int(rot, "dims")
    if dims % 2 or dims > limit:
        raise ConfigError(f"{where}.rot.dims must be even and at most {limit}, got {dims}")
    if not req_float(rot, "base") > 0.0:
        raise ConfigError(f"{where}.rot.base must be > 0")
    if rot.get("scaling") is not None:
        sc = _obj(rot, "scaling", where + ".rot")
        for k in ("factor", "original", "fast", "slow"):
            if not req_float(sc, k) > 0.0:
                raise ConfigError(f"{where}.rot.scaling.{k} must be > 0")


def _rot_spec(rot: Mapping[str, Any], pairing: str) -> dict:
    sc = rot.get("scaling")
    return {"dims": int(rot["dims"]), "base": float(rot["base"]), "pairing": pairing,
            "scaling": {k: float(sc[k]) for k in ("factor", "original", "fast", "slow")} if sc else None}


@dataclass(frozen=True)
class GomuzenConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: tuple                       # of plain dictionaries as in config.json, checked
    loop: Optional[tuple] = None        # (start, stop, times)
    has_max_positions: bool = False

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "GomuzenConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("missing config key: layers (a non-empty list)")
        mp = opt_int(d, "max_positions", None)
        loop = None
        if d.get("loop") is not None:
            lp = _obj(d, "loop", "config")
            loop = (req_int(lp, "start", 0), req_int(lp, "stop", 0), req_int(lp, "times", 1))
        cfg = cls(vocab=req_int(d, "vocab"), width=req_int(d, "width"), max_positions=mp if mp is not None else 1 << 20,
                  norm_eps=req_float(_obj(d, "norm", "config"), "eps"), layers=tuple(copy.deepcopy(layers)), loop=loop,
                  has_max_positions=mp is not None)
        cfg.check()
        return cfg

    def check(self) -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be > 0, got {self.norm_eps}")
        if self.max_positions < 1:
            raise ConfigError(f"max_positions must be >= 1, got {self.max_positions}")
        if self.loop is not None:
            start, stop, _ = self.loop
            if not 0 <= start < stop <= len(self.layers):
                raise ConfigError(f"loop: layers {start}..{stop - 1} do not lie inside the model's {len(self.layers)}")
        for i, L in enumerate(self.layers):
            w = f"layers[{i}]"
            if not isinstance(L, dict):
                raise ConfigError(f"{w} is not an object")
            kind = req_str(L, "type")
            if kind not in MIXERS:
                raise ConfigError(f"{w}.type is {kind!r}; known: {', '.join(MIXERS)}")
            m = _obj(L, "mixer", w)
            wm = w + ".mixer"
            if not req_float(m, "scale") > 0.0:
                raise ConfigError(f"{wm}.scale must be > 0")
            if kind == "latent_attention":
                for k in ("heads", "vdim", "kv_rank", "dim", "rot_dim"):
                    req_int(m, k)
                _check_rot(m.get("rot"), m["rot_dim"], wm)          # the rotated part's first rot.dims dimensions turn
            else:
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    req_int(m, k)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{wm}: heads is not a multiple of kv_heads")
                _check_rot(m.get("rot"), m["dim"], wm)
                if not req_float(m, "softcap") > 0.0:
                    raise ConfigError(f"{wm}.softcap must be > 0")
                if kind == "attention":
                    req_float(m, "diff")
                elif m.get("mask") is not None:
                    mk = _obj(m, "mask", wm)
                    req_int(mk, "size")
                    if (opt_int(mk, "keep_first", 0) or 0) < 0:
                        raise ConfigError(f"{wm}.mask.keep_first must not be negative")
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{w}.mlp is neither null nor an object")
                if req_str(mlp, "kind") != "moe":
                    raise ConfigError(f"{w}.mlp.kind is {mlp['kind']!r}; known: moe")
                ex, ro = _obj(mlp, "expert", w + ".mlp"), _obj(mlp, "router", w + ".mlp")
                req_int(ex, "ff")
                req_float(ex, "limit")
                E, top = req_int(ro, "experts"), req_int(ro, "top")
                req_float(ro, "scale")
                count = keep = 1
                if ro.get("groups") is not None:
                    gr = _obj(ro, "groups", w + ".mlp.router")
                    count, keep = req_int(gr, "count"), req_int(gr, "keep")
                if E % count or keep > count:
                    raise ConfigError(f"{w}.mlp.router: {E} experts do not form {count} equal groups of which {keep} are kept")
                if top > keep * (E // count):
                    raise ConfigError(f"{w}.mlp.router.top exceeds the experts of the kept groups")

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.has_max_positions:
            d["max_positions"] = self.max_positions
        return d

    # ---------------------------------------------------------------- spec
    def runs(self) -> list[tuple[int, Optional[int]]]:
        """(layer, number of the pass that it opens or None) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        out: list[tuple[int, Optional[int]]] = [(i, None) for i in range(start)]
        for t in range(times):
            out += [(i, t if i == start else None) for i in range(start, stop)]
        return out + [(i, None) for i in range(stop, n)]

    def _mixer(self, i: int, L: Mapping[str, Any]) -> PartSpec:
        p = f"l{i}.mix."
        m = L["mixer"]
        if L["type"] == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                "vdim": m["vdim"], "kv_rank": m["kv_rank"], "eps": self.norm_eps, "scale": float(m["scale"]),
                "window": None, "own_kv": True, "rot": _rot_spec(m["rot"], "interleaved"), "gate": p + "g",
                "q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv", "o": p + "o"})
        common = {"hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                  "vdim": m["vdim"], "scale": float(m["scale"]), "eps": self.norm_eps, "softcap": float(m["softcap"]),
                  "rot": _rot_spec(m["rot"], "half"), "q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}
        if L["type"] == "attention":
            return PartSpec("capped_attention", {
                **common, "maps": 2, "diff": float(m["diff"]), "qk_norm": True, "q_norm": p + "q.norm", "k_norm": p + "k.norm",
                "lq1": p + "lq1", "lk1": p + "lk1", "lq2": p + "lq2", "lk2": p + "lk2"})
        mask = m.get("mask")
        return PartSpec("capped_attention", {
            **common, "bias": True, "q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b",
            "window": mask["size"] if mask else None, "keep_first": (mask.get("keep_first") or 0) if mask else 0})

    def _ffn(self, i: int, mlp: Mapping[str, Any]) -> PartSpec:
        p = f"l{i}.mlp."
        ro = mlp["router"]
        gr = ro.get("groups") or {"count": 1, "keep": 1}
        return PartSpec("group_router_experts", {
            "hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"], "experts": ro["experts"], "top": ro["top"],
            "groups": gr["count"], "keep": gr["keep"], "weight_scale": float(ro["scale"]),
            "limit": float(mlp["expert"]["limit"]), "alpha": GATE_ALPHA,
            "router": p + "router", "correction": p + "correction", "expert_prefix": p + "e"})

    def model_spec(self) -> ModelSpec:
        layers = []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            norm = lambda name: PartSpec("rmsnorm", {"eps": self.norm_eps, "dim": self.width, "name": name})
            mlp = L.get("mlp")
            norms = {"mixer": norm(p + "norm1")}
            if mlp is not None:
                norms["ffn"] = norm(p + "norm2")
            layers.append(LayerSpec(block=PartSpec("prenorm_residual", {}), mixer=self._mixer(i, L),
                                    ffn=self._ffn(i, mlp) if mlp is not None else None, norms=norms, prefix=p))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=self.max_positions,
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, add_vector=t) for i, t in self.runs()),
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": self.vocab, "dim": self.width}),
            final_norm=PartSpec("rmsnorm", {"eps": self.norm_eps, "dim": self.width, "name": "final.norm"}),
            head=PartSpec("linear_head", {"tied": False, "name": "head", "vocab_size": self.vocab, "dim": self.width}),
            stream_vectors=(PartSpec("stream_vectors", {"name": "loop.step", "count": self.loop[2], "dim": self.width})
                            if self.loop is not None else None))
        spec.validate()
        return spec
