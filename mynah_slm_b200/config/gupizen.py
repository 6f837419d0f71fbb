"""Typed configuration of the Gupizen design, read from its config.json.

A small decoder-only model whose layers are listed one by one: `layers[i]`
names the layer's mixer (`type`: "parallel" or "channel_delta"), the mixer's
sizes (`mixer`) and its feed-forward (`mlp`, or null for none). A range of
layers may run several times in a row with the same weights (`loop`), every
pass with cache and state of its own, the embedding's output being added to
the stream again before every pass but the first. Every size and every
constant that can differ between two models of the design is read from the
file; what the design fixes (the -8 of the recurrent unit's decay, the epsilon
of the delta rule's unit vectors, the activations) lives in the parts.

  architecture    "Gupizen"
  vocab, width, max_positions (optional)
  norm.eps        epsilon of every RMS norm
  canon.taps      taps of the causal convolution on every sublayer's input
  embedding.scale factor on the token embedding
  loop            {start, stop, times} | absent
  layers[i]       {type, mixer: {...}, mlp: {kind: "moe", expert: {ff}, router: {experts, top}} | null}
    parallel      left:  heads, kv_heads, dim, vdim, scale, mask: {size},
                         rot: {dims, base, scaling: {factor, low, high, original} | absent}
                  right: width, blocks, conv
    channel_delta heads, kv_heads, dim, vdim, conv; decay_rank and gate_rank (optional: the narrow sizes of the
                  decay's and the gate's two-step projections, which otherwise the checkpoint's tensors give)

Layer i's tensors start with "l<i>."; every sublayer sits between two RMS norms
whose gains are stored around zero (`sandwich_residual`); the head is the
embedding matrix itself, without the embedding's factor.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .keys import ConfigError, opt_int, req_float, req_int, req_str
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Gupizen"
MIXERS = ("parallel", "channel_delta")
LRU_DECAY_SCALE = 8.0        # log a = -LRU_DECAY_SCALE * r * softplus(lam)


def _obj(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: missing config key: {key} (an object)")
    return v


@dataclass(frozen=True)
class GupizenConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    canon_taps: int
    embedding_scale: float
    layers: tuple                       # of plain dictionaries as in config.json, checked
    loop: Optional[tuple] = None        # (start, stop, times)
    has_max_positions: bool = False

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "GupizenConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("missing config key: layers (a non-empty list)")
        mp = opt_int(d, "max_positions", None)
        loop = None
        if d.get("loop") is not None:
            lp = _obj(d, "loop", "config")
            loop = (req_int(lp, "start", 0), req_int(lp, "stop", 0), req_int(lp, "times", 1))
        cfg = cls(vocab=req_int(d, "vocab"), width=req_int(d, "width"), max_positions=mp if mp is not None else 1 << 20,
                  norm_eps=req_float(_obj(d, "norm", "config"), "eps"),
                  canon_taps=req_int(_obj(d, "canon", "config"), "taps"),
                  embedding_scale=req_float(_obj(d, "embedding", "config"), "scale"),
                  layers=tuple(copy.deepcopy(layers)), loop=loop, has_max_positions=mp is not None)
        cfg.check()
        return cfg

    def check(self) -> None:
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be > 0, got {self.norm_eps}")
        if self.max_positions < 1:
            raise ConfigError(f"max_positions must be >= 1, got {self.max_positions}")
        if self.loop is not None:
            start, stop, times = self.loop
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
            if kind == "parallel":
                a, r = _obj(m, "left", w + ".mixer"), _obj(m, "right", w + ".mixer")
                wa = w + ".mixer.left"
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    req_int(a, k)
                req_float(a, "scale")
                if a["heads"] % a["kv_heads"]:
                    raise ConfigError(f"{wa}: heads is not a multiple of kv_heads")
                if a["vdim"] % 2:
                    raise ConfigError(f"{wa}.vdim must be even (values are rotated pair by pair), got {a['vdim']}")
                req_int(_obj(a, "mask", wa), "size")
                rot = _obj(a, "rot", wa)
                dims = req_int(rot, "dims")
                if dims % 2 or dims > a["dim"]:
                    raise ConfigError(f"{wa}.rot.dims must be even and at most dim, got {dims}")
                if not req_float(rot, "base") > 0.0:
                    raise ConfigError(f"{wa}.rot.base must be > 0")
                if rot.get("scaling") is not None:
                    sc = _obj(rot, "scaling", wa + ".rot")
                    for k in ("factor", "low", "high", "original"):
                        if not req_float(sc, k) > 0.0:
                            raise ConfigError(f"{wa}.rot.scaling.{k} must be > 0")
                    if sc["high"] == sc["low"]:
                        raise ConfigError(f"{wa}.rot.scaling: high equals low")
                for k in ("width", "blocks", "conv"):
                    req_int(r, k)
                if r["width"] % r["blocks"]:
                    raise ConfigError(f"{w}.mixer.right: width is not a multiple of blocks")
            else:
                for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    req_int(m, k)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"{w}.mixer: heads is not a multiple of kv_heads")
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise ConfigError(f"{w}.mlp is neither null nor an object")
                if req_str(mlp, "kind") != "moe":
                    raise ConfigError(f"{w}.mlp.kind is {mlp['kind']!r}; known: moe")
                req_int(_obj(mlp, "expert", w + ".mlp"), "ff")
                ro = _obj(mlp, "router", w + ".mlp")
                if req_int(ro, "top") > req_int(ro, "experts"):
                    raise ConfigError(f"{w}.mlp.router: top exceeds experts")

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "canon": {"taps": self.canon_taps}, "embedding": {"scale": self.embedding_scale},
             "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.has_max_positions:
            d["max_positions"] = self.max_positions
        return d

    # ---------------------------------------------------------------- spec
    def runs(self) -> list[tuple[int, bool]]:
        """(layer, the embedding's output is added before it) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        out = [(i, False) for i in range(start)]
        for p in range(times):
            out += [(i, p > 0 and i == start) for i in range(start, stop)]
        return out + [(i, False) for i in range(stop, n)]

    def _mixer(self, i: int, L: Mapping[str, Any]) -> PartSpec:
        p = f"l{i}.mix."
        m = L["mixer"]
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            rot = a["rot"]
            sc = rot.get("scaling")
            pl, pr = p + "left.", p + "right."
            left = PartSpec("sink_talk_attention", {
                "hidden_size": self.width, "heads": a["heads"], "kv_heads": a["kv_heads"], "dim": a["dim"],
                "vdim": a["vdim"], "scale": float(a["scale"]), "window": a["mask"]["size"],
                "rot": {"dims": rot["dims"], "base": float(rot["base"]), "pairing": "interleaved",
                        "scaling": ({"kind": "wavelength", **{k: float(sc[k]) for k in ("factor", "low", "high", "original")}}
                                    if sc else None)},
                "value_rot": {"dims": a["vdim"], "base": float(rot["base"]), "pairing": "interleaved", "scaling": None},
                "q": pl + "q", "k": pl + "k", "v": pl + "v", "o": pl + "o", "talk": pl + "talk", "sink": pl + "sink"})
            right = PartSpec("rglru", {
                "hidden_size": self.width, "width": r["width"], "blocks": r["blocks"], "conv": r["conv"],
                "decay_scale": LRU_DECAY_SCALE,
                "y": pr + "y", "y_bias": pr + "y.b", "x": pr + "x", "x_bias": pr + "x.b", "conv_name": pr + "conv",
                "conv_bias": pr + "conv.b", "ra": pr + "ra", "ra_bias": pr + "ra.b", "ri": pr + "ri",
                "ri_bias": pr + "ri.b", "lam": pr + "lam", "o": pr + "o"})
            return PartSpec("parallel_mixers", {
                "hidden_size": self.width, "eps": self.norm_eps, "branches": (left, right),
                "out_norms": (pl + "out", pr + "out"), "weight": 0.5})
        return PartSpec("gated_delta", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
            "vdim": m["vdim"], "conv": m["conv"], "eps": self.norm_eps, "decay": "channel", "gate_act": "sigmoid",
            "a_rank": m.get("decay_rank"), "g_rank": m.get("gate_rank"),
            "q": p + "q", "k": p + "k", "v": p + "v", "q_conv": p + "q.conv", "k_conv": p + "k.conv",
            "v_conv": p + "v.conv", "b": p + "b", "a": p + "a2", "a_in": p + "a1", "A_log": p + "A_log",
            "dt_bias": p + "dt_bias", "g": p + "g2", "g_in": p + "g1", "norm": p + "norm", "o": p + "o"})

    def model_spec(self) -> ModelSpec:
        layers = []
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            nm = lambda name: PartSpec("rmsnorm_offset", {"eps": self.norm_eps, "dim": self.width, "name": p + name})
            mlp = L.get("mlp")
            ffn = None
            norms = {"mixer": nm("norm1"), "mixer_out": nm("norm1b")}
            if mlp is not None:
                ffn = PartSpec("router_experts", {
                    "hidden_size": self.width, "intermediate_size": mlp["expert"]["ff"],
                    "experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "activation": "gelu_erf",
                    "router": p + "mlp.router", "router_bias": p + "mlp.router.b", "expert_prefix": p + "mlp.e"})
                norms["ffn"] = nm("norm2")
                norms["ffn_out"] = nm("norm2b")
            layers.append(LayerSpec(
                block=PartSpec("sandwich_residual", {"hidden_size": self.width, "input_conv_taps": self.canon_taps,
                                                     "mixer_conv_name": p + "canon1", "ffn_conv_name": p + "canon2"}),
                mixer=self._mixer(i, L), ffn=ffn, norms=norms, prefix=p))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=self.max_positions,
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, add_embedding=add) for i, add in self.runs()),
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": self.vocab, "dim": self.width,
                                                   "scale": self.embedding_scale}),
            final_norm=PartSpec("rmsnorm_offset", {"eps": self.norm_eps, "dim": self.width, "name": "final.norm"}),
            head=PartSpec("linear_head", {"tied": True, "name": "head", "vocab_size": self.vocab, "dim": self.width}))
        spec.validate()
        return spec
