"""Position encodings that a mixer applies to its queries and keys.

`rope_neox`: rotary embedding in the split-half ("NeoX") pairing, element i
with element i + rotary_dim/2, not the interleaved pairing (mynah-slm
src/kernels.c:173-189; docs/qwen3-arch.md:49-53). Parameters: theta and
rotary_dim (the reference rotates the whole head: rotary_dim = head_dim). The
cos/sin table is built once per (theta, rotary_dim) in double precision and
stored as float, like the reference's (src/kernels.c:141-164), and is shared
by every layer that asks for the same pair.

`rotary`: the general rotary encoding, for mixers that rotate inside kernels of
their own: pairing "half" (i with i + dims/2) or "interleaved" (2i with 2i+1),
over the first `dims` dimensions, frequencies f_i = base^(-2i/dims), and
optionally the interpolation for contexts longer than the trained one
(`scaling`: factor, original, fast, slow): with d(t) = dims ln(original /
(2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)),
dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i
turns at f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are both
multiplied by 0.1 ln(factor) + 1. Frequencies are made in double on the host,
angles in double on the device; the tables are float. A second form of
scaling, `kind: "wavelength"` (factor, low, high, original), goes by each pair's
wavelength l_i = 2 pi / f_i: pairs with l_i < original / high keep f_i, pairs
with l_i > original / low turn at f_i / factor, and between the two, with
s = (original / l_i - low) / (high - low), at (1 - s) f_i / factor + s f_i;
cos and sin keep their size.

`none`: no position encoding (the mixer then only norms and stores).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels
from .base import PositionEncoding, register_position


class RopeNeox(PositionEncoding):
    fusable = True

    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            from ..config.keys import ConfigError
            raise ConfigError(f"rope_neox: rotary_dim {self.rotary_dim} must be positive and even")
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, runtime) -> None:
        key = ("rope_neox", self.theta, self.rotary_dim)
        if key not in runtime.tables:
            runtime.tables[key] = kernels.rope_table(runtime.max_positions, self.rotary_dim, self.theta, runtime.device)
        self.cos, self.sin = runtime.tables[key]

    def fused_tables(self):
        return self.cos, self.sin, self.rotary_dim


def rotary_frequencies(dims: int, base: float, scaling=None) -> tuple[list[float], float]:
    """Per-pair frequencies (double) and the factor on cos and sin."""
    import math
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if scaling.get("kind") == "wavelength":
        low, high = float(scaling["low"]), float(scaling["high"])
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < original / high:
                out.append(fi)
            elif wavelength > original / low:
                out.append(fi / factor)
            else:
                s = (original / wavelength - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        return out, 1.0

    def at(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(at(float(scaling["fast"]))), 0)
    hi = min(math.ceil(at(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


class Rotary(PositionEncoding):
    """Parameters: dims, base, pairing ("half" | "interleaved"), scaling (None, or a mapping with factor,
    original, fast, slow, or one with kind "wavelength", factor, original, low, high)."""
    fusable = True

    def __init__(self, spec):
        super().__init__(spec)
        from ..config.keys import ConfigError
        self.dims = int(spec["dims"])
        self.base = float(spec["base"])
        self.pairing = str(spec.get("pairing", "half"))
        sc = spec.get("scaling")
        self.scaling = None
        if sc and sc.get("kind") == "wavelength":
            self.scaling = {"kind": "wavelength", **{k: float(sc[k]) for k in ("factor", "original", "low", "high")}}
            if self.scaling["low"] == self.scaling["high"]:
                raise ConfigError("rotary: the wavelength scaling's low and high are equal")
        elif sc:
            self.scaling = {k: float(sc[k]) for k in ("factor", "original", "fast", "slow")}
        if self.dims <= 0 or self.dims % 2:
            raise ConfigError(f"rotary: dims {self.dims} must be positive and even")
        if self.pairing not in ("half", "interleaved"):
            raise ConfigError(f"rotary: pairing {self.pairing!r} is neither 'half' nor 'interleaved'")
        if not self.base > 0.0 or (self.scaling and not all(v > 0.0 for v in self.scaling.values() if not isinstance(v, str))):
            raise ConfigError("rotary: base and the scaling's constants must be positive")
        self.interleaved = self.pairing == "interleaved"
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, runtime) -> None:
        key = ("rotary", self.dims, self.base, tuple(sorted(self.scaling.items(), key=lambda kv: kv[0])) if self.scaling else None)
        if key not in runtime.tables:
            freqs, mult = rotary_frequencies(self.dims, self.base, self.scaling)
            runtime.tables[key] = kernels.rope_table_freqs(runtime.max_positions, freqs, mult, runtime.device)
        self.cos, self.sin = runtime.tables[key]

    def fused_tables(self):
        return self.cos, self.sin, self.dims


class NoPosition(PositionEncoding):
    fusable = True

    def fused_tables(self):
        return None, None, 0


register_position("rope_neox", RopeNeox)
register_position("rotary", Rotary)
register_position("none", NoPosition)
