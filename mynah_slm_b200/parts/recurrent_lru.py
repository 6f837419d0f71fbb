"""Recurrent block with a real-gated linear recurrent unit (the recurrent
block of Griffin: De, Smith, Fernando et al., "Griffin: Mixing Gated Linear
Recurrences with Local Attention for Efficient Language Models", 2024).

With h the mixer's input and W = `width` channels:

  y = gelu_tanh(W_y h + b_y)                        the gate branch
  u = conv(W_x h + b_x)                             causal convolution per channel, with bias, no activation
  the channels are cut into `blocks` equal parts; in part p, with square matrices Ra_p, Ri_p [out, in]:
      r = sigmoid(Ra_p u_p + ba_p),   i = sigmoid(Ri_p u_p + bi_p)
  log a = -c r softplus(lam),   a = exp(log a)      c = `decay_scale`
  S_t = a S_(t-1) + sqrt(1 - a^2) (i u)             from S = 0, the first token included
  out = W_o (S y)

S (fp32, [W]) and the convolution's last taps-1 inputs (fp32) are the
sequence's state. The gates, the decay and the recurrence are fp32
(`csrc/rglru.cu`); the two projections of h run as one product.

Parameters: hidden_size, width, blocks, conv (taps), decay_scale, and the
tensors' names: y, y_bias, x, x_bias, conv_name, conv_bias, ra, ra_bias, ri,
ri_bias, lam, o.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import kernels
from .base import CacheView, Mixer, StateRequest, TensorSpec, register_mixer

_NAMES = ("y", "y_bias", "x", "x_bias", "conv_name", "conv_bias", "ra", "ra_bias", "ri", "ri_bias", "lam", "o")


class RecurrentLRU(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.W, self.blocks, self.taps = g("hidden_size"), g("width"), g("blocks"), g("conv")
        self.decay_scale = float(spec["decay_scale"])
        self.names = {k: str(spec[k]) for k in _NAMES}
        if self.blocks < 1 or self.W % self.blocks:
            raise ConfigError(f"rglru: {self.W} channels do not split into {self.blocks} equal parts")
        if self.taps < 1:
            raise ConfigError(f"rglru: a convolution of {self.taps} taps does not exist")
        self.bw = self.W // self.blocks

    def tensor_specs(self) -> list[TensorSpec]:
        n, D, W, B, bw = self.names, self.D, self.W, self.blocks, self.bw
        vec = lambda name, std: TensorSpec(n[name], (W,), role="gain", init="normal", std=std)
        return [TensorSpec(n["y"], (W, D)), vec("y_bias", 0.1), TensorSpec(n["x"], (W, D)), vec("x_bias", 0.1),
                TensorSpec(n["conv_name"], (W, self.taps), init="normal", std=0.3), vec("conv_bias", 0.1),
                TensorSpec(n["ra"], (B, bw, bw), std=0.2), TensorSpec(n["ra_bias"], (B, bw), role="gain", init="normal", std=0.5),
                TensorSpec(n["ri"], (B, bw, bw), std=0.2), TensorSpec(n["ri_bias"], (B, bw), role="gain", init="normal", std=0.5),
                vec("lam", 1.0), TensorSpec(n["o"], (D, W))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n, W = self.names, self.W
        parts = [tensors[n["y"]]]
        self.x_off = (W + 7) // 8 * 8                     # the second projection's columns start aligned
        if self.x_off != W:
            parts.append(torch.zeros((self.x_off - W, self.D), dtype=parts[0].dtype, device=parts[0].device))
        parts.append(tensors[n["x"]])
        rows = self.x_off + W
        if rows % 8:
            parts.append(torch.zeros((8 - rows % 8, self.D), dtype=parts[0].dtype, device=parts[0].device))
        self.w_yx = torch.cat(parts, dim=0).contiguous()
        vt = tensors[n["lam"]].dtype
        self.b_y, self.b_x = tensors[n["y_bias"]].to(vt).contiguous(), tensors[n["x_bias"]].to(vt).contiguous()
        self.conv_w = tensors[n["conv_name"]].contiguous()
        self.conv_b = tensors[n["conv_bias"]].to(self.conv_w.dtype).contiguous()
        self.ra, self.ri = tensors[n["ra"]].contiguous(), tensors[n["ri"]].contiguous()
        self.ba = tensors[n["ra_bias"]].to(vt).reshape(-1).contiguous()
        self.bi = tensors[n["ri_bias"]].to(vt).reshape(-1).contiguous()
        self.lam = tensors[n["lam"]].contiguous()
        self.w_o = tensors[n["o"]]

    def streamed_tensors(self) -> list:
        return [self.w_yx, self.ra, self.ri, self.w_o]

    def state_request(self):
        req = {"S": StateRequest((self.W,), torch.float32)}
        if self.taps > 1:
            req["conv"] = StateRequest((self.taps - 1, self.W), torch.float32)
        return req

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        p = kernels.linear(h, self.w_yx)
        y, x = kernels.rglru_in(p, 0, self.x_off, self.W, self.b_y, self.b_x)
        u = kernels.causal_conv(x, self.conv_w, self.conv_b, cache.state.get("conv"), ctx, torch.float32)
        a, b = kernels.rglru_gates(u, self.ra, self.ri, self.ba, self.bi, self.lam, self.decay_scale)
        out = kernels.rglru_scan(a, b, y, cache.state["S"], ctx)
        return kernels.linear(out, self.w_o, out_dtype=torch.float32)      # unrounded into the norm that follows


register_mixer("rglru", RecurrentLRU)
