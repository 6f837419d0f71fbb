"""Gated delta rule mixer: linear attention whose state is corrected towards
each new value along its key, with a learned per-head decay.

With h the mixer's input (`csrc/delta_rule.cu` states the formulas):

  q = W_q h, k = W_k h   (kv_heads x dim),   v = W_v h   (heads x vdim);   no biases
  each passes a short causal convolution per channel (no bias) and silu
  q, k <- unit vectors per head, x / sqrt(sum(x^2) + 1e-6);   q <- q * dim^(-1/2)
  beta = sigmoid(W_b h);   g = exp(-exp(A_log) * softplus(W_a h + dt_bias))      one each per head
  per head:   S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
  out = W_o (o / rms(o over vdim) * norm_w * silu(W_g h))

Head h reads q/k head h // (heads / kv_heads). S (fp32, [heads, dim, vdim]) and
the convolutions' last taps-1 inputs are the sequence's state.

Variants, chosen by parameters:
  decay "channel"   one decay a head AND key channel: W_a has heads x dim rows, dt_bias heads x dim values
                    (A_log stays one a head), and g multiplies the rows of S: S <- diag(g) S
  gate_act          "silu" (default) or "sigmoid"
  a_in, g_in        names of a first, narrow matrix: the decay's input is then W_a (W_a_in h) and the gate's
                    W_g (W_g_in h). The narrow size is `a_rank` / `g_rank` when given, else whatever the
                    checkpoint's tensors have (the two matrices of a pair must agree)

The six projections of h run as one product (their matrices stacked at bind
time, padded to a multiple of 8 rows), the three convolutions as one launch over
the stacked channels.

Parameters: hidden_size, heads, kv_heads, dim, vdim, conv (taps), eps, decay,
gate_act, a_rank, g_rank, and the tensors' names: q, k, v, q_conv, k_conv,
v_conv, b, a, A_log, dt_bias, g, norm, o, and optionally a_in, g_in.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import kernels
from .base import CacheView, Mixer, StateRequest, TensorSpec, register_mixer

_NAMES = ("q", "k", "v", "q_conv", "k_conv", "v_conv", "b", "a", "A_log", "dt_bias", "g", "norm", "o")


class GatedDelta(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.H, self.G, self.dim, self.vd, self.taps = (g("hidden_size"), g("heads"), g("kv_heads"), g("dim"),
                                                               g("vdim"), g("conv"))
        self.eps = float(spec["eps"])
        self.names = {k: str(spec[k]) for k in _NAMES}
        for k in ("a_in", "g_in"):
            self.names[k] = str(spec[k]) if spec.get(k) else None
        self.channel_decay = spec.get("decay", "head") == "channel"
        self.gate_act = str(spec.get("gate_act", "silu"))
        rank = lambda k: -1 if spec.get(k) in (None, "from_checkpoint") else int(spec[k])
        self.a_rank, self.g_rank = rank("a_rank"), rank("g_rank")
        if spec.get("decay", "head") not in ("head", "channel"):
            raise ConfigError(f"gated_delta: decay {spec.get('decay')!r} is neither 'head' nor 'channel'")
        if self.gate_act not in ("silu", "sigmoid"):
            raise ConfigError(f"gated_delta: gate activation {self.gate_act!r} is neither 'silu' nor 'sigmoid'")
        if self.H % self.G:
            raise ConfigError(f"gated_delta: {self.H} heads are not a multiple of {self.G} q/k heads")
        if self.dim > 512:
            raise ConfigError(f"gated_delta: keys of {self.dim} values exceed the 512 that the recurrence kernel stages")
        if self.channel_decay != bool(self.names["a_in"]):
            raise ConfigError("gated_delta: a decay per channel, and only that, is built from a narrow projection (a_in)")
        self.n_qk = 2 * self.G * self.dim
        self.n_conv = self.n_qk + self.H * self.vd
        self.n_decay = self.H * self.dim if self.channel_decay else self.H

    def tensor_specs(self) -> list[TensorSpec]:
        n, D, H, G, dim, vd, t = self.names, self.D, self.H, self.G, self.dim, self.vd, self.taps
        specs = [TensorSpec(n["q"], (G * dim, D)), TensorSpec(n["k"], (G * dim, D)), TensorSpec(n["v"], (H * vd, D)),
                 TensorSpec(n["q_conv"], (G * dim, t), init="normal", std=0.3),
                 TensorSpec(n["k_conv"], (G * dim, t), init="normal", std=0.3),
                 TensorSpec(n["v_conv"], (H * vd, t), init="normal", std=0.3),
                 TensorSpec(n["b"], (H, D)),
                 TensorSpec(n["A_log"], (H,), role="gain", init="normal", std=0.5),
                 TensorSpec(n["dt_bias"], (self.n_decay,), role="gain", init="normal", std=0.5),
                 TensorSpec(n["norm"], (vd,), role="gain", init="gain", std=0.1),
                 TensorSpec(n["o"], (D, H * vd))]
        if n["a_in"]:
            specs += [TensorSpec(n["a_in"], (self.a_rank, D), free_size=16), TensorSpec(n["a"], (self.n_decay, self.a_rank), std=0.2, free_size=16)]
        else:
            specs.append(TensorSpec(n["a"], (self.n_decay, D)))
        if n["g_in"]:
            specs += [TensorSpec(n["g_in"], (self.g_rank, D), free_size=16), TensorSpec(n["g"], (H * vd, self.g_rank), std=0.2, free_size=16)]
        else:
            specs.append(TensorSpec(n["g"], (H * vd, D)))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n = self.names
        # the projections of h, stacked: q, k, v, then the gate's (or its narrow matrix), beta's, the decay's (or its
        # narrow matrix); every piece starts at a multiple of 8 rows, so that a column slice of the product is aligned
        pieces = [("qkv", torch.cat([tensors[n[k]] for k in ("q", "k", "v")], dim=0)),
                  ("g", tensors[n["g_in"] or n["g"]]), ("b", tensors[n["b"]]), ("a", tensors[n["a_in"] or n["a"]])]
        self.at: dict[str, tuple[int, int]] = {}
        parts, row = [], 0
        for name, w in pieces:
            self.at[name] = (row, row + w.shape[0])
            parts.append(w)
            row += w.shape[0]
            if row % 8:
                parts.append(torch.zeros((8 - row % 8, self.D), dtype=w.dtype, device=w.device))
                row += 8 - row % 8
        self.w_all = torch.cat(parts, dim=0).contiguous()
        self.w_a = self.w_g = None
        if n["a_in"]:
            if tensors[n["a"]].shape[1] != tensors[n["a_in"]].shape[0]:
                raise ConfigError(f"gated_delta: {n['a_in']} and {n['a']} do not agree on the narrow size")
            self.w_a = tensors[n["a"]].contiguous()
        if n["g_in"]:
            if tensors[n["g"]].shape[1] != tensors[n["g_in"]].shape[0]:
                raise ConfigError(f"gated_delta: {n['g_in']} and {n['g']} do not agree on the narrow size")
            self.w_g = tensors[n["g"]].contiguous()
        self.conv_w = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0).contiguous()
        self.A_log = tensors[n["A_log"]]
        self.dt_bias = tensors[n["dt_bias"]].to(self.A_log.dtype)
        self.norm_w = tensors[n["norm"]]
        self.w_o = tensors[n["o"]]
        self.act_dtype = runtime.act_dtype

    def streamed_tensors(self) -> list:
        return [t for t in (self.w_all, self.w_a, self.w_g, self.w_o) if t is not None]

    def state_request(self):
        req = {"S": StateRequest((self.H, self.dim, self.vd), torch.float32)}
        if self.taps > 1:
            req["conv"] = StateRequest((self.taps - 1, self.n_conv), torch.float32)
        return req

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        H, G, dim, vd = self.H, self.G, self.dim, self.vd
        p = kernels.linear(h, self.w_all)
        col = lambda name: p[:, self.at[name][0]: self.at[name][1]]
        qkv = kernels.causal_conv(col("qkv"), self.conv_w, None, cache.state.get("conv"), ctx, self.act_dtype, act="silu")
        gate = col("g") if self.w_g is None else kernels.linear(col("g"), self.w_g)
        if self.w_a is None:
            qn, kn, g, beta = kernels.delta_prep(qkv[:, : self.n_qk], col("a"), col("b"), self.A_log, self.dt_bias, H, G, dim)
        else:
            a = kernels.linear(col("a"), self.w_a, out_dtype=torch.float32)       # the decay's input is not rounded
            qn, kn, g, beta = kernels.delta_prep(qkv[:, : self.n_qk], None, col("b"), self.A_log, self.dt_bias, H, G, dim,
                                                 a_channels=a)
        o = kernels.delta_rule(qn, kn, qkv[:, self.n_qk:], g, beta, cache.state["S"], ctx, H, G, dim, vd,
                               channel_decay=self.channel_decay)
        out = kernels.gated_rmsnorm(o, gate, self.norm_w, H, vd, self.eps, gate_act=self.gate_act)
        return kernels.linear(out, self.w_o, out_dtype=torch.float32)      # unrounded into the norm that follows


register_mixer("gated_delta", GatedDelta)
