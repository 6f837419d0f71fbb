"""Grouped-query softmax attention with the options that several designs combine differently: biases on the
projections, an RMS norm per head with one gain for all heads, a rotation over part of each head with any table
of the `rotary` position part, scores squashed by a cap, a window that keeps a sequence's first tokens, and heads
that hold two score maps over the same values ("differential" attention).

Per token, with h the mixer's input, H query heads, G kv heads (query head n reads kv head n // (H / G)), M maps a
head (1 or 2), `dim` values a map and `vdim` a value head:

  q = W_q h (+ b_q)   [H, M, dim]      k = W_k h (+ b_k)   [G, M, dim]      v = W_v h (+ b_v)   [G, vdim]
  qk_norm:   every [dim] of q and k <- x / sqrt(mean(x^2) + eps) * gain      (one gain for q, one for k)
  rot:       the first rot.dims of every [dim] of q and k turned by the position's angles
  score_m(i, j) = q_m(i) . k_m(j) * scale;   softcap c:  score <- c tanh(score / c)
  visible:   j <= i, and with window W:  i - j < W  or  j < keep_first
  a_m = softmax_j(score_m) v
  M = 1:  o = a_0
  M = 2:  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff  (one number a layer);
          o = (a_0 - lambda a_1) / sqrt(mean((a_0 - lambda a_1)^2) + eps) * (1 - diff)   over the head's vdim values
  out = W_o on the concatenated heads

Norm, rotation, scores, softmax, the combination of the maps and its norm are fp32 (`csrc/capped_attn.cu`, the
attention kernels). The cache holds G * M key heads and G value heads a position; a query map and its key map meet
through the kernels' own head grouping (the packed query row is ordered kv head, map, query head of the group),
and key head g * M + m reads value head g.

A window with kept first tokens keeps every page (the pages between the first tokens and the window are not
given back); a window alone frees pages as the other windowed mixers do.

Parameters: hidden_size, heads, kv_heads, dim, vdim, scale, eps, maps (1), diff (with maps = 2), softcap (None),
window (None), keep_first (0), qk_norm (False), bias (False), rot (None or the parameters of a `rotary` part), and
the tensors' names: q, k, v, o; q_bias, k_bias, v_bias; q_norm, k_norm; lq1, lk1, lq2, lk2.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import attention_dispatch, kernels
from .base import CacheView, KVRequest, Mixer, TensorSpec, build_part, register_mixer


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class CappedAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.H, self.G, self.dim, self.vd = g("hidden_size"), g("heads"), g("kv_heads"), g("dim"), g("vdim")
        self.M = int(spec.get("maps", 1))
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.softcap = float(spec.get("softcap") or 0.0)
        self.window: Optional[int] = spec.get("window")
        self.keep_first = int(spec.get("keep_first") or 0)
        self.qk_norm, self.bias = bool(spec.get("qk_norm", False)), bool(spec.get("bias", False))
        self.diff = float(spec.get("diff", 0.0))
        if self.M not in (1, 2):
            raise ConfigError(f"capped_attention: {self.M} maps a head (1 or 2)")
        if self.H % self.G:
            raise ConfigError(f"capped_attention: {self.H} heads are not a multiple of {self.G} kv heads")
        self.R = self.H // self.G
        self.dimp, self.vdp = _pad8(self.dim), _pad8(self.vd)
        if max(self.dimp, self.vdp) > kernels.MAX_HEAD_DIM:
            raise ConfigError(f"capped_attention: heads of {self.dim} / {self.vd} exceed {kernels.MAX_HEAD_DIM}")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"capped_attention: window {self.window} must be positive")
        if self.keep_first < 0 or self.softcap < 0.0 or not self.scale > 0.0:
            raise ConfigError("capped_attention: keep_first and softcap must not be negative, scale must be positive")
        names = ["q", "k", "v", "o"] + (["q_bias", "k_bias", "v_bias"] if self.bias else []) \
            + (["q_norm", "k_norm"] if self.qk_norm else []) + (["lq1", "lk1", "lq2", "lk2"] if self.M == 2 else [])
        self.names = {k: str(spec[k]) for k in names}
        rot = spec.get("rot")
        self.position = build_part("position", PartSpec("rotary", dict(rot))) if rot else None
        if self.position is not None and self.position.dims > self.dim:
            raise ConfigError(f"capped_attention: {self.position.dims} rotated dims exceed the head's {self.dim}")

    def tensor_specs(self) -> list[TensorSpec]:
        n, H, G, M, dim, vd, D = self.names, self.H, self.G, self.M, self.dim, self.vd, self.D
        specs = [TensorSpec(n["q"], (H * M * dim, D)), TensorSpec(n["k"], (G * M * dim, D)), TensorSpec(n["v"], (G * vd, D)),
                 TensorSpec(n["o"], (D, H * vd))]
        if self.bias:
            specs += [TensorSpec(n["q_bias"], (H * M * dim,), role="gain", init="normal", std=0.1),
                      TensorSpec(n["k_bias"], (G * M * dim,), role="gain", init="normal", std=0.1),
                      TensorSpec(n["v_bias"], (G * vd,), role="gain", init="normal", std=0.1)]
        if self.qk_norm:
            specs += [TensorSpec(n["q_norm"], (dim,), role="gain", init="gain", std=0.1),
                      TensorSpec(n["k_norm"], (dim,), role="gain", init="gain", std=0.1)]
        if M == 2:
            specs += [TensorSpec(n[k], (dim,), role="gain", init="normal", std=0.1) for k in ("lq1", "lk1", "lq2", "lk2")]
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n = self.names
        self.n_q = tensors[n["q"]].shape[0]
        self.w_qkv = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        self.b_qkv = (torch.cat([tensors[n[k]].to(torch.float32) for k in ("q_bias", "k_bias", "v_bias")]).contiguous()
                      if self.bias else None)
        w_o = tensors[n["o"]]
        if self.M == 1 and self.vdp != self.vd:            # the attention's rows carry padded heads: zero columns for them
            padded = torch.zeros((self.D, self.H, self.vdp), dtype=w_o.dtype, device=w_o.device)
            padded[:, :, : self.vd] = w_o.view(self.D, self.H, self.vd)
            w_o = padded.view(self.D, self.H * self.vdp).contiguous()
        self.w_o = w_o
        self.q_gain = tensors[n["q_norm"]] if self.qk_norm else None
        self.k_gain = tensors[n["k_norm"]].to(self.q_gain.dtype) if self.qk_norm else None
        self.lam = 0.0
        if self.M == 2:
            dot = lambda a, b: float((tensors[n[a]].double() * tensors[n[b]].double()).sum().item())
            self.lam = math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + self.diff
        self.cos = self.sin = None
        self.rot, self.interleaved = 0, False
        if self.position is not None:
            self.position.prepare(runtime)
            self.cos, self.sin, self.rot = self.position.fused_tables()
            self.interleaved = self.position.interleaved
        self.runtime = runtime

    def streamed_tensors(self) -> list:
        return [self.w_qkv, self.w_o]

    def kv_request(self) -> KVRequest:
        frees = self.window if not self.keep_first else None
        return KVRequest(self.G * self.M, self.dimp, frees, v_head_dim=self.vdp, v_heads=self.G)

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        H, G, M, dimp, vdp = self.H, self.G, self.M, self.dimp, self.vdp
        T = h.shape[0]
        writes = cache.writes
        pages = ctx.pages[cache.group]
        qkv = kernels.linear(h, self.w_qkv if writes else self.w_qkv[: self.n_q])
        q = torch.empty((T, H * M * dimp), dtype=qkv.dtype, device=qkv.device)
        kernels.capped_attn_prep(qkv, q, H * M, G * M, G, self.dim, self.vd, dimp, vdp, M, self.R, self.b_qkv, self.q_gain,
                                 self.k_gain, self.eps, self.cos, self.sin, self.rot, self.interleaved, ctx, pages,
                                 cache.k if writes else None, cache.v if writes else None)
        a = torch.empty((T, H * M * vdp), dtype=qkv.dtype, device=qkv.device)
        if ctx.is_decode:
            attention_dispatch.decode_capped(q, a, ctx, H * M, G * M, dimp, vdp, cache.k, cache.v, pages, self.window or 0,
                                             self.scale, self.softcap, self.keep_first, M,
                                             self.runtime.attn_scratch(ctx.B, H * M, vdp, ctx.decode_splits))
        else:
            attention_dispatch.prefill_capped(q, a, ctx, H * M, G * M, dimp, vdp, cache.k, cache.v, pages, self.window or 0,
                                              self.scale, self.softcap, self.keep_first, M)
        if M == 2:
            a = kernels.diff_combine(a, H, self.R, self.vd, vdp, self.lam, 1.0 - self.diff, self.eps, ctx)
        return kernels.linear(a, self.w_o)


register_mixer("capped_attention", CappedAttention)
