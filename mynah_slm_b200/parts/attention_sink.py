"""Sliding-window softmax attention with a sink, heads whose weights are mixed
after the softmax, and values that carry a rotation of their own.

With h the mixer's input, position i the query's and j a key's:

  q = W_q h (heads x dim),  k = W_k h (kv_heads x dim),  v = W_v h (kv_heads x vdim);  no biases
  q, k rotated over their first rot.dims dimensions (`rot`: dims, base, pairing, scaling)
  v(j) rotated by j over all its vdim dimensions (`value_rot`: base, pairing; None: values stay as they are);
      it is cached rotated
  s_g(i, j) = scale * q_g(i) . k(j)          for 0 <= i - j < window (window None: every earlier key)
  w_g(i, j) = exp(s_g(i, j)) / (exp(sink_g) + sum_j' exp(s_g(i, j')))
  m_h(i, j) = sum_g talk[h, g] w_g(i, j)
  o_h(i)    = R(-i) sum_j m_h(i, j) v(j)     the sum is turned back by the query's position
  out = W_o [o_0 | o_1 | ...]

Query head h reads key/value head h // (heads / kv_heads). The sink has no
key and no value: it only takes its share of the softmax, and that share is
not mixed. Scores, the softmax, the mixing and both rotations are fp32.

Parameters: hidden_size, heads, kv_heads, dim, vdim, scale, window, rot,
value_rot, and the tensors' names q, k, v, o, talk ([heads, heads]), sink
([heads]).
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import kernels
from .base import CacheView, KVRequest, Mixer, TensorSpec, build_part, register_mixer


class SinkTalkAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.H, self.G, self.dim, self.vd = g("hidden_size"), g("heads"), g("kv_heads"), g("dim"), g("vdim")
        self.scale = float(spec["scale"])
        self.window: Optional[int] = spec.get("window")
        self.names = {k: str(spec[k]) for k in ("q", "k", "v", "o", "talk", "sink")}
        if self.H % self.G:
            raise ConfigError(f"sink_talk_attention: {self.H} heads are not a multiple of {self.G} kv heads")
        if max(self.dim, self.vd) > kernels.MAX_HEAD_DIM:
            raise ConfigError(f"sink_talk_attention: heads of {self.dim} / {self.vd} exceed {kernels.MAX_HEAD_DIM}")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"sink_talk_attention: window {self.window} must be positive")
        rot = spec.get("rot")
        self.rot_dims = int(rot["dims"]) if rot else 0
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ConfigError(f"sink_talk_attention: {self.rot_dims} rotated dimensions must be even and at most {self.dim}")
        self.position = build_part("position", PartSpec("rotary", dict(rot))) if self.rot_dims else None
        vrot = spec.get("value_rot")
        self.value_position = None
        if vrot:
            if int(vrot["dims"]) != self.vd or self.vd % 2:
                raise ConfigError("sink_talk_attention: values are rotated over all their dimensions, which must be even")
            self.value_position = build_part("position", PartSpec("rotary", dict(vrot)))
        pairings = {p.pairing for p in (self.position, self.value_position) if p is not None}
        if len(pairings) > 1:
            raise ConfigError("sink_talk_attention: keys and values must pair their dimensions the same way")
        self.interleaved = pairings == {"interleaved"}

    def tensor_specs(self) -> list[TensorSpec]:
        n, H, G, dim, vd, D = self.names, self.H, self.G, self.dim, self.vd, self.D
        return [TensorSpec(n["q"], (H * dim, D)), TensorSpec(n["k"], (G * dim, D)), TensorSpec(n["v"], (G * vd, D)),
                TensorSpec(n["o"], (D, H * vd)),
                TensorSpec(n["talk"], (H, H), role="gain", init="normal", std=0.5),
                TensorSpec(n["sink"], (H,), role="gain", init="normal", std=1.0)]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n = self.names
        parts = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        rows = sum(p.shape[0] for p in parts)
        if rows % 8:
            parts.append(torch.zeros((8 - rows % 8, self.D), dtype=parts[0].dtype, device=parts[0].device))
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        self.talk = tensors[n["talk"]].contiguous()
        self.sink = tensors[n["sink"]].to(self.talk.dtype).contiguous()
        self.runtime = runtime
        self.cos_k = self.sin_k = self.cos_v = self.sin_v = None
        if self.position is not None:
            self.position.prepare(runtime)
            self.cos_k, self.sin_k, _ = self.position.fused_tables()
        if self.value_position is not None:
            self.value_position.prepare(runtime)
            self.cos_v, self.sin_v, _ = self.value_position.fused_tables()

    def streamed_tensors(self) -> list:
        return [self.w_qkv, self.w_o]

    def kv_request(self) -> KVRequest:
        return KVRequest(self.G, self.dim, self.window, v_head_dim=self.vd)

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        H, G, dim, vd = self.H, self.G, self.dim, self.vd
        T = h.shape[0]
        pages = ctx.pages[cache.group]
        writes = cache.writes
        qkv = kernels.linear(h, self.w_qkv if writes else self.w_qkv[: H * dim])
        q = torch.empty((T, H * dim), dtype=qkv.dtype, device=qkv.device)
        kernels.sink_attn_prep(qkv, q, cache.k if writes else None, cache.v if writes else None, self.cos_k, self.sin_k,
                               self.cos_v, self.sin_v, ctx, pages, H, G, dim, vd, self.rot_dims, self.interleaved)
        out = torch.empty((T, H * vd), dtype=qkv.dtype, device=qkv.device)
        if kernels.sink_attn_tc_supported(qkv.dtype, H, G, dim, vd) and cache.k.dtype == torch.bfloat16:
            # a decode step shares a sequence's key tiles among CTAs, one share per page in sight
            in_sight = ctx.decode_splits if self.window is None else min(ctx.decode_splits, (self.window + 126) // 64 + 1)
            splits = max(1, in_sight) if ctx.is_decode else 1
            words = kernels.sink_attn_tc_scratch(T, H, vd, splits)
            scratch = self.runtime.attn_scratch(1, 1, words, 1)
            kernels.sink_attn_tc(q, out, scratch, cache.k, cache.v, self.talk, self.sink, self.cos_v, self.sin_v, ctx, pages,
                                 H, G, dim, vd, self.window or 0, self.scale, self.interleaved, splits)
            return kernels.linear(out, self.w_o, out_dtype=torch.float32)
        kernels.sink_attn(q, out, cache.k, cache.v, self.talk, self.sink, self.cos_v, self.sin_v, ctx, pages, H, G, dim, vd,
                          self.window or 0, self.scale, self.interleaved)
        return kernels.linear(out, self.w_o, out_dtype=torch.float32)      # unrounded into the norm that follows


register_mixer("sink_talk_attention", SinkTalkAttention)
