"""Softmax attention over one latent vector per position: every head's keys and
values are linear maps of the latent, and one rotated key part is shared by all
heads. Only the latent and that part are cached.

With h the mixer's input, H heads, per head `dim` unrotated and `rot_dim`
rotated query/key dimensions, values of `vdim`, a latent of `kv_rank`:

  q = W_q h                      per head [dim unrotated | rot_dim rotated]
  d = W_dkv h                    kv_rank + rot_dim outputs
  c = rms_norm(d[:kv_rank]) * w  (plain weight)      k_r = d[kv_rank:]     (not normed)
  q_r (every head) and k_r are rotated (the position part's pairing, tables and scaling)
  per head:  k_u = W_uk c,  v = W_uv c,  score = (q_u . k_u + q_r . k_r) * scale
  causal softmax (within `window` when given), W_o on the concatenated heads
  with `gate` (a tensor name): head h's output is multiplied by sigmoid(W_g h)_h first; W_g [H, hidden] reads the
  same input as the projections

The maps move to the query side (`csrc/latent_attn.cu`): q_a = W_uk^T q_u per
head, the cache row of a position is [c | k_r] for ONE kv head, the library's
attention kernels run with that row as key and as value, and W_uv maps the
first kv_rank columns of their output to the head's values. A run that reads
another run's cache (`cache_from` in the schedule) has no W_dkv: it brings its
own queries, W_uk, W_uv and W_o.

Parameters: hidden_size, heads, dim, rot_dim, vdim, kv_rank, eps, scale, window,
rot (None or the parameters of a `rotary` position part), own_kv (False for a
run that reads another's cache), gate (None, or the name of the output gate's
matrix), and the tensors' names: q, dkv, dkv_norm, uk, uv, o.

Cache rows are padded with zeros to a multiple of 8 values (the attention
kernels' 16-byte loads).
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import attention_dispatch, kernels
from .base import CacheView, KVRequest, Mixer, TensorSpec, build_part, register_mixer


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class LatentAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.H, self.dim, self.rd, self.vd, self.r = (g("hidden_size"), g("heads"), g("dim"), g("rot_dim"),
                                                              g("vdim"), g("kv_rank"))
        self.eps, self.scale = float(spec["eps"]), float(spec["scale"])
        self.window: Optional[int] = spec.get("window")
        self.own_kv = bool(spec.get("own_kv", True))
        self.names = {k: str(spec[k]) for k in ("q", "dkv", "dkv_norm", "uk", "uv", "o")}
        self.gate_name: Optional[str] = spec.get("gate")
        self.HDp = _pad8(self.r + self.rd)
        if self.HDp > kernels.MAX_HEAD_DIM:
            raise ConfigError(f"latent_attention: a cache row of {self.r} + {self.rd} values exceeds {kernels.MAX_HEAD_DIM}")
        if self.window is not None and self.window < 1:
            raise ConfigError(f"latent_attention: window {self.window} must be positive")
        rot = spec.get("rot")
        self.position = None
        if rot and self.rd:
            self.position = build_part("position", PartSpec("rotary", dict(rot)))
            if self.position.dims > self.rd:
                raise ConfigError(f"latent_attention: {self.position.dims} rotated dims exceed the rotated part of {self.rd}")

    def tensor_specs(self) -> list[TensorSpec]:
        n, H, D, r = self.names, self.H, self.D, self.r
        specs = [TensorSpec(n["q"], (H * (self.dim + self.rd), D)),
                 TensorSpec(n["uk"], (H * self.dim, r)), TensorSpec(n["uv"], (H * self.vd, r)),
                 TensorSpec(n["o"], (D, H * self.vd))]
        if self.gate_name:
            specs.append(TensorSpec(self.gate_name, (H, D)))
        if self.own_kv:
            specs += [TensorSpec(n["dkv"], (r + self.rd, D)),
                      TensorSpec(n["dkv_norm"], (r,), role="gain", init="gain", std=0.1)]
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        n = self.names
        wq = tensors[n["q"]]
        self.n_q = wq.shape[0]
        parts = [wq]
        if self.own_kv:
            parts.append(tensors[n["dkv"]])
        self.norm_w = tensors[n["dkv_norm"]] if self.own_kv else None
        rows = sum(t.shape[0] for t in parts)
        self.gate_off = rows                     # the gate's logits follow the projections in the same product
        if self.gate_name:
            parts.append(tensors[self.gate_name])
            rows += self.H
        if len(parts) > 1 and rows % 8:
            parts.append(torch.zeros((8 - rows % 8, self.D), dtype=wq.dtype, device=wq.device))
        self.w_in = torch.cat(parts, dim=0).contiguous() if len(parts) > 1 else wq
        # W_uk per head, transposed: q_a[r] = sum_i W_uk[h, i, r] q_u[i]
        self.w_ukT = tensors[n["uk"]].view(self.H, self.dim, self.r).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].view(self.H, self.vd, self.r).contiguous()
        self.w_o = tensors[n["o"]]
        self.cos = self.sin = None
        self.rot, self.interleaved = 0, False
        if self.position is not None:
            self.position.prepare(runtime)
            self.cos, self.sin, self.rot = self.position.fused_tables()
            self.interleaved = self.position.interleaved
        self.runtime = runtime

    def streamed_tensors(self) -> list:
        return [self.w_in, self.w_ukT, self.w_uv, self.w_o]

    def kv_request(self) -> KVRequest:
        return KVRequest(1, self.HDp, self.window, values=False)

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        if cache.writes != self.own_kv:
            raise ConfigError("latent_attention: a layer with a down-projection keeps its own cache, one without reads another's")
        H, HDp, r = self.H, self.HDp, self.r
        T = h.shape[0]
        pages = ctx.pages[cache.group]
        p = kernels.linear(h, self.w_in)
        q = torch.empty((T, H * HDp), dtype=p.dtype, device=p.device)
        kernels.latent_prep(p, 0, p if self.own_kv else None, self.n_q, q, H, self.dim, self.rd, r, HDp,
                            self.norm_w, self.eps, self.cos, self.sin, self.rot, self.interleaved, ctx, pages,
                            cache.k if self.own_kv else None)
        kernels.head_linear(p, self.dim + self.rd, 0, self.w_ukT, q, HDp, 0)
        lat = torch.empty((T, H * HDp), dtype=p.dtype, device=p.device)
        if ctx.is_decode:
            scratch = self.runtime.attn_scratch(ctx.B, H, HDp, ctx.decode_splits)
            # the tensor-core decode kernel takes up to 16 query heads a kv head: more heads go in groups of 16
            G = 16 if (H > 16 and attention_dispatch.USE_TC_MASKED and kernels.attn_decode_tc_supported(p.dtype, 16, 1, HDp)
                       and attention_dispatch._tc_fits(16, 1, ctx.decode_splits)) else H
            for h0 in range(0, H, G):
                n = min(G, H - h0)
                cols = slice(h0 * HDp, (h0 + n) * HDp)
                attention_dispatch.decode_masked(q[:, cols] if n < H else q, lat[:, cols] if n < H else lat, ctx, n, 1, HDp,
                                                 HDp, cache.k, cache.k, pages, self.window or 0, 0, self.scale, scratch)
        else:
            attention_dispatch.prefill_masked(q, lat, ctx, H, 1, HDp, HDp, cache.k, cache.k, pages, self.window or 0, 0,
                                              self.scale)
        v = torch.empty((T, H * self.vd), dtype=p.dtype, device=p.device)
        # the gate rides on the value product's accumulators
        kernels.head_linear(lat, HDp, 0, self.w_uv, v, self.vd, 0,
                            gate=p[:, self.gate_off: self.gate_off + H] if self.gate_name else None)
        return kernels.linear(v, self.w_o)


register_mixer("latent_attention", LatentAttention)
