"""Two mixers side by side: both read the same input, each output is RMS-normed
over the model width with a plain gain of its own, and the result is their
weighted sum:

  out = weight * (a / rms(a) * g_a + b / rms(b) * g_b),   a = left(h),  b = right(h)

The sum and both norms are fp32 (`csrc/norm_post.cu`); the branches hand over
fp32 rows. Each branch is a mixer of any registered kind, built from its own
`PartSpec`. At most one branch keeps keys and values (a run of a layer has one
place in a storage group); the branches' fixed-size states are asked for side
by side, branch i's under the name "i".

Parameters: hidden_size, eps, weight, branches (two PartSpecs), out_norms (the
two gains' tensor names).
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..config.spec import PartSpec
from ..ops import kernels
from .base import CacheView, Mixer, TensorSpec, build_part, register_mixer


class ParallelMixers(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.D = int(spec["hidden_size"])
        self.eps = float(spec["eps"])
        self.weight = float(spec.get("weight", 0.5))
        branches = tuple(spec["branches"])
        self.gain_names = tuple(str(n) for n in spec["out_norms"])
        if len(branches) != 2 or len(self.gain_names) != 2:
            raise ConfigError("parallel_mixers: exactly two branches, each with the gain of its output's norm")
        self.branches = [build_part("mixer", b) for b in branches]
        if sum(b.kv_request() is not None for b in self.branches) > 1:
            raise ConfigError("parallel_mixers: only one branch may keep keys and values")

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [ts for b in self.branches for ts in b.tensor_specs()]
        return specs + [TensorSpec(n, (self.D,), role="gain", init="gain", std=0.1) for n in self.gain_names]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        for b in self.branches:
            b.bind({ts.name: tensors[ts.name] for ts in b.tensor_specs() if ts.name in tensors}, runtime)
        g0 = tensors[self.gain_names[0]]
        self.gains = (g0.contiguous(), tensors[self.gain_names[1]].to(g0.dtype).contiguous())

    def streamed_tensors(self) -> list:
        return [t for b in self.branches for t in b.streamed_tensors()]

    def kv_request(self):
        for b in self.branches:
            if b.kv_request() is not None:
                return b.kv_request()
        return None

    def state_request(self):
        req = {str(i): b.state_request() for i, b in enumerate(self.branches) if b.state_request() is not None}
        return req or None

    def forward(self, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        outs = []
        for i, b in enumerate(self.branches):
            state = cache.state.get(str(i)) if cache.state is not None else None
            keeps = b.kv_request() is not None
            view = CacheView(group=cache.group, k=cache.k if keeps else None, v=cache.v if keeps else None,
                             writes=cache.writes, state=state)
            y = b.forward(h, ctx, view)
            if y.dtype != torch.float32:
                raise ConfigError("parallel_mixers: a branch must hand over fp32 rows")
            outs.append(y)
        return kernels.rms_pair_mean(outs[0], outs[1], self.gains[0], self.gains[1], self.eps, self.weight)


register_mixer("parallel_mixers", ParallelMixers)
