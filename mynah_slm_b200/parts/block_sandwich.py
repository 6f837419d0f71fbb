"""A block with a norm before AND after each sublayer:

  x <- x + post_mixer(mixer(in1(pre_mixer(x)))),   then   x <- x + post_ffn(ffn(in2(pre_ffn(x))))

`in(h)`, optional, is a short causal convolution over time on every channel of
the normed rows, added to them: in(h) = h + conv(h), with a filter
[hidden, taps] and no bias (parameters `input_conv_taps`, `mixer_conv_name`,
`ffn_conv_name`; taps 0 or None: the sublayers read the normed rows). The last
taps-1 normed rows of each sublayer are part of a sequence's state: the block
asks the cache for them. The feed-forward may be missing (`ffn` None).

The stream, the norms and the sums are fp32: the norm in front hands fp32 rows
to the convolution (which keeps fp32 inputs as its state and rounds only its
result to the activation type), the sublayers hand back fp32 rows, and the norm
behind a sublayer adds into the stream in the same pass. That pass also forms
the next norm in front where the block knows it (the feed-forward's, after the
mixer), so a layer costs three norm launches, not four.

The norms are named "mixer", "mixer_out", "ffn", "ffn_out" and are RMS norms
(they must offer `gain` and `eps`).
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.keys import ConfigError
from ..ops import kernels
from .base import Block, CacheView, Residual, StateRequest, TensorSpec, register_block


class SandwichResidual(Block):
    def __init__(self, spec, mixer, ffn, norms):
        super().__init__(spec, mixer, ffn, norms)
        need = ("mixer", "mixer_out") + (("ffn", "ffn_out") if ffn is not None else ())
        for n in need:
            if n not in self.norms:
                raise ConfigError(f"sandwich_residual: the layer gives no {n!r} norm")
            if not hasattr(self.norms[n], "gain") or not hasattr(self.norms[n], "eps"):
                raise ConfigError(f"sandwich_residual: norm {n!r} is not an RMS norm (no gain and eps)")
        self.D = int(spec["hidden_size"])
        self.taps = int(spec.get("input_conv_taps") or 0)
        self.conv_names = {"mixer": spec.get("mixer_conv_name"), "ffn": spec.get("ffn_conv_name")}
        if self.taps and not (self.conv_names["mixer"] and (ffn is None or self.conv_names["ffn"])):
            raise ConfigError("sandwich_residual: an input convolution needs its tensors' names")
        self.conv_w: dict[str, Optional[torch.Tensor]] = {"mixer": None, "ffn": None}
        self.act_dtype = torch.float32

    def _sublayers(self) -> tuple[str, ...]:
        return ("mixer",) + (("ffn",) if self.ffn is not None else ())

    def tensor_specs(self) -> list[TensorSpec]:
        if not self.taps:
            return []
        return [TensorSpec(self.conv_names[s], (self.D, self.taps), init="normal", std=0.1) for s in self._sublayers()]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        if self.taps:
            for s in self._sublayers():
                self.conv_w[s] = tensors[self.conv_names[s]].contiguous()
        self.act_dtype = runtime.act_dtype

    def state_request(self):
        if self.taps > 1:
            return {s + "_input_conv": StateRequest((self.taps - 1, self.D), torch.float32) for s in self._sublayers()}
        return None

    def _input(self, which: str, h: torch.Tensor, ctx, cache: CacheView) -> torch.Tensor:
        """The sublayer's input from the fp32 normed rows."""
        if self.taps:
            state = cache.block_state[which + "_input_conv"] if self.taps > 1 else None
            return kernels.causal_conv(h, self.conv_w[which], None, state, ctx, self.act_dtype, add_input=True)
        return h if self.act_dtype == torch.float32 else kernels.cast_rows(h, self.act_dtype)

    def forward(self, stream: Residual, ctx, cache: CacheView) -> None:
        x = stream.flush()
        pre, post = self.norms["mixer"], self.norms["mixer_out"]
        h = kernels.rmsnorm(x, pre.gain, pre.eps, torch.float32)
        y = self.mixer.forward(self._input("mixer", h, ctx, cache), ctx, cache)
        if self.ffn is None:
            kernels.rmsnorm_add(x, y, post.gain, post.eps)
            return
        pre2, post2 = self.norms["ffn"], self.norms["ffn_out"]
        h = kernels.rmsnorm_add(x, y, post.gain, post.eps, gain2=pre2.gain, eps2=pre2.eps)
        y = self.ffn.forward(self._input("ffn", h, ctx, cache), ctx)
        kernels.rmsnorm_add(x, y, post2.gain, post2.eps)


register_block("sandwich_residual", SandwichResidual)
