"""Feed-forwards of several small experts, of which every token uses `top`.

`table_routed_experts` picks without a router: a table [vocab, top] gives each token id its experts (the
entries of a row differ), and each counts 1/top.

An expert, with h its input (no biases):

  g = min(W_gate h, limit),   u = clamp(W_up h, -limit, limit)
  y = g * sigmoid(alpha g) * (u + 1),   out = W_down y

The step's (token, choice) pairs are sorted by expert on the device and the two
products run tile by tile over rows that share an expert (`csrc/moe.cu`); the
experts' matrices are stacked at bind time.

Parameters: hidden_size, intermediate_size (of one expert), experts, top, limit,
alpha (1.702 unless given), vocab_size, table (tensor name) and expert_prefix:
expert e's tensors are `<expert_prefix><e>.gate`, `.up` and `.down`.

`router_experts` picks with a learned router:

  z = W_r h + b_r  (fp32);  the `top` largest z (the lower index wins a tie);
  their weights are softmax over the chosen z alone
  expert:  out = W_down act(W_up h),  act the exact (erf) GELU, no gate, no biases
  result = sum over the chosen of weight * expert(h),  fp32 rows (not rounded to the activation type)

Parameters: hidden_size, intermediate_size, experts, top, activation
("gelu_erf"), router, router_bias (tensor names) and expert_prefix: expert e's
tensors are `<expert_prefix><e>.up` and `.down`.

`group_router_experts` picks with sigmoid scores, a correction and groups:

  s = sigmoid(W_r h)  (fp32);  the choice goes by s + correction
  the experts form `groups` equal groups of neighbours; a group counts the sum of its two largest choice scores;
  only experts of the `keep` best groups can be chosen (the lower index wins every tie)
  the `top` largest choice scores among them; each counts s (without the correction) * weight_scale, not renormalised
  expert: the clamped-gate expert of `table_routed_experts` (limit, alpha)

Parameters: hidden_size, intermediate_size, experts, top, groups (1), keep (= groups), weight_scale (1), limit, alpha
(1.702), router, correction (tensor names) and expert_prefix.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..config.keys import ConfigError
from ..ops import kernels
from .base import FeedForward, TensorSpec, register_ffn


class TableRoutedExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.F, self.E, self.top, self.V = (g("hidden_size"), g("intermediate_size"), g("experts"), g("top"),
                                                    g("vocab_size"))
        self.limit = float(spec["limit"])
        self.alpha = float(spec.get("alpha", 1.702))
        self.table_name = str(spec["table"])
        self.prefix = str(spec["expert_prefix"])
        if not 1 <= self.top <= self.E:
            raise ConfigError(f"table_routed_experts: top {self.top} does not fit {self.E} experts")
        if self.E > 1024:
            raise ConfigError(f"table_routed_experts: {self.E} experts exceed the 1024 that the routing kernel counts")

    def _name(self, e: int, which: str) -> str:
        return f"{self.prefix}{e}.{which}"

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [TensorSpec(self.table_name, (self.V, self.top), role="table", init=f"distinct:{self.E}")]
        for e in range(self.E):
            specs += [TensorSpec(self._name(e, "gate"), (self.F, self.D)), TensorSpec(self._name(e, "up"), (self.F, self.D)),
                      TensorSpec(self._name(e, "down"), (self.D, self.F))]
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.table = tensors[self.table_name].contiguous()
        self.w_gu = torch.stack([torch.stack([tensors[self._name(e, "gate")], tensors[self._name(e, "up")]])
                                 for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[self._name(e, "down")] for e in range(self.E)]).contiguous()

    def streamed_tensors(self) -> list:
        return []          # a step reads only the experts its tokens pick

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return kernels.moe_table_ffn(h, self.table, self.w_gu, self.w_down, ctx, self.top, self.limit, self.alpha)


register_ffn("table_routed_experts", TableRoutedExperts)


class RouterExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.F, self.E, self.top = g("hidden_size"), g("intermediate_size"), g("experts"), g("top")
        self.router_name, self.bias_name = str(spec["router"]), str(spec["router_bias"])
        self.prefix = str(spec["expert_prefix"])
        if spec.get("activation", "gelu_erf") != "gelu_erf":
            raise ConfigError(f"router_experts: activation {spec.get('activation')!r} is not built in (gelu_erf)")
        if not 1 <= self.top <= self.E:
            raise ConfigError(f"router_experts: top {self.top} does not fit {self.E} experts")
        if self.E > 1024:
            raise ConfigError(f"router_experts: {self.E} experts exceed the 1024 that the routing kernel counts")

    def _name(self, e: int, which: str) -> str:
        return f"{self.prefix}{e}.{which}"

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [TensorSpec(self.router_name, (self.E, self.D), std=0.3),
                 TensorSpec(self.bias_name, (self.E,), role="gain", init="normal", std=0.3)]
        for e in range(self.E):
            specs += [TensorSpec(self._name(e, "up"), (self.F, self.D)), TensorSpec(self._name(e, "down"), (self.D, self.F))]
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.w_router = tensors[self.router_name].contiguous()
        self.b_router = tensors[self.bias_name].contiguous()
        self.w_up = torch.stack([tensors[self._name(e, "up")] for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[self._name(e, "down")] for e in range(self.E)]).contiguous()

    def streamed_tensors(self) -> list:
        return [self.w_router]          # of the experts a step reads only those its tokens pick

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return kernels.moe_router_ffn(h, self.w_router, self.b_router, self.w_up, self.w_down, ctx, self.top)


register_ffn("router_experts", RouterExperts)


class GroupRouterExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        g = lambda k: int(spec[k])
        self.D, self.F, self.E, self.top = g("hidden_size"), g("intermediate_size"), g("experts"), g("top")
        self.groups = int(spec.get("groups", 1))
        self.keep = int(spec.get("keep", self.groups))
        self.weight_scale = float(spec.get("weight_scale", 1.0))
        self.limit = float(spec["limit"])
        self.alpha = float(spec.get("alpha", 1.702))
        self.router_name, self.correction_name = str(spec["router"]), str(spec["correction"])
        self.prefix = str(spec["expert_prefix"])
        if self.E > 1024:
            raise ConfigError(f"group_router_experts: {self.E} experts exceed the 1024 that the routing kernel counts")
        if self.groups < 1 or self.E % self.groups or not 1 <= self.keep <= self.groups:
            raise ConfigError(f"group_router_experts: {self.E} experts do not form {self.groups} equal groups of which "
                              f"{self.keep} are kept")
        if not 1 <= self.top <= self.keep * (self.E // self.groups):
            raise ConfigError(f"group_router_experts: top {self.top} does not fit the experts of {self.keep} kept groups")

    def _name(self, e: int, which: str) -> str:
        return f"{self.prefix}{e}.{which}"

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [TensorSpec(self.router_name, (self.E, self.D), std=0.3),
                 TensorSpec(self.correction_name, (self.E,), role="gain", init="normal", std=0.1)]
        for e in range(self.E):
            specs += [TensorSpec(self._name(e, "gate"), (self.F, self.D)), TensorSpec(self._name(e, "up"), (self.F, self.D)),
                      TensorSpec(self._name(e, "down"), (self.D, self.F))]
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.w_router = tensors[self.router_name].contiguous()
        self.correction = tensors[self.correction_name].contiguous()
        self.w_gu = torch.stack([torch.stack([tensors[self._name(e, "gate")], tensors[self._name(e, "up")]])
                                 for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[self._name(e, "down")] for e in range(self.E)]).contiguous()

    def streamed_tensors(self) -> list:
        return [self.w_router]          # of the experts a step reads only those its tokens pick

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        return kernels.moe_group_router_ffn(h, self.w_router, self.correction, self.w_gu, self.w_down, ctx, self.top,
                                            self.groups, self.keep, self.weight_scale, self.limit, self.alpha)


register_ffn("group_router_experts", GroupRouterExperts)
