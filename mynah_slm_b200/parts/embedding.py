"""Token embedding and output head.

Embedding: x = E[token], no scaling by sqrt(hidden) (mynah-slm
src/arch_qwen3.c:186); a design that multiplies its embedding by a constant
gives `scale` (the product is fp32), and one that multiplies its logits by a
constant gives the head `logit_scale`. Head: logits = Head . h in fp32, where Head is the
embedding matrix when the configuration ties them and `lm_head.weight`
otherwise; the configuration decides, not the presence of the tensor
(docs/qwen3-arch.md:91-113: the official checkpoint ships a duplicate
`lm_head.weight` although it is tied).
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..ops import kernels
from .base import Embedding, Head, Part, TensorSpec, register_embedding, register_head


class TokenEmbedding(Embedding):
    def __init__(self, spec):
        super().__init__(spec)
        self.name = str(spec["name"])
        self.V, self.D = int(spec["vocab_size"]), int(spec["dim"])
        self.scale = float(spec.get("scale", 1.0))
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.V, self.D))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.table = tensors[self.name]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return kernels.embed_gather(self.table, tokens, scale=self.scale)


class LinearHead(Head):
    def __init__(self, spec, embedding):
        super().__init__(spec)
        self.tied = bool(spec["tied"])
        self.name = str(spec["name"])
        self.V, self.D = int(spec["vocab_size"]), int(spec["dim"])
        self.embedding = embedding
        self.logit_scale = float(spec.get("logit_scale", 1.0))
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        # tied: a stored copy is tolerated and left unread
        return [TensorSpec(self.name, (self.V, self.D), ignorable=self.tied)]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        if self.tied and getattr(self.embedding, "table", None) is None:
            from ..config.keys import ConfigError
            raise ConfigError("linear_head: a tied head needs an embedding part that keeps its matrix as `table`")
        self.weight = self.embedding.table if self.tied else tensors[self.name]

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = kernels.linear(h, self.weight, out_dtype=torch.float32)
        return logits if self.logit_scale == 1.0 else kernels.scale_(logits, self.logit_scale)


register_embedding("token_embedding", TokenEmbedding)
register_head("linear_head", LinearHead)


class TokenPositionEmbedding(Embedding):
    """x = E[token] + P[position]: a learned vector per absolute position, added unscaled to the token's.
    Parameters: name, position_name, vocab_size, dim, max_positions. It reads the rows' positions, so the
    engine hands it the step's context."""
    needs_context = True

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.pos_name = str(spec["name"]), str(spec["position_name"])
        self.V, self.D, self.P = int(spec["vocab_size"]), int(spec["dim"]), int(spec["max_positions"])
        self.table: Optional[torch.Tensor] = None
        self.pos_table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.V, self.D)), TensorSpec(self.pos_name, (self.P, self.D))]

    def bind(self, tensors: Mapping[str, torch.Tensor], runtime) -> None:
        self.table, self.pos_table = tensors[self.name], tensors[self.pos_name]

    def forward(self, tokens: torch.Tensor, ctx) -> torch.Tensor:
        return kernels.embed_positions(self.table, self.pos_table, tokens, ctx.tok_pos, ctx.status)


register_embedding("token_position_embedding", TokenPositionEmbedding)


class StreamVectors(Part):
    """Learned vectors [count, dim] that the schedule adds to every row of the residual stream before chosen runs
    (`ScheduleEntry.add_vector`); kept in fp32, like the stream. Parameters: name, count, dim."""

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.count, self.dim = str(spec["name"]), int(spec["count"]), int(spec["dim"])
        self.rows = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.count, self.dim), role="gain", init="normal", std=0.1)]

    def bind(self, tensors, runtime) -> None:
        self.rows = tensors[self.name].to(torch.float32).contiguous()
