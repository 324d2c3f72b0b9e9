"""Token embedding and output head (python/helios/exec/model.py:419,424,486,493-496)."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import InputStage, Norm, OutputStage, Part, WeightSpec


class TokenEmbedding(InputStage):
    """hidden = table[token ids]; no scale and no position term.  The residual stream
    it starts is float32."""

    def __init__(self, vocab: int, width: int) -> None:
        self.vocab = vocab
        self.vocab_size = vocab
        self.width = width
        self.table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.vocab, self.width))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors["weight"].contiguous()

    def forward(self, ctx) -> torch.Tensor:
        return ops.embedding(ctx.token_ids, self.table)


class OutputHead(Part):
    """logits = rows x W^T, float32, without a bias."""

    def __init__(self, vocab: int, width: int) -> None:
        self.vocab = vocab
        self.width = width
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.vocab, self.width))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype)

    def forward(self, ctx, rows: torch.Tensor) -> torch.Tensor:
        return ops.linear_logits(rows, self.weight)


class NormedHead(OutputStage):
    """The usual end of a decoder: the last pending add and the final norm on the wanted rows
    only, then the projection to the vocabulary (python/helios/exec/model.py:491-496 norms
    every row and then selects)."""

    def __init__(self, norm: Norm, head: Part, norm_prefix: str = "model.norm.",
                 head_prefix: str = "lm_head.") -> None:
        self.norm = norm
        self.head = head
        self.norm_prefix = norm_prefix
        self.head_prefix = head_prefix

    @property
    def graph_safe(self) -> bool:
        return self.norm.graph_safe and self.head.graph_safe

    def named_parts(self):
        return [(self.norm_prefix, self.norm), (self.head_prefix, self.head)]

    def forward(self, ctx, residual: torch.Tensor, delta) -> torch.Tensor:
        rows = self.norm.add_forward(residual, delta, ctx.act_dtype, rows=ctx.want_rows)
        return self.head.forward(ctx, rows)
