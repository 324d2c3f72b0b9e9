"""Token embedding and output head (python/helios/exec/model.py:419,424,486,493-496)."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Part, WeightSpec


class TokenEmbedding(Part):
    """hidden = table[token ids]; no scale and no position term.  The residual stream
    it starts is float32."""

    def __init__(self, vocab: int, width: int) -> None:
        self.vocab = vocab
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

    def forward(self, ctx, rows: torch.Tensor) -> torch.Tensor:
        return ops.linear_logits(rows, self.weight)
