"""RMSNorm (python/helios/exec/model.py:95-114): statistics in float32, no mean
subtraction, no bias.  The weight is kept in float32 in both modes."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Norm, WeightSpec, register_part


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float) -> None:
        self.width = width
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.width,), kind="vector", init="ones_jitter")}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def add_forward(self, residual, delta, out_dtype, rows=None):
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out_dtype, rows)


register_part("norm", "rmsnorm", RMSNorm)
