"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(python/helios/exec/model.py:321-337).  gate and up are one fused projection."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, WeightSpec, register_part


class SwiGLU(FeedForward):
    def __init__(self, width: int, inner: int) -> None:
        self.width = width
        self.inner = inner
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {
            "gate_proj.weight": WeightSpec((self.inner, self.width)),
            "up_proj.weight": WeightSpec((self.inner, self.width)),
            "down_proj.weight": WeightSpec((self.width, self.inner)),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]],
                                   dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.linear_swiglu(x, self.w_gate_up), self.w_down)


register_part("feed_forward", "swiglu", SwiGLU)
