"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(python/helios/exec/model.py:321-337).  gate and up are one fused projection."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, WeightSpec, register_part
from .norm import RMSNorm


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

    def kernel_libraries(self, dtype):
        return ops.linear_libraries(dtype, self.width)

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]],
                                   dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.linear_swiglu(x, self.w_gate_up), self.w_down)

    def forward_from_residual(self, ctx, residual: torch.Tensor, norm) -> bool:
        """Steps of very few tokens: norm + gate|up + SwiGLU in one launch, down + residual
        add in another."""
        if ctx.act_dtype != torch.bfloat16 or type(norm) is not RMSNorm \
                or not ops.small_step_fits(ctx.num_tokens, self.width, self.width, self.inner):
            return False
        h = ops.small_norm_swiglu(residual, norm.weight, norm.eps, self.w_gate_up)
        ops.small_linear_residual(residual, h, self.w_down)
        return True


register_part("feed_forward", "swiglu", SwiGLU)
