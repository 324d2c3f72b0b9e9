"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(python/helios/exec/model.py:321-337).  gate and up are one fused projection."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import DeferredNorm, FeedForward, WeightSpec, register_part
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

    def forward_from_residual(self, ctx, residual: torch.Tensor, norm, pre=None, then=None):
        """Steps of few tokens run without norm launches: gate|up takes the 1 / rms of ``pre``
        as a factor on its accumulators, and the down projection adds into the residual and
        leaves ``then`` all but done."""
        if ctx.act_dtype != torch.bfloat16 or type(norm) is not RMSNorm \
                or not ops.deferred_norm_fits(ctx.num_tokens, self.w_gate_up, self.w_down):
            return False
        if pre is not None:
            h = ops.linear_bf16(pre.scaled, self.w_gate_up, glu=True, sumsq=pre.sumsq, eps=norm.eps)
        else:
            h = ops.linear_bf16(norm.add_forward(residual, None, ctx.act_dtype), self.w_gate_up, glu=True)
        if type(then) is RMSNorm:
            scaled, sumsq = ops.linear_bf16(h, self.w_down, residual=residual, norm_weight=then.weight)
            return DeferredNorm(then, scaled, sumsq)
        ops.linear_bf16(h, self.w_down, residual=residual)
        return True


register_part("feed_forward", "swiglu", SwiGLU)
