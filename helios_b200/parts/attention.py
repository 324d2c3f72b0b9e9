"""Grouped-query attention over the paged cache
(python/helios/exec/model.py:156-251; math of python/helios/exec/paged_attn.py:264-408).

One fused projection gives q, k and v (+ bias where the configuration has one);
one kernel rotates q and k and writes k and v into the request's pages before
attending, so a portion of a prompt sees itself (model.py:203-206); attention
runs over the cache for every token of the batch, whatever mix of prompt
portions and single decoded tokens it is; then the output projection.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import DeferredNorm, LayerCache, Mixer, PagedCacheSpec, WeightSpec, register_part
from .norm import RMSNorm


class GQAAttention(Mixer):
    def __init__(self, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, qkv_bias: bool, window: Optional[int] = None,
                 rotary: bool = True, position=None) -> None:
        """``position``: the encoding whose cos/sin tables rotate q and k (its
        ``tables(ctx)``); None takes the tables the plan's own encoding left on the step
        context.  ``rotary=False``: no rotation at all."""
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported (even, at most 256)")
        self.width = width
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.qkv_bias = qkv_bias
        self.window = window
        self.rotary = rotary
        self.position = position
        self.w_qkv = self.b_qkv = self.w_o = None

    # ---------------------------------------------------------------- what it keeps
    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def kernel_libraries(self, dtype):
        return (ops.linear_libraries(dtype, self.width)
                + ops.attention_libraries(dtype, self.num_heads, self.num_kv_heads, self.head_dim))

    # ---------------------------------------------------------------- tensors
    def weight_specs(self) -> Dict[str, WeightSpec]:
        q, kv = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = {
            "q_proj.weight": WeightSpec((q, self.width)),
            "k_proj.weight": WeightSpec((kv, self.width)),
            "v_proj.weight": WeightSpec((kv, self.width)),
            "o_proj.weight": WeightSpec((self.width, q)),
        }
        if self.qkv_bias:
            specs["q_proj.bias"] = WeightSpec((q,), kind="vector", init="normal")
            specs["k_proj.bias"] = WeightSpec((kv,), kind="vector", init="normal")
            specs["v_proj.bias"] = WeightSpec((kv,), kind="vector", init="normal")
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"],
                                    tensors["v_proj.bias"]], dim=0).contiguous()

    # ---------------------------------------------------------------- forward
    def _rotary_tables(self, ctx):
        if not self.rotary:
            return None, None
        if self.position is not None:
            return self.position.tables(ctx)
        return ctx.rotary_cos, ctx.rotary_sin

    def forward_from_residual(self, ctx, residual: torch.Tensor, norm, cache: LayerCache, state=None,
                              pre=None, then=None):
        """Steps of few tokens run without norm launches: q|k|v takes the 1 / rms of ``pre``
        as a factor on its accumulators (the norm kernel runs where nothing was handed over),
        and the output projection adds into the residual and leaves ``then`` all but done."""
        if ctx.act_dtype != torch.bfloat16 or type(norm) is not RMSNorm or cache is None \
                or not ops.deferred_norm_fits(ctx.num_tokens, self.w_qkv, self.w_o):
            return False
        if pre is not None:
            qkv = ops.linear_bf16(pre.scaled, self.w_qkv, self.b_qkv, sumsq=pre.sumsq, eps=norm.eps)
        else:
            qkv = ops.linear_bf16(norm.add_forward(residual, None, ctx.act_dtype), self.w_qkv, self.b_qkv)
        attn = self._attend(ctx, qkv, cache)
        if type(then) is RMSNorm:
            scaled, sumsq = ops.linear_bf16(attn, self.w_o, residual=residual, norm_weight=then.weight)
            return DeferredNorm(then, scaled, sumsq)
        ops.linear_bf16(attn, self.w_o, residual=residual)
        return True

    def _attend(self, ctx, qkv: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        table = ctx.block_tables[cache.group]
        cos, sin = self._rotary_tables(ctx)
        return ops.attention(ctx, qkv, cache.k_pages, cache.v_pages, table, self.num_heads,
                             self.num_kv_heads, self.head_dim, cache.page_size, self.window,
                             self.scale, fresh=(cos, sin, cache.write))

    def forward(self, ctx, x: torch.Tensor, cache: LayerCache, state=None) -> torch.Tensor:
        return ops.linear(self._attend(ctx, ops.linear(x, self.w_qkv, self.b_qkv), cache), self.w_o)


register_part("mixer", "gqa_attention", GQAAttention)
