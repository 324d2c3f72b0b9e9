"""Pre-norm residual block (python/helios/exec/model.py:340-392):
x + mixer(norm(x)), then x + feed_forward(norm(x)).

The residual stream is float32.  A block receives the stream and the output of
the part before that is still to be added; the add is fused into the next norm.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .base import Block, DeferredNorm, FeedForward, LayerCache, Mixer, Norm, Part, register_part


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward,
                 names: Tuple[str, str, str, str] = ("input_layernorm.", "self_attn.",
                                                     "post_attention_layernorm.", "mlp.")) -> None:
        self.mixer_norm = mixer_norm
        self._mixer = mixer
        self.ffn_norm = ffn_norm
        self.ffn = ffn
        self.names = names

    @property
    def mixer(self) -> Mixer:
        return self._mixer

    def named_parts(self) -> List[Tuple[str, Part]]:
        return list(zip(self.names, (self.mixer_norm, self._mixer, self.ffn_norm, self.ffn)))

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for _, p in self.named_parts())

    @property
    def first_norm(self) -> Norm:
        return self.mixer_norm

    def forward(self, ctx, residual: torch.Tensor, delta, cache: Optional[LayerCache],
                state: Optional[torch.Tensor]):
        # A part may take the norm before it and the add after it into its own kernels (steps
        # of few tokens); that needs a residual stream to which nothing is pending.  Such a
        # part may also leave the NEXT norm all but done (a DeferredNorm) for the part after it.
        pre = None
        if isinstance(delta, DeferredNorm):
            pre, delta = (delta if delta.norm is self.mixer_norm else None), None
        done = False
        if delta is None:
            done = self._mixer.forward_from_residual(ctx, residual, self.mixer_norm, cache, state,
                                                     pre=pre, then=self.ffn_norm)
        if done is False:
            x = self.mixer_norm.add_forward(residual, delta, ctx.act_dtype)
            delta = self._mixer.forward(ctx, x, cache, state)
        else:
            delta = None
            done = self.ffn.forward_from_residual(ctx, residual, self.ffn_norm,
                                                  pre=done if isinstance(done, DeferredNorm) else None,
                                                  then=ctx.norm_after_block)
            if done is not False:
                return residual, (done if isinstance(done, DeferredNorm) else None)
        x = self.ffn_norm.add_forward(residual, delta, ctx.act_dtype)
        return residual, self.ffn.forward(ctx, x)


register_part("block", "pre_norm", PreNormBlock)
