"""The step function: model + cache, one batch of (request, its next tokens) in,
logits at the wanted places out.  Generation, the scheduler and trace replay all
go through ``EngineCore.step``."""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence

import torch

from ..cache.manager import KVCacheManager, bytes_per_page
from .batch import StepEntry, build_context
from .model import DecoderModel


class EngineCore:
    def __init__(self, model: DecoderModel, page_size: int, num_pages, max_slots: int,
                 watermark: float = 0.0, max_model_len: Optional[int] = None,
                 poison_cache: Optional[float] = None) -> None:
        self.model = model
        self.cache = KVCacheManager(model.plan, page_size, num_pages, max_slots, model.dtype,
                                    model.device, watermark=watermark, poison=poison_cache)
        self.max_model_len = max_model_len
        self.vocab_size = model.plan.embedding.vocab
        self.steps_run = 0
        self.tokens_run = 0

    @staticmethod
    def pages_for_bytes(model: DecoderModel, page_size: int, kv_cache_bytes: int) -> int:
        """Pages per group a byte budget pays for; every group gets the same number
        (python/helios/engine.py:147-155)."""
        per_page = sum(bytes_per_page(model.plan, page_size,
                                      torch.empty((), dtype=model.dtype).element_size()))
        return max(8, kv_cache_bytes // max(1, per_page))

    # ------------------------------------------------------------------ requests
    def begin(self, request_id: Hashable) -> int:
        return self.cache.admit(request_id)

    def end(self, request_id: Hashable) -> None:
        if self.cache.has(request_id):
            self.cache.release(request_id)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], manage_cache: bool = True) -> Optional[torch.Tensor]:
        """Run exactly the given tokens as one batch over the cache earlier steps left.
        Returns float32 logits [sum of len(want), vocab] in the order of the entries and
        of their ``want``.  With ``manage_cache`` requests not seen before are admitted,
        pages for the new tokens are taken and the new length is committed; a scheduler
        that does this bookkeeping itself passes False."""
        entries = [e for e in entries]
        if not entries:
            return None
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise ValueError(f"token id {t} of request {e.request_id!r} is outside "
                                     f"the vocabulary (0..{self.vocab_size - 1})")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"request {e.request_id!r} wants place {w} of {n} tokens")
        for e in entries:
            if not self.cache.has(e.request_id):
                if not manage_cache:
                    raise ValueError(f"request {e.request_id!r} has no cache entry")
                self.cache.admit(e.request_id)
            if self.max_model_len is not None and \
                    self.cache.length(e.request_id) + len(e.tokens) > self.max_model_len:
                raise ValueError(f"request {e.request_id!r} would exceed max_model_len "
                                 f"{self.max_model_len}")
        if manage_cache:
            for e in entries:
                self.cache.extend(e.request_id, len(e.tokens))
        else:
            for e in entries:
                if any(self.cache.pages_needed(e.request_id, len(e.tokens))):
                    raise ValueError(f"request {e.request_id!r} has no pages for its "
                                     f"{len(e.tokens)} new tokens")
        ctx = build_context(entries, self.cache, self.model.dtype, self.model.device)
        logits = self.model.forward(ctx, self.cache)
        if manage_cache:
            for e in entries:
                self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        self.tokens_run += ctx.num_tokens
        return logits
