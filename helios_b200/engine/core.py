"""The step function: model + cache, one batch of (request, its next tokens) in,
logits at the wanted places out.  Generation, the scheduler and trace replay all
go through ``EngineCore.step``."""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence

import torch

from ..cache.manager import KVCacheManager, bytes_per_page
from .batch import MetaLayout, StepEntry, build_context, context_from_views, fill_meta
from .model import DecoderModel


class _DecodeGraph:
    """A captured decode step for a fixed number of requests (padded) and fixed block-table
    widths: static inputs, one CUDA graph, static logits."""

    def __init__(self, core: "EngineCore", bucket: int) -> None:
        cache, model = core.cache, core.model
        self.bucket = bucket
        self.layout = MetaLayout(bucket, bucket, bucket, core.graph_table_widths)
        self.host = torch.empty(self.layout.total, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(self.layout.total, dtype=torch.int32, device=model.device)
        self.ctx = context_from_views(self.layout, self.dev, [], model.dtype, model.device, 1,
                                      core.graph_max_context)
        from ..csrc import ops
        self.ctx.extras["decode_splits"] = ops.decode_splits(
            bucket, max(s.num_kv_heads for s in cache.specs) if cache.specs else 1,
            core.graph_max_context)
        self.graph = None
        self.logits = None
        self.launches = 0
        self.copied = torch.cuda.Event()

    def fill(self, entries, cache) -> None:
        self.copied.synchronize()        # the staging buffer is free again
        self.ctx.seqs = fill_meta(self.layout, self.host.numpy(), entries, cache, cache.pad_pages)
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()

    def capture(self, core: "EngineCore") -> None:
        from ..csrc import ops
        before = ops.launch_count
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.logits = core.model.forward(self.ctx, core.cache)
        self.launches = ops.launch_count - before
        ops.launch_count = before
        self.graph = graph

    def replay(self) -> torch.Tensor:
        from ..csrc import ops
        self.graph.replay()
        ops.launch_count += self.launches
        return self.logits


class EngineCore:
    def __init__(self, model: DecoderModel, page_size: int, num_pages, max_slots: int,
                 watermark: float = 0.0, max_model_len: Optional[int] = None,
                 poison_cache: Optional[float] = None, use_cuda_graphs: bool = True) -> None:
        self.model = model
        self.cache = KVCacheManager(model.plan, page_size, num_pages, max_slots, model.dtype,
                                    model.device, watermark=watermark, poison=poison_cache)
        self.max_model_len = max_model_len
        self.vocab_size = model.plan.embedding.vocab
        self.steps_run = 0
        self.tokens_run = 0
        # decode steps (one token per request) run as captured CUDA graphs, one per
        # padded batch size; a size is captured the second time it is seen
        self.use_cuda_graphs = bool(use_cuda_graphs) and model.plan.graph_safe
        pool_tokens = max(p.num_pages for p in self.cache.pools) * page_size if self.cache.pools else 0
        self.graph_max_context = min(max_model_len or pool_tokens, pool_tokens) or 1
        self.graph_table_widths = [-(-self.graph_max_context // page_size)] * len(self.cache.groups)
        self._graphs = {}
        self._bucket_seen = {}

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
    def step(self, entries: Sequence[StepEntry], manage_cache: bool = True,
             token_feed: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run exactly the given tokens as one batch over the cache earlier steps left.
        Returns float32 logits [sum of len(want), vocab] in the order of the entries and
        of their ``want``.  With ``manage_cache`` requests not seen before are admitted,
        pages for the new tokens are taken and the new length is committed; a scheduler
        that does this bookkeeping itself passes False.  ``token_feed`` (int32 on the
        device, one per entry) replaces the one token of every entry: token ids that an
        earlier step left on the device and the host has not seen."""
        entries = [e for e in entries]
        if not entries:
            return None
        if token_feed is not None:
            if any(len(e.tokens) != 1 for e in entries) or token_feed.numel() != len(entries) \
                    or token_feed.dtype != torch.int32 or token_feed.device.type != self.model.device.type:
                raise ValueError("token_feed takes int32 on the model's device, one token per entry")
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
        logits = None
        if self.use_cuda_graphs and all(len(e.tokens) == 1 for e in entries):
            logits = self._graph_step(entries, token_feed)
        if logits is None:
            ctx = build_context(entries, self.cache, self.model.dtype, self.model.device)
            if token_feed is not None:
                ctx.token_ids.copy_(token_feed)
            logits = self.model.forward(ctx, self.cache)
        if manage_cache:
            for e in entries:
                self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits

    # ------------------------------------------------------------------ captured decode steps
    def _graph_step(self, entries, token_feed=None) -> Optional[torch.Tensor]:
        S = len(entries)
        bucket = 1
        while bucket < S:
            bucket *= 2
        if any(self.cache.length(e.request_id) + 1 > self.graph_max_context for e in entries):
            return None
        g = self._graphs.get(bucket)
        if g is None:
            seen = self._bucket_seen.get(bucket, 0)
            self._bucket_seen[bucket] = seen + 1
            if seen == 0:
                return None                    # first time: run eagerly (also warms everything up)
            g = _DecodeGraph(self, bucket)
            g.fill(entries, self.cache)
            torch.cuda.synchronize(self.model.device)
            g.capture(self)
            self._graphs[bucket] = g
        g.fill(entries, self.cache)
        if token_feed is not None:
            g.ctx.token_ids[:S].copy_(token_feed)
        logits = g.replay()
        if all(len(e.want) == 1 for e in entries):
            return logits[:S]
        rows = [i for i, e in enumerate(entries) if e.want]
        if not rows:
            return None
        return logits.index_select(0, torch.tensor(rows, device=logits.device))
