"""The step function: model + cache, one batch of (request, its next tokens) in,
logits at the wanted places out.  Generation, the scheduler and trace replay all
go through ``EngineCore.step``."""
from __future__ import annotations

import gc
from typing import Hashable, List, Optional, Sequence

import torch

from ..cache.manager import KVCacheManager, pool_sizes_for_bytes
from .batch import MetaLayout, SeqSlice, StepEntry, build_context, context_from_views, fill_meta
from .model import DecoderModel


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


class _StepGraph:
    """A captured step for a fixed number of requests and tokens (both padded) and fixed
    block-table widths: static inputs, one CUDA graph, static logits (one row a request).
    Decode steps have one token a request; mixed steps (prompt portions beside decoded
    tokens) are padded to a token count from ``EngineCore.GRAPH_TOKEN_BUCKETS``."""

    def __init__(self, core: "EngineCore", num_seqs: int, num_tokens: int) -> None:
        cache, model = core.cache, core.model
        self.num_seqs, self.num_tokens = num_seqs, num_tokens
        self.decode = num_seqs == num_tokens
        self.layout = MetaLayout(num_seqs, num_tokens, num_seqs, core.graph_table_widths)
        self.host = torch.empty(self.layout.total, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(self.layout.total, dtype=torch.int32, device=model.device)
        # what kernels are chosen by must not change from step to step: a mixed step always
        # counts as one with long portions
        self.ctx = context_from_views(self.layout, self.dev, [], model.dtype, model.device,
                                      1 if self.decode else num_tokens, core.graph_max_context)
        from ..csrc import ops
        if self.decode:
            self.ctx.extras["decode_splits"] = ops.decode_splits(
                num_seqs, max(s.num_kv_heads for s in cache.specs) if cache.specs else 1,
                core.graph_max_context, max(s.head_dim for s in cache.specs) if cache.specs else 128)
        self.ctx.extras["tile_provider"] = self._tiles
        self._tile_buffers = {}          # (tile, longest first) -> (pinned rows, device rows)
        self._rows_kept = {}             # block-table rows of the staging buffer that are still right
        self._page_size = cache.page_size
        self.graph = None
        self.warmed = False
        self.logits = None
        self.launches = 0
        self.copied = torch.cuda.Event()

    # query tiles of the prefill attention kernels: buffers of a fixed size, refilled with
    # every step's tiles and padded with tiles that hold no work
    def _tiles(self, tile: int, longest_first: bool) -> torch.Tensor:
        key = (tile, longest_first)
        if key not in self._tile_buffers:
            if self.graph is not None or torch.cuda.is_current_stream_capturing():
                raise RuntimeError("a captured step met a tile size its warm-up run did not")
            rows = self.num_tokens // tile + self.num_seqs
            host = torch.empty((rows, 2), dtype=torch.int32, pin_memory=True)
            dev = torch.zeros((rows, 2), dtype=torch.int32, device=self.dev.device)
            self._tile_buffers[key] = (host, dev)
            self._fill_tiles(key)
            self.copied.record()         # the next fill waits for this copy too
        return self._tile_buffers[key][1]

    def _fill_tiles(self, key) -> None:
        from ..csrc import ops
        tile, longest_first = key
        host, dev = self._tile_buffers[key]
        seqs = self.ctx.seqs
        rows = ops.query_tile_rows([s.num_tokens for s in seqs], tile,
                                   [s.start_pos for s in seqs] if longest_first else None)
        view = host.numpy()
        view[:, 0] = 0
        view[:, 1] = ops.EMPTY_TILE_TOKEN
        if rows:
            view[:len(rows)] = rows
        dev.copy_(host, non_blocking=True)

    def fill(self, entries, cache) -> None:
        self.copied.synchronize()        # the staging buffers are free again
        self.ctx.seqs = fill_meta(self.layout, self.host.numpy(), entries, cache, cache.pad_pages,
                                  self._page_size, rows_kept=self._rows_kept)
        # the padding requests count as requests of the step (the tile lists cover them)
        off = sum(s.num_tokens for s in self.ctx.seqs)
        for i in range(len(entries), self.num_seqs):
            n = 1 + (self.num_tokens - off - (self.num_seqs - i) if i == self.num_seqs - 1 else 0)
            self.ctx.seqs.append(SeqSlice(None, 0, 0, n, off))
            off += n
        self.dev.copy_(self.host, non_blocking=True)
        for key in self._tile_buffers:
            self._fill_tiles(key)
        self.copied.record()

    def capture(self, core: "EngineCore") -> None:
        from ..csrc import ops
        before = ops.launch_count
        graph = torch.cuda.CUDAGraph()
        # A CUDA graph that the garbage collector frees while this capture runs (an engine
        # that is no longer used) would invalidate the capture: no collection meanwhile.
        collecting = gc.isenabled()
        gc.disable()
        # Captured by hand on a side stream: torch's ``cuda.graph`` context first gives all
        # cached device memory back to the driver, which stalls a serving loop for 0.2 s and
        # makes the following steps allocate anew.
        stream = core.capture_stream
        stream.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(stream):
                graph.capture_begin(pool=core.graph_pool)
                try:
                    self.logits = core.model.forward(self.ctx, core.cache)
                finally:
                    graph.capture_end()
        finally:
            if collecting:
                gc.enable()
        torch.cuda.current_stream().wait_stream(stream)
        self.launches = ops.launch_count - before
        ops.launch_count = before
        self.graph = graph

    def replay(self) -> torch.Tensor:
        from ..csrc import ops
        self.graph.replay()
        ops.launch_count += self.launches
        return self.logits


class EngineCore:
    #: token counts that mixed steps are padded to when they run as captured graphs; larger
    #: steps keep the device busy longer than the host needs to launch them kernel by kernel
    GRAPH_TOKEN_BUCKETS = (16, 32, 64, 128, 192, 256, 384, 512)
    #: ... except steps that fill one of these counts to seven eighths or more: the full
    #: portions of a long prompt under the usual token budgets, which come many times in a row
    GRAPH_FULL_TOKEN_BUCKETS = (1024, 2048, 4096, 8192)
    #: A small model's steps of some hundred tokens are over on the device before the host has
    #: launched them kernel by kernel (Qwen2.5-0.5B sizes, 768 tokens: 3.4 ms against 1.5 ms at
    #: 512 as a graph), and padding them costs little: models of at most this many parameters
    #: take these token counts too.
    SMALL_MODEL_PARAMETERS = 2_000_000_000
    SMALL_MODEL_TOKEN_BUCKETS = (640, 768, 896, 1024, 1280, 1536, 1792, 2048)
    MAX_FULL_GRAPHS = 8
    FULL_GRAPH_EAGER_RUNS = 6

    def __init__(self, model: DecoderModel, page_size: int, num_pages, max_slots: int,
                 watermark: float = 0.0, max_model_len: Optional[int] = None,
                 poison_cache: Optional[float] = None, use_cuda_graphs: bool = True) -> None:
        self.model = model
        self.cache = KVCacheManager(model.plan, page_size, num_pages, max_slots, model.dtype,
                                    model.device, watermark=watermark, poison=poison_cache)
        self.max_model_len = max_model_len
        self.vocab_size = model.plan.vocab_size
        self.steps_run = 0
        self.tokens_run = 0
        # decode steps (one token per request) run as captured CUDA graphs, one per
        # padded batch size; a size is captured the second time it is seen
        self.use_cuda_graphs = bool(use_cuda_graphs) and model.plan.graph_safe
        # all graphs of the engine draw their intermediate tensors from one pool: they replay
        # one after the other on one stream, and a step's logits hold until the next step only
        self.capture_stream = self.graph_pool = None
        if self.use_cuda_graphs and model.device.type == "cuda":
            self.capture_stream = torch.cuda.Stream(model.device)
            self.graph_pool = torch.cuda.graph_pool_handle()
        # the longest context a request can reach: the smallest pool among the groups that
        # keep every key (a group with a window holds window + portion, whatever the length)
        pool_tokens = self.context_limit(self.cache.groups, page_size)
        if pool_tokens is None:
            pool_tokens = max_model_len or \
                (max(p.num_pages for p in self.cache.pools) * page_size if self.cache.pools else 0)
        self.graph_max_context = min(max_model_len or pool_tokens, pool_tokens) or 1
        self.graph_table_widths = [-(-self.graph_max_context // page_size)] * len(self.cache.groups)
        self._graphs = {}
        self._bucket_seen = {}
        parameters = sum(_numel(spec.shape) for _prefix, part in model.plan.named_parts()
                         for spec in part.weight_specs().values())
        self.graph_token_buckets = self.GRAPH_TOKEN_BUCKETS + (
            self.SMALL_MODEL_TOKEN_BUCKETS if parameters <= self.SMALL_MODEL_PARAMETERS else ())

    @staticmethod
    def padded_requests(n: int) -> int:
        """The number of requests a captured step of ``n`` requests is padded to: ``n`` itself
        up to 8, then the next multiple of 2 up to 16, of 4 up to 32, of 8 up to 64 and so on,
        so that padding adds less than a quarter.  The context slices of decode attention are
        chosen for the padded number, and a captured step costs what its padded number costs:
        9 requests padded to 16 took 4.70 ms a step at Llama-3.1-8B sizes where 8 take 3.84;
        48 padded to 64 gave 5,380 tokens/s against 6,700."""
        if n <= 8:
            return max(1, n)
        step = 2
        while 8 * step < n:
            step *= 2
        return -(-n // step) * step

    @staticmethod
    def context_limit(groups, page_size: int) -> Optional[int]:
        """Tokens the smallest pool among the groups that keep every key holds; None when
        every group has a window (then the pools bound no request's length)."""
        full = [g.num_pages for g in groups if g.window is None]
        return min(full) * page_size if full else None

    @staticmethod
    def pages_for_bytes(model: DecoderModel, page_size: int, kv_cache_bytes: int,
                        max_slots: Optional[int] = None,
                        largest_portion: Optional[int] = None) -> List[int]:
        """Pages of every cache group that a byte budget pays for
        (python/helios/engine.py:147-155 has one kind of layer and one number).  The groups
        that keep every key get the same number of pages each, since a request needs as many
        in one as in another.  A group with a window W never holds more than W + a portion
        (+ a page at either end) per request, so with ``max_slots`` and ``largest_portion``
        given it gets no more than all slots together can use, and the bytes it leaves go
        to the others."""
        elt = torch.empty((), dtype=model.dtype).element_size()
        return pool_sizes_for_bytes(model.plan, page_size, elt, kv_cache_bytes, max_slots,
                                    largest_portion)

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
        earlier step left on the device and the host has not seen.  The logits may lie in a
        captured graph's own buffer: they hold until the next step; keep a copy for longer."""
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
        ran, logits = self._graph_step(entries, token_feed) if self.use_cuda_graphs else (False, None)
        if not ran:
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

    # ------------------------------------------------------------------ captured steps
    def _graph_step(self, entries, token_feed=None):
        """(ran, logits).  A step runs as a captured graph when it fits a shape that has been
        seen before: decode steps by their padded number of requests, mixed steps by their
        padded numbers of requests and tokens.  The first step of a shape runs kernel by
        kernel; the second runs kernel by kernel on the graph's static buffers (which fixes
        what the graph will need); from the third on the graph is replayed."""
        S = len(entries)
        T = sum(len(e.tokens) for e in entries)
        if any(len(e.want) > 1 for e in entries):
            return False, None
        if any(self.cache.length(e.request_id) + len(e.tokens) > self.graph_max_context for e in entries):
            return False, None
        num_seqs = self.padded_requests(S)
        if T == S:
            num_tokens = num_seqs
        else:
            if token_feed is not None:
                return False, None
            if num_seqs == S and T not in self.graph_token_buckets:
                num_seqs = self.padded_requests(S + 1)   # a padding request has to take the spare tokens
            fits = [b for b in self.graph_token_buckets if b >= T + (num_seqs - S)]
            if not fits:
                # a full portion: the requests as they are, and one padding request only if
                # tokens are to spare (such steps come with the same number of requests many
                # times in a row, so the number is not rounded up)
                fits = [b for b in self.GRAPH_FULL_TOKEN_BUCKETS if b >= T and 8 * T >= 7 * b]
                if fits:
                    num_seqs = S if fits[0] == T else S + 1
                    if (num_seqs, fits[0]) not in self._graphs and \
                            sum(t > self.graph_token_buckets[-1] for _s, t in self._graphs) >= self.MAX_FULL_GRAPHS:
                        return False, None
            if not fits or fits[0] > self.graph_max_context:
                return False, None
            num_tokens = fits[0]
        key = (num_seqs, num_tokens)
        g = self._graphs.get(key)
        if g is None:
            seen = self._bucket_seen.get(key, 0)
            self._bucket_seen[key] = seen + 1
            # first time: run eagerly (also warms everything up).  Capturing a step of
            # thousands of tokens costs as much as it saves in a hundred replays: only a
            # shape that keeps coming is worth it.
            eager_runs = 1 if num_tokens <= self.graph_token_buckets[-1] else self.FULL_GRAPH_EAGER_RUNS
            if seen < eager_runs:
                return False, None
            g = self._graphs[key] = _StepGraph(self, num_seqs, num_tokens)
        g.fill(entries, self.cache)
        if token_feed is not None:
            g.ctx.token_ids[:S].copy_(token_feed)
        if g.graph is None and not g.warmed:
            g.warmed = True
            logits = self.model.forward(g.ctx, self.cache)          # on the static buffers, not captured
        else:
            if g.graph is None:
                torch.cuda.synchronize(self.model.device)
                g.capture(self)
            logits = g.replay()
        rows = [i for i, e in enumerate(entries) if e.want]
        if not rows:
            return True, None
        if len(rows) == S:
            return True, logits[:S]
        return True, logits.index_select(0, torch.tensor(rows, device=logits.device))
