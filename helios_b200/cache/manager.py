"""The cache of a model on the device: page pools per group, one view per cache
id, and the fixed-size state of every request slot
(python/helios/exec/paged_attn.py:25-115 holds the same bytes, one object per layer;
python/helios/exec/runner.py:64-74 allocates them).

Layout of a group: ``[cache ids in the group, 2 (k, v), pages, kv heads,
page_size, head_dim]``; one page id addresses the same page in every cache id of
the group, and a (page, kv head) tile of ``page_size x head_dim`` is contiguous.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Tuple

import torch

from ..parts import LayerCache, ModelPlan, PagedCacheSpec
from .pages import CacheLayout, GroupLayout


def cache_groups_of(plan: ModelPlan) -> Tuple[List[PagedCacheSpec], Dict[int, Tuple[int, int]]]:
    """Group the plan's cache ids by what they store.  Returns the group specs and
    cache id -> (group, index inside the group)."""
    specs: List[PagedCacheSpec] = []
    where: Dict[int, Tuple[int, int]] = {}
    counts: List[int] = []
    for entry, run in enumerate(plan.schedule):
        if plan.cache_id(entry) != entry:
            continue
        mixer = plan.layers[run.layer].mixer
        spec = mixer.cache_spec() if mixer is not None else None
        if spec is None:
            continue
        if spec not in specs:
            specs.append(spec)
            counts.append(0)
        g = specs.index(spec)
        where[entry] = (g, counts[g])
        counts[g] += 1
    return specs, where


def bytes_per_page(plan: ModelPlan, page_size: int, dtype_bytes: int) -> List[int]:
    """Bytes of one page id in every group (python/helios/core/allocator.py:136-162:
    2 x layers x page_size x kv heads x head_dim x bytes)."""
    specs, where = cache_groups_of(plan)
    counts = [0] * len(specs)
    for g, _ in where.values():
        counts[g] += 1
    return [2 * counts[g] * page_size * s.num_kv_heads * s.head_dim * dtype_bytes
            for g, s in enumerate(specs)]


def pool_sizes_for_bytes(plan: ModelPlan, page_size: int, dtype_bytes: int, kv_cache_bytes: int,
                         max_slots: Optional[int] = None,
                         largest_portion: Optional[int] = None) -> List[int]:
    """Pages of every cache group that a byte budget pays for
    (python/helios/engine.py:147-155 has one kind of layer and one number).  The groups
    that keep every key get the same number of pages each, since a request needs as many
    in one as in another.  A group with a window W never holds more than W + a portion
    (+ a page at either end) per request, so with ``max_slots`` and ``largest_portion``
    given it gets no more than all slots together can use, and the bytes it leaves go
    to the others."""
    per_page = bytes_per_page(plan, page_size, dtype_bytes)
    specs, _ = cache_groups_of(plan)
    if not specs:
        return []
    share = max(8, kv_cache_bytes // max(1, sum(per_page)))
    sizes: List[Optional[int]] = [None] * len(specs)
    left = kv_cache_bytes
    for g, spec in enumerate(specs):
        if spec.window is not None:
            sizes[g] = share
            if max_slots is not None and largest_portion is not None:
                per_request = -(-(spec.window + largest_portion) // page_size) + 2
                sizes[g] = max(8, min(share, max_slots * per_request))
            left -= sizes[g] * per_page[g]
    full_bytes = sum(per_page[g] for g in range(len(specs)) if sizes[g] is None)
    for g in range(len(specs)):
        if sizes[g] is None:
            sizes[g] = max(8, left // max(1, full_bytes))
    return [int(n) for n in sizes]


class KVCacheManager(CacheLayout):
    """Bookkeeping (``CacheLayout``) plus the tensors."""

    def __init__(self, plan: ModelPlan, page_size: int, num_pages, max_slots: int,
                 dtype: torch.dtype, device, watermark: float = 0.0,
                 poison: Optional[float] = None) -> None:
        specs, where = cache_groups_of(plan)
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(specs)
        if len(num_pages) != len(specs):
            raise ValueError(f"{len(num_pages)} pool sizes for {len(specs)} cache groups")
        super().__init__([GroupLayout(s.window, n) for s, n in zip(specs, num_pages)],
                         page_size, max_slots, watermark)
        self.plan = plan
        self.specs = specs
        self.dtype = dtype
        self.device = torch.device(device)
        self._where = where
        counts = [0] * len(specs)
        for g, _ in where.values():
            counts[g] += 1
        self.storage: List[torch.Tensor] = []
        for g, spec in enumerate(specs):
            # one page more than the pool hands out: padding rows of captured graphs write there
            shape = (counts[g], 2, num_pages[g] + 1, spec.num_kv_heads, page_size, spec.head_dim)
            t = torch.empty(shape, dtype=dtype, device=self.device)
            t.fill_(poison) if poison is not None else t.zero_()
            self.storage.append(t)
        # fixed-size state per request slot, for the mixers that keep one
        self.states: Dict[int, torch.Tensor] = {}
        for entry, run in enumerate(plan.schedule):
            mixer = plan.layers[run.layer].mixer
            spec = mixer.state_spec() if mixer is not None else None
            if spec is not None and plan.cache_id(entry) == entry:
                self.states[entry] = torch.zeros((max_slots,) + tuple(spec.shape),
                                                 dtype=spec.dtype, device=self.device)
        # ... and for the other parts of a block that keep one (a feed-forward, say):
        # cache id -> {id(part): [slots, *shape]}
        self.other_states: Dict[int, Dict[int, torch.Tensor]] = {}
        for entry, run in enumerate(plan.schedule):
            if plan.cache_id(entry) != entry:
                continue
            for part, spec in plan.layers[run.layer].state_specs():
                self.other_states.setdefault(entry, {})[id(part)] = torch.zeros(
                    (max_slots,) + tuple(spec.shape), dtype=spec.dtype, device=self.device)
        self._views: Dict[int, LayerCache] = {}
        #: per group, the id of the spare page no request ever gets
        self.pad_pages: List[int] = list(num_pages)

    # ------------------------------------------------------------------ views
    def layer_cache(self, entry: int) -> Optional[LayerCache]:
        """The pages schedule entry ``entry`` works on (its own, or the ones it reads)."""
        view = self._views.get(entry)
        if view is None:
            cid = self.plan.cache_id(entry)
            if cid not in self._where:
                return None
            g, idx = self._where[cid]
            view = LayerCache(self.storage[g][idx, 0], self.storage[g][idx, 1], g,
                              self.page_size, write=self.plan.schedule[entry].writes_cache)
            self._views[entry] = view
        return view

    def layer_state(self, entry: int) -> Optional[torch.Tensor]:
        return self.states.get(self.plan.cache_id(entry))

    def part_states(self, entry: int) -> Dict[int, torch.Tensor]:
        """id(part) -> state tensor of the parts of schedule entry ``entry`` other than its mixer."""
        return self.other_states.get(self.plan.cache_id(entry), {})

    # ------------------------------------------------------------------ requests
    def admit(self, request_id: Hashable) -> int:
        slot = super().admit(request_id)
        for state in self.states.values():
            state[slot].zero_()
        for states in self.other_states.values():
            for state in states.values():
                state[slot].zero_()
        return slot

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.storage)
