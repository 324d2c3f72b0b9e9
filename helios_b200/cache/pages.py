"""Host-side bookkeeping of cache pages: which page is free, which request holds
which page of which group, and the per-request state slots.  No tensor lives
here, so the scheduler and its tests run without a GPU
(python/helios/core/allocator.py:84-341 keeps the same split: the allocator owns
the mapping, the executor owns the bytes).

A model's cache ids are put into groups by what they store per token (KV heads,
head size, all keys or a window).  Every group has a pool of pages of its own
and every request a block table per group.  Pages are taken when tokens are
about to be written, given back when the request ends, and, in a group with a
window, as soon as the window has passed them; a page that was given back is
handed out again (first freed, first reused).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence


class OutOfPages(RuntimeError):
    """Not enough free pages (or no free slot); nothing was taken."""


class CacheInvariantError(AssertionError):
    pass


class PagePool:
    """Page ids 0..n-1 of one group with a first-in-first-out free list
    (python/helios/core/allocator.py:86-118)."""

    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free: Deque[int] = deque(range(num_pages))
        self._owner: List[Optional[Hashable]] = [None] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int, owner: Hashable) -> List[int]:
        if owner is None:
            raise ValueError("an owner is required")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free")
        pages = [self._free.popleft() for _ in range(n)]
        for p in pages:
            self._owner[p] = owner
        return pages

    def give_back(self, pages: Sequence[int], owner: Hashable) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise CacheInvariantError(f"page {p} does not exist")
            if self._owner[p] is None:
                raise CacheInvariantError(f"page {p} is freed twice")
            if self._owner[p] != owner:
                raise CacheInvariantError(f"page {p} is held by {self._owner[p]!r}, not {owner!r}")
        for p in pages:
            self._owner[p] = None
            self._free.append(p)

    def owner_of(self, page: int) -> Optional[Hashable]:
        return self._owner[page]

    def check_invariants(self) -> None:
        free = list(self._free)
        if len(set(free)) != len(free):
            raise CacheInvariantError("a page is on the free list twice")
        for p in free:
            if self._owner[p] is not None:
                raise CacheInvariantError(f"free page {p} has an owner")
        held = sum(1 for o in self._owner if o is not None)
        if held + len(free) != self.num_pages:
            raise CacheInvariantError(f"{self.num_pages - held - len(free)} pages are lost")


@dataclass(frozen=True)
class GroupLayout:
    """What the bookkeeping has to know of a group."""
    window: Optional[int]      # None: all keys; W: the last W keys
    num_pages: int


@dataclass
class RequestPages:
    slot: int
    length: int = 0                                  # tokens written and committed
    tables: List[List[int]] = field(default_factory=list)   # per group: logical page -> id, -1 once given back
    first_held: List[int] = field(default_factory=list)     # per group: first logical page still held
    version: int = 0                                 # counts the changes of ``tables``
    arrays: dict = field(default_factory=dict)       # group -> (version, tables[group] as int32 array)


class CacheLayout:
    """Block tables, page pools and slots of all live requests."""

    def __init__(self, groups: Sequence[GroupLayout], page_size: int, max_slots: int,
                 watermark: float = 0.0) -> None:
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.groups = list(groups)
        self.pools = [PagePool(g.num_pages) for g in self.groups]
        self.max_slots = max_slots
        self.watermark = watermark
        self._free_slots: Deque[int] = deque(range(max_slots))
        self.requests: Dict[Hashable, RequestPages] = {}

    # ------------------------------------------------------------------ sizes
    def usable_pages(self, group: int) -> int:
        """Pages admission may count on (python/helios/core/allocator.py:183-207)."""
        return int(self.groups[group].num_pages * (1.0 - self.watermark))

    def pages_for_tokens(self, n_tokens: int) -> int:
        return -(-n_tokens // self.page_size)

    def peak_pages(self, group: int, total_tokens: int, largest_portion: int) -> int:
        """Most pages of ``group`` a request of ``total_tokens`` holds at any time when it
        is fed in portions of at most ``largest_portion`` tokens."""
        w = self.groups[group].window
        if w is None:
            return self.pages_for_tokens(total_tokens)
        span = min(total_tokens, w + max(1, largest_portion))
        return min(self.pages_for_tokens(total_tokens), self.pages_for_tokens(span) + 1)

    # ------------------------------------------------------------------ requests
    def has(self, request_id: Hashable) -> bool:
        return request_id in self.requests

    def length(self, request_id: Hashable) -> int:
        return self.requests[request_id].length

    def slot(self, request_id: Hashable) -> int:
        return self.requests[request_id].slot

    def table(self, request_id: Hashable, group: int) -> List[int]:
        return self.requests[request_id].tables[group]

    def table_array(self, request_id: Hashable, group: int):
        """``table`` as an int32 array, rebuilt only when the table has changed (a step's
        metadata copies every live request's table; with long contexts the conversion
        from a list every step costs more than the step's kernels)."""
        import numpy as np
        req = self.requests[request_id]
        hit = req.arrays.get(group)
        if hit is None or hit[0] != req.version:
            hit = (req.version, np.asarray(req.tables[group], dtype=np.int32))
            req.arrays[group] = hit
        return hit[1]

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self, request_id: Hashable) -> int:
        """Give the request a slot and empty block tables."""
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise OutOfPages("no free request slot")
        slot = self._free_slots.popleft()
        n = len(self.groups)
        self.requests[request_id] = RequestPages(slot, 0, [[] for _ in range(n)], [0] * n)
        return slot

    def pages_needed(self, request_id: Hashable, n_new: int) -> List[int]:
        """New pages per group for ``n_new`` more tokens."""
        req = self.requests[request_id]
        want = self.pages_for_tokens(req.length + n_new)
        return [max(0, want - len(t)) for t in req.tables]

    def pages_needed_each(self, request_ids: Sequence[Hashable], n_new: int = 1) -> List[int]:
        """``pages_needed`` summed over many requests that each get ``n_new`` more tokens (a
        decode step of hundreds of requests asks this every step: one loop, no lists)."""
        need = [0] * len(self.groups)
        requests, page = self.requests, self.page_size
        for rid in request_ids:
            req = requests[rid]
            want = -(-(req.length + n_new) // page)
            for g, t in enumerate(req.tables):
                d = want - len(t)
                if d > 0:
                    need[g] += d
        return need

    def extend_each(self, request_ids: Sequence[Hashable], n_new: int = 1) -> None:
        """``extend`` for every request in turn (the caller has made sure of the pages with
        ``pages_needed_each``; a request that finds none raises as ``extend`` does)."""
        requests, page, pools = self.requests, self.page_size, self.pools
        for rid in request_ids:
            req = requests[rid]
            want = -(-(req.length + n_new) // page)
            grow = False
            for g, t in enumerate(req.tables):
                d = want - len(t)
                if d > 0:
                    grow = True
                    if d > pools[g].num_free:         # all of a request's groups, or none
                        raise OutOfPages(f"request {rid!r} needs {d} pages of group {g}, "
                                         f"{pools[g].num_free} free")
            if grow:
                for g, t in enumerate(req.tables):
                    d = want - len(t)
                    if d > 0:
                        t.extend(pools[g].take(d, rid))
                        req.version += 1

    def can_extend(self, request_id: Hashable, n_new: int, keep_free: int = 0) -> bool:
        need = self.pages_needed(request_id, n_new)
        return all(n + keep_free <= pool.num_free for n, pool in zip(need, self.pools))

    def pages_held(self, request_id: Hashable) -> List[int]:
        """Pages per group the request holds now (the ones a window has passed are gone)."""
        req = self.requests[request_id]
        return [len(t) - first for t, first in zip(req.tables, req.first_held)]

    def tokens_that_fit(self, request_id: Hashable, keep_free: Optional[Sequence[int]] = None) -> int:
        """How many more tokens the request can take pages for right now, leaving
        ``keep_free[group]`` pages of every group to others."""
        req = self.requests[request_id]
        fit = None
        for g, (table, pool) in enumerate(zip(req.tables, self.pools)):
            spare = pool.num_free - (keep_free[g] if keep_free is not None else 0)
            n = (len(table) + max(0, spare)) * self.page_size - req.length
            fit = n if fit is None else min(fit, n)
        return max(0, fit) if fit is not None else 1 << 30

    def extend(self, request_id: Hashable, n_new: int) -> None:
        """Take the pages for ``n_new`` more tokens in every group, or none at all."""
        req = self.requests[request_id]
        need = self.pages_needed(request_id, n_new)
        for g, n in enumerate(need):
            if n > self.pools[g].num_free:
                raise OutOfPages(f"request {request_id!r} needs {n} pages of group {g}, "
                                 f"{self.pools[g].num_free} free")
        for g, n in enumerate(need):
            if n:
                req.tables[g].extend(self.pools[g].take(n, request_id))
                req.version += 1

    def commit_each(self, request_ids: Sequence[Hashable], counts: Sequence[int]) -> None:
        """``commit`` for every request of a step; without a window group nothing is given
        back and a commit is a check and an addition."""
        if any(g.window is not None for g in self.groups):
            for rid, n in zip(request_ids, counts):
                self.commit(rid, n)
            return
        requests, page = self.requests, self.page_size
        for rid, n in zip(request_ids, counts):
            req = requests[rid]
            length = req.length + n
            want = -(-length // page)
            for t in req.tables:
                if want > len(t):
                    raise CacheInvariantError(f"request {rid!r} commits tokens it has no pages for")
            req.length = length

    def commit(self, request_id: Hashable, n_new: int) -> None:
        """``n_new`` tokens were written.  In a group with a window W the next token, at
        position ``length``, sees keys from ``length - W + 1`` on; pages wholly before
        that are given back now."""
        req = self.requests[request_id]
        have = min((len(t) for t in req.tables), default=self.pages_for_tokens(req.length + n_new))
        if self.pages_for_tokens(req.length + n_new) > have:
            raise CacheInvariantError(f"request {request_id!r} commits tokens it has no pages for")
        req.length += n_new
        for g, group in enumerate(self.groups):
            if group.window is None:
                continue
            first_needed = max(0, req.length - group.window + 1) // self.page_size
            table = req.tables[g]
            dead = []
            while req.first_held[g] < min(first_needed, len(table)):
                j = req.first_held[g]
                dead.append(table[j])
                table[j] = -1
                req.first_held[g] += 1
            if dead:
                self.pools[g].give_back(dead, request_id)
                req.version += 1

    def release(self, request_id: Hashable) -> None:
        """The request is over (or preempted): all pages and the slot go back."""
        req = self.requests.pop(request_id)
        for g, table in enumerate(req.tables):
            live = [p for p in table if p >= 0]
            if live:
                self.pools[g].give_back(live, request_id)
        self._free_slots.append(req.slot)

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost, held twice or free while held; tables cover the length
        (the spirit of python/helios/core/allocator.py:513-597)."""
        for pool in self.pools:
            pool.check_invariants()
        slots = [r.slot for r in self.requests.values()] + list(self._free_slots)
        if sorted(slots) != list(range(self.max_slots)):
            raise CacheInvariantError("a slot is lost or held twice")
        for g, pool in enumerate(self.pools):
            seen: Dict[int, Hashable] = {}
            for rid, req in self.requests.items():
                table = req.tables[g]
                if len(table) < self.pages_for_tokens(req.length):
                    raise CacheInvariantError(f"request {rid!r} has tokens without pages")
                for j, p in enumerate(table):
                    if p < 0:
                        if self.groups[g].window is None or j >= req.first_held[g]:
                            raise CacheInvariantError(f"request {rid!r} lost page {j} of group {g}")
                        continue
                    if j < req.first_held[g]:
                        raise CacheInvariantError(f"request {rid!r} holds a page behind its window")
                    if p in seen:
                        raise CacheInvariantError(f"page {p} of group {g} is held by {seen[p]!r} and {rid!r}")
                    seen[p] = rid
                    if pool.owner_of(p) != rid:
                        raise CacheInvariantError(f"page {p} of group {g}: pool names another owner")
            if len(seen) != pool.num_used:
                raise CacheInvariantError(f"group {g}: {pool.num_used - len(seen)} pages held by nobody")
