"""Iteration-level scheduler: admits requests, cuts prompts into portions under a
token budget, decodes, finishes and frees (python/helios/core/scheduler.py:158-1206,
without its priority classes, prefix cache, swap tier and speculation).

It is pure host code over the cache's bookkeeping (``cache.pages.CacheLayout``)
and an executor with one method, so tests drive it with a scripted executor and
no GPU.  It uses no clock, no random numbers and no unordered iteration: the same
requests give the same steps (scheduler.py:7-20).

What happens when pages run out
-------------------------------
* Pages are taken portion by portion, when a portion is put into a step, not for
  the whole prompt at admission (the reference takes them all at admission:
  scheduler.py:597-627).  What a request will hold at most is its *claim*:
  ``CacheLayout.peak_pages`` per group, all its pages where every key is kept,
  window + portion where a window is.  Admission wants the claim plus one page
  to grow, beside what the running requests still have to take of their claims,
  free now in every group; else the request waits and a later, smaller one may
  pass it (scheduler.py:466-489).  After ``reservation_after_steps`` steps of
  being passed, the head of the queue alone may be admitted (scheduler.py:421-439).
* ``add_request`` judges by the same claim against the usable pool: what it
  accepts, an idle scheduler can admit.  A request that could never fit is refused
  when added, or finished with ``length`` if it grew to that size.
* A portion is cut to the pages that are free (beyond the page each decoding
  request needs next); a request that gets none waits a step.  If nobody can take
  a step, the newest running request is preempted.
* Before a step, every decoding request must be able to take its next page; if
  not, the newest running request is preempted: its pages are freed, its outputs
  are kept, and it goes to the FRONT of the queue to be run again from its first
  token (scheduler.py:682-763).  The only running request is never preempted.
* If the page for a freshly sampled token cannot be had, the request is preempted
  the same way, or, when it is the only one and nothing waits, finished with
  ``length`` (scheduler.py:951-978).
After a preemption the prompt AND the outputs made so far are run again in
portions and the last portion samples the next new token, so the output equals
that of an undisturbed run.  (The reference re-runs the prompt only and samples
a duplicate token: scheduler.py:810-831 slices ``prompt_token_ids``.)
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Protocol

from ..cache.pages import CacheLayout, OutOfPages
from .types import FinishReason, Request, SamplingParams, SeqState, Sequence


@dataclass
class SchedulerConfig:
    """python/helios/core/scheduler.py:49-107, the options that remain."""
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048
    max_model_len: int = 4096
    enable_chunked_prefill: bool = True
    reservation_after_steps: int = 32

    def validate(self) -> None:
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0 or self.max_model_len <= 0:
            raise ValueError("max_num_seqs, max_num_batched_tokens and max_model_len must be positive")


#: stands for a token that is not known on the host yet (``PlanItem.fed_on_device``)
PLACEHOLDER = 0


@dataclass
class PlanItem:
    """A request's tokens for this step (python/helios/core/execstep.py:24-49: a decode
    is an item of one token)."""
    seq_id: int
    token_ids: List[int]
    start_pos: int
    sample: bool                  # the item reaches the end of the sequence: sample the next token
    params: SamplingParams
    rng_seed: int = 0
    rng_offset: int = 0           # number of tokens this request has sampled so far
    fed_on_device: bool = False   # the token is the one the step before is sampling

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)


@dataclass
class StepPlan:
    step_id: int
    items: List[PlanItem] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(i.num_tokens for i in self.items)

    @property
    def is_empty(self) -> bool:
        return not self.items


class ExecFault(Exception):
    """The executor could not run the step for these sequences
    (python/helios/core/execstep.py:129-156)."""

    def __init__(self, message: str, seq_ids: Optional[List[int]] = None) -> None:
        super().__init__(message)
        self.seq_ids = list(seq_ids or [])


class Executor(Protocol):
    def run(self, plan: StepPlan) -> Dict[int, int]:
        """seq_id -> sampled token, for every item with ``sample``."""


@dataclass
class SchedulerStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    faults: int = 0
    max_running: int = 0


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheLayout) -> None:
        config.validate()
        self.config = config
        self.cache = cache
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.finished: List[Sequence] = []
        self.seqs: Dict[int, Sequence] = {}
        self.stats = SchedulerStats()
        self.step_t = 0
        self._next_seq_id = 0
        self._skipped_head_steps = 0
        self._decode_need: List[int] = [0] * len(cache.groups)
        self.last_plan: Optional[StepPlan] = None

    # ------------------------------------------------------------------ queue
    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _claim(self, total_tokens: int) -> List[int]:
        """Most pages per group a request of ``total_tokens`` holds at any time."""
        portion = self.config.max_num_batched_tokens
        if not self.config.enable_chunked_prefill:
            portion = max(portion, total_tokens)
        return [self.cache.peak_pages(g, total_tokens, portion) for g in range(len(self.cache.groups))]

    def _fits_ever(self, total_tokens: int) -> bool:
        return all(c + 1 <= self.cache.usable_pages(g)
                   for g, c in enumerate(self._claim(total_tokens)))

    def _unclaimed(self, seqs) -> List[int]:
        """Pages per group that ``seqs`` have yet to take of their claims."""
        out = [0] * len(self.cache.groups)
        for seq in seqs:
            held = self.cache.pages_held(seq.seq_id)
            for g, c in enumerate(self._claim(seq.total_tokens)):
                out[g] += max(0, c - held[g])
        return out

    def add_request(self, request: Request, rng_seed: int = 0) -> int:
        """Validate and queue (python/helios/core/scheduler.py:219-276)."""
        if request.prompt_len == 0:
            raise ValueError("empty prompt")
        if request.prompt_len >= self.config.max_model_len:
            raise ValueError(f"prompt of {request.prompt_len} tokens does not fit max_model_len "
                             f"{self.config.max_model_len}")
        request.params.validate()
        if not self._fits_ever(request.prompt_len):
            raise ValueError(f"prompt of {request.prompt_len} tokens needs more cache pages than "
                             "the pool has")
        seq = Sequence(self._next_seq_id, request, rng_seed=rng_seed)
        self._next_seq_id += 1
        request.arrival_step = self.step_t
        self.seqs[seq.seq_id] = seq
        self.waiting.append(seq)
        return seq.seq_id

    def abort(self, seq_id: int) -> bool:
        seq = self.seqs.get(seq_id)
        if seq is None or seq.is_finished:
            return False
        if seq in self.waiting:
            self.waiting.remove(seq)
        if seq in self.running:
            self.running.remove(seq)
        self._retire(seq, FinishReason.ABORTED, SeqState.ABORTED)
        return True

    def take_finished(self) -> List[Sequence]:
        out, self.finished = self.finished, []
        return out

    # ------------------------------------------------------------------ one iteration
    def step(self, executor: Executor) -> Dict[int, int]:
        """python/helios/core/scheduler.py:312-365."""
        plan = self.schedule()
        if plan.is_empty:
            return {}
        try:
            tokens = executor.run(plan)
        except ExecFault as fault:
            self.fault(plan, fault)
            return {}
        self.launched(plan)
        self.complete(plan, tokens)
        return tokens

    # The three phases of an iteration, for an executor that works asynchronously:
    # ``schedule`` decides the step, ``launched`` records that its tokens are in the cache
    # (true, in the device's order of work, once the step is enqueued), ``complete`` takes
    # the sampled tokens.  Between ``launched(p)`` and ``complete(p)`` a caller may ask
    # ``schedule_ahead(p)`` for the step after it and launch that too.
    def schedule(self) -> StepPlan:
        self.step_t += 1
        self.stats.steps += 1
        self._admit()
        self._ensure_running_can_progress()
        plan = self._build_plan()
        self.last_plan = plan
        return plan

    def launched(self, plan: StepPlan) -> None:
        items, by_id = plan.items, self.seqs
        counts = [len(item.token_ids) for item in items]
        self.cache.commit_each([item.seq_id for item in items], counts)
        prefill = decode = 0
        for item, n in zip(items, counts):
            seq = by_id[item.seq_id]
            seq.num_computed_tokens += n
            if n > 1 or item.start_pos < len(seq.request.prompt_token_ids):
                prefill += n
            else:
                decode += 1
        self.stats.prefill_tokens += prefill
        self.stats.decode_tokens += decode

    def complete(self, plan: StepPlan, tokens: Dict[int, int],
                 ahead: Optional[StepPlan] = None) -> None:
        """``ahead``: the step that was launched after ``plan`` with ``schedule_ahead``; the
        places of its tokens are taken already."""
        reserved = {i.seq_id for i in ahead.items} if ahead is not None else ()
        for item in plan.items:
            if not item.sample:
                continue
            seq = self.seqs[item.seq_id]
            if seq.state is not SeqState.RUNNING:
                continue          # finished, aborted or preempted while the step ran
            if item.seq_id not in tokens:
                raise RuntimeError(f"the executor returned no token for sequence {item.seq_id}")
            self._accept(seq, int(tokens[item.seq_id]), reserve=item.seq_id not in reserved)
        self.stats.max_running = max(self.stats.max_running, len(self.running))

    def fault(self, plan: StepPlan, fault: ExecFault) -> None:
        self._handle_fault(plan, fault)

    def schedule_ahead(self, prev: StepPlan) -> Optional[StepPlan]:
        """The step after ``prev`` while ``prev`` still runs: every request of ``prev`` gets
        as its one token the token ``prev`` is sampling for it (``PLACEHOLDER`` here; the
        executor feeds it on the device), in the order of ``prev``'s items.  Only when that
        is certainly the step ``schedule`` would make if no request stops: nothing waits (or
        nothing that waits could be admitted: all slots are taken),
        ``prev`` sampled for every running request, none of them reaches its length with
        the token in flight, and the places for the new tokens can be had.  Else None, and
        nothing has changed.  A request that does stop on the token in flight is dropped by
        ``complete``; what the step ahead computed for it is ignored."""
        if prev.is_empty or len(prev.items) != len(self.running):
            return None
        if len(prev.items) > self.config.max_num_batched_tokens:
            return None
        if self.waiting and not self._admission_closed():
            return None           # a waiting request might join the next step
        seqs = []
        by_id, running, most_len = self.seqs, SeqState.RUNNING, self.config.max_model_len
        for item in prev.items:                # (hundreds of requests a step: no property chains here)
            seq = by_id[item.seq_id]
            if not item.sample or seq.state is not running:
                return None
            outputs = len(seq.output_token_ids)
            total = len(seq.request.prompt_token_ids) + outputs
            if total != seq.num_computed_tokens:
                return None       # ``launched(prev)`` has not been called
            if outputs + 1 >= seq.request.params.max_tokens:
                return None
            if total + 1 >= most_len:
                return None
            seqs.append(seq)
        ids = [seq.seq_id for seq in seqs]
        need = self.cache.pages_needed_each(ids, 1)
        if any(n > pool.num_free for n, pool in zip(need, self.cache.pools)):
            return None
        self.step_t += 1
        self.stats.steps += 1
        if self.waiting:
            self._skipped_head_steps += 1      # as ``_admit`` counts a step without admission
        plan = StepPlan(self.step_t)
        self.cache.extend_each(ids, 1)
        items = plan.items
        for seq in seqs:
            items.append(PlanItem(seq.seq_id, [PLACEHOLDER], seq.num_computed_tokens, True,
                                  seq.request.params, seq.rng_seed, len(seq.output_token_ids) + 1, True))
        self.last_plan = plan
        return plan

    # ------------------------------------------------------------------ admission
    def _admission_closed(self) -> bool:
        """No waiting request can be admitted whatever its size: every slot is taken, or the
        running requests use up the token budget."""
        return len(self.running) >= self.config.max_num_seqs or \
            self.config.max_num_batched_tokens - len(self.running) <= 0

    def _admit(self) -> None:
        if not self.waiting:
            self._skipped_head_steps = 0
            return
        if self._admission_closed():
            self._skipped_head_steps += 1      # nobody can be admitted: the head is passed once more
            return
        # preempted requests were put to the front and stay there; the rest in arrival order
        pending = sorted(self.waiting, key=lambda s: (0 if s.state is SeqState.PREEMPTED else 1,
                                                      s.request.arrival_step, s.seq_id))
        blocked_head = None
        if pending and self._skipped_head_steps >= self.config.reservation_after_steps:
            blocked_head = pending[0]
        budget = self.config.max_num_batched_tokens - len(self.running)
        admitted: List[Sequence] = []
        for seq in pending:
            if len(self.running) + len(admitted) >= self.config.max_num_seqs:
                break
            if budget <= 0:
                break
            if blocked_head is not None and seq is not blocked_head:
                continue
            new_tokens = seq.num_pending_tokens
            chunk = min(new_tokens, budget)
            if not self.config.enable_chunked_prefill and new_tokens > budget:
                if self.running or admitted:
                    break
                chunk = new_tokens
            if not self._fits_ever(seq.total_tokens):
                self.waiting.remove(seq)
                self._retire(seq, FinishReason.LENGTH if seq.num_output_tokens else FinishReason.ABORTED)
                continue
            if not self._reserve(seq, admitted):
                continue          # does not fit now; a smaller one behind it may
            seq.state = SeqState.RUNNING
            admitted.append(seq)
            budget -= chunk
        if pending and pending[0] not in admitted and pending[0] in self.waiting:
            self._skipped_head_steps += 1
        else:
            self._skipped_head_steps = 0
        for seq in admitted:
            self.waiting.remove(seq)
            self.running.append(seq)

    def _reserve(self, seq: Sequence, admitted: List[Sequence]) -> bool:
        """A slot, if the request's claim and a page to grow are free in every group beside
        what the running requests (and those admitted in this step) have yet to take.
        The pages themselves are taken portion by portion (``_build_plan``)."""
        cache = self.cache
        if cache.num_free_slots == 0:
            return False
        promised = self._unclaimed(self.running + admitted)
        for g, c in enumerate(self._claim(seq.total_tokens)):
            if c + 1 + promised[g] > cache.pools[g].num_free:
                return False
        cache.admit(seq.seq_id)
        return True

    # ------------------------------------------------------------------ progress guarantee
    def _ensure_running_can_progress(self) -> None:
        """Every decoding request must be able to place its next sampled token, and when
        nobody decodes, some request must be able to take a portion; else the newest
        running request gives way (python/helios/core/scheduler.py:682-712).  Leaves in
        ``_decode_need`` the pages per group that portions must leave to the decoders."""
        guard = 0
        self._decode_need = [0] * len(self.cache.groups)
        while self.running and guard <= self.config.max_num_seqs + 1:
            guard += 1
            need = [0] * len(self.cache.groups)
            decoding = False
            for seq in self.running:
                if seq.num_pending_tokens == 1:
                    decoding = True
                    # its next sampled token will need a place
                    for g, n in enumerate(self.cache.pages_needed(seq.seq_id, 2)):
                        need[g] += n
            if all(n <= pool.num_free for n, pool in zip(need, self.cache.pools)):
                if decoding or any(self.cache.tokens_that_fit(s.seq_id) > 0 for s in self.running):
                    self._decode_need = need
                    return
            victim = self._pick_victim()
            if victim is None:
                if not decoding:
                    # alone, and not a page to be had for its next portion: it cannot go on
                    self._finish(self.running[0], FinishReason.LENGTH)
                return
            self._preempt(victim)

    def _pick_victim(self) -> Optional[Sequence]:
        """The newest running request; never the only one
        (python/helios/core/scheduler.py:714-742)."""
        if len(self.running) <= 1:
            return None
        return max(self.running, key=lambda s: s.seq_id)

    def _preempt(self, seq: Sequence) -> None:
        if seq in self.running:
            self.running.remove(seq)
        if self.cache.has(seq.seq_id):
            self.cache.release(seq.seq_id)
        seq.reset_for_recompute()
        self.waiting.appendleft(seq)
        self.stats.preemptions += 1

    # ------------------------------------------------------------------ the plan
    def _build_plan(self) -> StepPlan:
        """Decoding requests first claim one token each; portions of prompts share the
        rest of the budget in admission order (python/helios/core/scheduler.py:790-861)."""
        plan = StepPlan(self.step_t)
        budget = self.config.max_num_batched_tokens
        # a decoding request holds the place of its one token already (``_accept`` took it);
        # a request of one token that was just admitted takes it like any portion
        decoding = [s for s in self.running if s.num_pending_tokens == 1
                    and not any(self.cache.pages_needed(s.seq_id, 1))]
        placed = {s.seq_id for s in decoding}
        prefilling = [s for s in self.running if s.num_pending_tokens >= 1 and s.seq_id not in placed]
        decoding = decoding[:budget]
        prefill_budget = max(0, budget - len(decoding))
        for seq in prefilling:
            if prefill_budget <= 0:
                break
            n = min(seq.num_pending_tokens, prefill_budget)
            if not self.config.enable_chunked_prefill:
                n = seq.num_pending_tokens
                if n > prefill_budget and (plan.items or decoding):
                    continue
            # the portion's pages are taken now; it is cut to what is free beyond the page
            # every decoding request needs next (without chunking: all or nothing)
            fit = self.cache.tokens_that_fit(seq.seq_id, self._decode_need)
            if fit < n:
                if not self.config.enable_chunked_prefill or fit <= 0:
                    continue
                n = fit
            self.cache.extend(seq.seq_id, n)
            plan.items.append(self._item(seq, n))
            prefill_budget -= n
        for seq in decoding:
            plan.items.append(self._item(seq, 1))
        return plan

    def _item(self, seq: Sequence, n: int) -> PlanItem:
        start = seq.num_computed_tokens
        toks = seq.token_slice(start, n)
        return PlanItem(seq.seq_id, toks, start, sample=(start + n >= seq.total_tokens),
                        params=seq.request.params, rng_seed=seq.rng_seed,
                        rng_offset=seq.num_output_tokens)

    # ------------------------------------------------------------------ results
    def _accept(self, seq: Sequence, token: int, reserve: bool = True) -> None:
        """python/helios/core/scheduler.py:913-949."""
        params = seq.request.params
        seq.output_token_ids.append(token)
        if seq.first_token_step is None:
            seq.first_token_step = self.step_t
        seq.last_token_step = self.step_t
        if token in params.stop_token_ids:
            self._finish(seq, FinishReason.STOP)
            return
        if seq.num_output_tokens >= params.max_tokens:
            self._finish(seq, FinishReason.LENGTH)
            return
        if seq.total_tokens >= self.config.max_model_len:
            self._finish(seq, FinishReason.LENGTH)
            return
        if not reserve:
            return
        try:
            self.cache.extend(seq.seq_id, 1)       # the place of the new token
        except OutOfPages:
            self._preempt_for_oom(seq)

    def _preempt_for_oom(self, seq: Sequence) -> None:
        if len(self.running) <= 1 and not self.waiting:
            self._finish(seq, FinishReason.LENGTH)
            return
        self._preempt(seq)

    def _finish(self, seq: Sequence, reason: FinishReason) -> None:
        if seq in self.running:
            self.running.remove(seq)
        self._retire(seq, reason)

    def _retire(self, seq: Sequence, reason: FinishReason,
                state: SeqState = SeqState.FINISHED) -> None:
        if self.cache.has(seq.seq_id):
            self.cache.release(seq.seq_id)
        seq.state = state
        seq.finish_reason = reason
        self.finished.append(seq)
        self.stats.finished += 1

    def _handle_fault(self, plan: StepPlan, fault: ExecFault) -> None:
        """Nothing of the step counts; the affected sequences (all of the step's if none
        are named) are run again from their first token
        (python/helios/core/scheduler.py:1057-1073)."""
        self.stats.faults += 1
        affected = fault.seq_ids or [i.seq_id for i in plan.items]
        for sid in affected:
            seq = self.seqs.get(sid)
            if seq is not None and seq in self.running:
                self._preempt(seq)

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        self.cache.check_invariants()
        live = {s.seq_id for s in self.running}
        if len(live) != len(self.running):
            raise AssertionError("a sequence runs twice")
        for s in self.waiting:
            if s.seq_id in live:
                raise AssertionError(f"sequence {s.seq_id} both waits and runs")
            if self.cache.has(s.seq_id):
                raise AssertionError(f"waiting sequence {s.seq_id} holds cache pages")
        for s in self.running:
            if not self.cache.has(s.seq_id):
                raise AssertionError(f"running sequence {s.seq_id} has no cache entry")
            if self.cache.length(s.seq_id) != s.num_computed_tokens:
                raise AssertionError(f"sequence {s.seq_id}: cache length and computed tokens differ")
        held = set(self.cache.requests)
        if held != live:
            raise AssertionError(f"cache entries {sorted(held)} vs running {sorted(live)}")
