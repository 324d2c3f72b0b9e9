"""The scheduler's decisions, with a scripted executor and no GPU
(the reference tests its scheduler the same way: tests/scheduler/test_scheduler.py:48-80)."""
import pytest

from helios_b200.cache import CacheLayout, GroupLayout
from helios_b200.engine.scheduler import ExecFault, Scheduler, SchedulerConfig
from helios_b200.engine.types import FinishReason, Request, SamplingParams, SeqState


class ScriptedExecutor:
    """Returns token 1000 + seq_id * 100 + (number of outputs so far); can fail at a step."""

    def __init__(self, fault_at=None, fault_seqs=None, eos_after=None):
        self.plans = []
        self.fault_at = fault_at
        self.fault_seqs = fault_seqs
        self.eos_after = eos_after or {}

    def run(self, plan):
        self.plans.append(plan)
        if self.fault_at is not None and plan.step_id == self.fault_at:
            raise ExecFault("scripted", self.fault_seqs)
        out = {}
        for item in plan.items:
            if item.sample:
                if self.eos_after.get(item.seq_id) == item.rng_offset:
                    out[item.seq_id] = 2
                else:
                    out[item.seq_id] = 1000 + item.seq_id * 100 + item.rng_offset
        return out


def make(num_pages=64, page=4, budget=16, max_seqs=8, max_len=256, window=None, chunked=True,
         watermark=0.0):
    groups = [GroupLayout(None, num_pages)]
    if window:
        groups.append(GroupLayout(window, num_pages))
    cache = CacheLayout(groups, page, max_slots=max_seqs, watermark=watermark)
    sched = Scheduler(SchedulerConfig(max_num_seqs=max_seqs, max_num_batched_tokens=budget,
                                      max_model_len=max_len, enable_chunked_prefill=chunked), cache)
    return sched, cache


def req(n, max_tokens=4, rid="r", **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, **kw))


def run_all(sched, ex, limit=500):
    steps = 0
    while sched.has_work:
        sched.step(ex)
        sched.check_invariants()
        steps += 1
        assert steps < limit, "the scheduler does not finish"
    return steps


def test_request_validation():
    sched, _ = make(num_pages=4, page=4, max_len=32)
    with pytest.raises(ValueError):
        sched.add_request(req(0))
    with pytest.raises(ValueError):
        sched.add_request(req(32))                       # >= max_model_len
    with pytest.raises(ValueError):
        sched.add_request(req(13))                       # 4 pages + 1 to grow > pool
    with pytest.raises(ValueError):
        sched.add_request(Request("x", [1], SamplingParams(max_tokens=0)))
    with pytest.raises(ValueError):
        sched.add_request(Request("x", [1], SamplingParams(top_p=0.0)))
    sched.add_request(req(12))


def test_prompt_is_cut_into_portions_under_the_budget():
    sched, _ = make(budget=16)
    sched.add_request(req(40, max_tokens=3))
    ex = ScriptedExecutor()
    run_all(sched, ex)
    sizes = [[i.num_tokens for i in p.items] for p in ex.plans]
    assert sizes == [[16], [16], [8], [1], [1]]
    starts = [p.items[0].start_pos for p in ex.plans]
    assert starts == [0, 16, 32, 40, 41]
    assert [p.items[0].sample for p in ex.plans] == [False, False, True, True, True]
    seq = sched.take_finished()[0]
    assert seq.output_token_ids == [1000, 1001, 1002] and seq.finish_reason is FinishReason.LENGTH


def test_decodes_claim_budget_first_and_share_a_step_with_portions():
    sched, _ = make(budget=8)
    sched.add_request(req(3, max_tokens=6, rid="a"))
    ex = ScriptedExecutor()
    sched.step(ex)                                       # a: whole prompt
    sched.add_request(req(20, max_tokens=2, rid="b"))
    sched.step(ex)
    plan = ex.plans[-1]
    by_seq = {i.seq_id: i for i in plan.items}
    assert by_seq[0].num_tokens == 1 and by_seq[0].start_pos == 3      # a decodes
    assert by_seq[1].num_tokens == 7 and by_seq[1].start_pos == 0      # b gets what is left
    assert plan.num_tokens == 8
    run_all(sched, ex)
    assert all(p.num_tokens <= 8 for p in ex.plans)


def test_portions_down_to_one_token_when_decodes_take_the_budget():
    sched, _ = make(budget=4, max_seqs=4)
    for i in range(3):
        sched.add_request(req(2, max_tokens=30, rid=f"d{i}"))
    ex = ScriptedExecutor()
    sched.step(ex)
    sched.step(ex)
    sched.add_request(req(9, max_tokens=1, rid="long"))
    sched.step(ex)
    sizes = {i.seq_id: i.num_tokens for i in ex.plans[-1].items}
    assert sizes[3] == 1 and sum(sizes.values()) == 4


def test_without_chunking_a_long_prompt_runs_alone():
    sched, _ = make(budget=8, chunked=False)
    sched.add_request(req(3, max_tokens=2, rid="short"))
    sched.add_request(req(20, max_tokens=1, rid="long"))
    ex = ScriptedExecutor()
    run_all(sched, ex)
    for p in ex.plans:
        if any(i.num_tokens == 20 for i in p.items):
            assert len(p.items) == 1
    assert sorted(s.request.request_id for s in sched.take_finished()) == ["long", "short"]


def test_stop_token_finishes_and_is_kept():
    sched, _ = make()
    sched.add_request(req(5, max_tokens=10, stop_token_ids=[2]))
    ex = ScriptedExecutor(eos_after={0: 2})
    run_all(sched, ex)
    seq = sched.take_finished()[0]
    assert seq.output_token_ids == [1000, 1001, 2] and seq.finish_reason is FinishReason.STOP


def test_max_model_len_finishes_with_length():
    sched, _ = make(max_len=10)
    sched.add_request(req(7, max_tokens=50))
    run_all(sched, ScriptedExecutor())
    seq = sched.take_finished()[0]
    assert seq.total_tokens == 10 and seq.finish_reason is FinishReason.LENGTH


def test_a_request_that_does_not_fit_waits_and_a_smaller_one_passes():
    sched, cache = make(num_pages=10, page=4, budget=64)
    sched.add_request(req(20, max_tokens=8, rid="big1"))       # 5 pages + growth
    sched.add_request(req(20, max_tokens=2, rid="big2"))       # does not fit beside big1
    sched.add_request(req(4, max_tokens=2, rid="small"))
    ex = ScriptedExecutor()
    sched.step(ex)
    running = {s.request.request_id for s in sched.running}
    assert running == {"big1", "small"}
    assert [s.request.request_id for s in sched.waiting] == ["big2"]
    run_all(sched, ex)
    assert len(sched.take_finished()) == 3


def test_head_of_queue_gets_a_reservation_after_being_passed():
    sched, _ = make(num_pages=10, page=4, budget=64)
    sched.config.reservation_after_steps = 3
    sched.add_request(req(20, max_tokens=40, rid="runs"))
    ex = ScriptedExecutor()
    sched.step(ex)
    sched.add_request(req(30, max_tokens=1, rid="starved"))     # 8 pages + 1: not beside "runs"
    admitted_small = 0
    for i in range(12):
        sched.add_request(req(2, max_tokens=1, rid=f"s{i}"))
        sched.step(ex)
        sched.check_invariants()
    small_running_late = [s for s in sched.running if s.request.request_id.startswith("s")]
    waiting_small = [s for s in sched.waiting if s.request.request_id.startswith("s")]
    assert waiting_small, "after the reservation small requests must wait behind the head"
    run_all(sched, ex)
    done = {s.request.request_id for s in sched.take_finished()}
    assert "starved" in done


def test_pages_run_out_before_a_step_newest_is_preempted_and_output_is_unchanged():
    # two requests whose growth cannot both be served: the newer one is preempted,
    # recomputed with its outputs so far, and still produces the same tokens
    def outputs(num_pages):
        sched, _ = make(num_pages=num_pages, page=4, budget=64)
        sched.add_request(req(7, max_tokens=14, rid="old"))
        sched.add_request(req(7, max_tokens=14, rid="new"))
        ex = ScriptedExecutor()
        run_all(sched, ex)
        fin = {s.request.request_id: s for s in sched.take_finished()}
        return fin, sched.stats.preemptions, ex

    roomy, n0, _ = outputs(64)
    tight, n1, ex = outputs(8)
    assert n0 == 0 and n1 >= 1
    for rid in ("old", "new"):
        assert tight[rid].output_token_ids == roomy[rid].output_token_ids
        assert len(tight[rid].output_token_ids) == 14
    assert tight["new"].preempt_count >= 1 and tight["old"].preempt_count == 0
    # the recomputed portion brought prompt AND outputs, and sampled the NEXT token
    redo = [i for p in ex.plans for i in p.items if i.seq_id == 1 and i.start_pos == 0][1]
    assert redo.num_tokens > 7 and redo.rng_offset == redo.num_tokens - 7


def test_preempted_request_goes_to_the_front_of_the_queue():
    sched, _ = make(num_pages=8, page=4, budget=64)
    sched.add_request(req(7, max_tokens=14, rid="old"))
    sched.add_request(req(7, max_tokens=14, rid="new"))
    ex = ScriptedExecutor()
    sched.step(ex)
    sched.add_request(req(3, max_tokens=1, rid="later"))
    while sched.stats.preemptions == 0:
        sched.step(ex)
    assert sched.waiting[0].request.request_id == "new"
    assert sched.waiting[0].state is SeqState.PREEMPTED


def test_the_only_running_request_is_never_preempted_and_ends_with_length():
    sched, cache = make(num_pages=4, page=4, budget=64, max_len=200)
    sched.add_request(req(8, max_tokens=100))
    run_all(sched, ScriptedExecutor())
    seq = sched.take_finished()[0]
    assert seq.finish_reason is FinishReason.LENGTH and seq.preempt_count == 0
    # the pool holds 16 tokens; the token sampled from the 16th needs no place of its own
    assert seq.total_tokens == 17 and cache.pools[0].num_pages * 4 == 16
    assert cache.pools[0].num_free == 4


def test_fault_preempts_the_named_sequences_only():
    sched, _ = make()
    sched.add_request(req(5, max_tokens=6, rid="a"))
    sched.add_request(req(5, max_tokens=6, rid="b"))
    ex = ScriptedExecutor(fault_at=3, fault_seqs=[1])
    run_all(sched, ex)
    fin = {s.request.request_id: s for s in sched.take_finished()}
    assert fin["a"].preempt_count == 0 and fin["b"].preempt_count == 1
    assert fin["a"].output_token_ids == [1000 + k for k in range(6)]
    assert fin["b"].output_token_ids == [1100 + k for k in range(6)]
    assert sched.stats.faults == 1


def test_abort_frees_everything():
    sched, cache = make()
    a = sched.add_request(req(9, max_tokens=50, rid="a"))
    b = sched.add_request(req(9, max_tokens=50, rid="b"))
    ex = ScriptedExecutor()
    sched.step(ex)
    assert sched.abort(a) and not sched.abort(a)
    sched.check_invariants()
    sched.abort(b)
    assert cache.pools[0].num_free == 64 and not sched.has_work
    assert {s.finish_reason for s in sched.take_finished()} == {FinishReason.ABORTED}


def test_window_group_lets_long_requests_share_a_small_pool():
    sched, cache = make(num_pages=40, page=4, budget=16, window=8)
    for i in range(3):
        sched.add_request(req(30, max_tokens=20, rid=f"w{i}"))
    run_all(sched, ScriptedExecutor())
    assert len(sched.take_finished()) == 3
    assert all(p.num_free == p.num_pages for p in cache.pools)


def make_groups(groups, page, budget, max_seqs=4, max_len=4096):
    cache = CacheLayout(groups, page, max_slots=max_seqs)
    sched = Scheduler(SchedulerConfig(max_num_seqs=max_seqs, max_num_batched_tokens=budget,
                                      max_model_len=max_len), cache)
    return sched, cache


@pytest.mark.parametrize("groups,page,budget,prompt", [
    ([GroupLayout(8, 10)], 4, 16, 100),                          # every group has a window
    ([GroupLayout(32, 10)], 16, 16, 159),
    ([GroupLayout(None, 10), GroupLayout(32, 5)], 16, 16, 100),  # pools of different size
])
def test_what_add_request_accepts_is_admitted_and_finishes(groups, page, budget, prompt):
    # pages are taken portion by portion, so a window pool far smaller than the prompt
    # serves it; the request never holds more than its claim
    sched, cache = make_groups(groups, page, budget)
    sched.add_request(req(prompt, max_tokens=30))
    ex = ScriptedExecutor()
    steps = 0
    while sched.has_work:
        sched.step(ex)
        sched.check_invariants()
        for g, pool in enumerate(cache.pools):
            assert pool.num_used <= cache.peak_pages(g, prompt + 30, budget) + 1
        steps += 1
        assert steps < 200, "accepted, but never admitted or never finished"
    seq = sched.take_finished()[0]
    assert seq.output_token_ids == [1000 + k for k in range(30)]
    assert all(p.num_free == p.num_pages for p in cache.pools)
    # ... and what cannot fit even alone is refused when it is added
    too_long = max(g.num_pages for g in groups if g.window is None) * page + 1 \
        if any(g.window is None for g in groups) else None
    if too_long is not None:
        with pytest.raises(ValueError):
            sched.add_request(req(too_long))


def test_pages_are_taken_portion_by_portion():
    sched, cache = make(num_pages=64, page=4, budget=16)
    sched.add_request(req(40, max_tokens=2))
    ex = ScriptedExecutor()
    used = []
    while sched.has_work:
        sched.step(ex)
        used.append(cache.pools[0].num_used)
    assert used[:3] == [4, 8, 11]          # 16, 32, 40 tokens and the place of the first new one


def test_admission_counts_what_running_requests_have_yet_to_take():
    # two prompts of 5 pages each in a pool of 10: the second may not come in on the pages
    # the first has not taken yet
    sched, cache = make(num_pages=10, page=4, budget=8)
    sched.add_request(req(20, max_tokens=2, rid="first"))
    sched.add_request(req(20, max_tokens=2, rid="second"))
    ex = ScriptedExecutor()
    sched.step(ex)
    assert [s.request.request_id for s in sched.running] == ["first"]
    assert cache.pools[0].num_used == 2
    run_all(sched, ex)
    assert sched.stats.preemptions == 0 and len(sched.take_finished()) == 2


def test_a_portion_is_cut_to_the_free_pages_and_decoders_keep_their_next_page():
    # two decoding requests grow into the pages a later prompt was admitted on: its portions
    # shrink to what is free beyond the decoders' next pages, and nobody loses a token
    def run(num_pages):
        sched, cache = make(num_pages=num_pages, page=4, budget=4)
        sched.add_request(req(3, max_tokens=30, rid="d0"))
        sched.add_request(req(3, max_tokens=30, rid="d1"))
        ex = ScriptedExecutor()
        for _ in range(12):
            sched.step(ex)
        sched.add_request(req(10, max_tokens=3, rid="long"))
        sizes = []
        while sched.has_work:
            sched.step(ex)
            sched.check_invariants()
            sizes += [i.num_tokens for i in ex.plans[-1].items if i.seq_id == 2 and not i.sample]
            assert len(ex.plans) < 300
        out = {s.request.request_id: s.output_token_ids for s in sched.take_finished()}
        return out, sizes, sched.stats.preemptions

    roomy, sizes0, _ = run(64)
    tight, sizes1, preempted = run(12)
    assert tight == roomy and len(tight) == 3
    assert sizes0 and all(n == 2 for n in sizes0)
    assert preempted or any(n < 2 for n in sizes1) or len(sizes1) != len(sizes0)


def test_preemption_with_a_window_group_gives_the_same_outputs():
    def outputs(num_pages):
        sched, _ = make(num_pages=num_pages, page=4, budget=8, window=8)
        sched.add_request(req(7, max_tokens=14, rid="old"))
        sched.add_request(req(7, max_tokens=14, rid="new"))
        run_all(sched, ScriptedExecutor())
        return {s.request.request_id: s.output_token_ids for s in sched.take_finished()}, \
            sched.stats.preemptions

    roomy, n0 = outputs(64)
    tight, n1 = outputs(8)
    assert n0 == 0 and n1 >= 1 and tight == roomy


def test_same_requests_same_steps():
    # python/helios/core/scheduler.py:7-20: no clock, no randomness
    def trace():
        sched, _ = make(num_pages=12, page=4, budget=12, max_seqs=3)
        ex = ScriptedExecutor()
        for i, n in enumerate([9, 14, 5, 11, 3]):
            sched.add_request(req(n, max_tokens=5 + i, rid=f"r{i}"))
        run_all(sched, ex)
        return [[(i.seq_id, i.start_pos, i.num_tokens, i.sample) for i in p.items] for p in ex.plans]

    assert trace() == trace()


def test_scheduler_source_uses_no_clock_or_random():
    import inspect
    import helios_b200.engine.scheduler as mod

    src = inspect.getsource(mod)
    assert "import time" not in src and "import random" not in src


# ---------------------------------------------------------------------- running ahead
def run_all_ahead(sched, ex, arrivals=None, limit=2000):
    """Drives the scheduler the way the engine does when it launches the next decode step
    before it has read the tokens of the running one.  ``arrivals``: {call number: request}."""
    arrivals = dict(arrivals or {})
    in_flight, calls, ahead_steps = None, 0, 0
    while sched.has_work or arrivals:
        if calls in arrivals:
            sched.add_request(arrivals.pop(calls))
        calls += 1
        assert calls < limit, "the scheduler does not finish"
        if in_flight is None:
            plan = sched.schedule()
            if plan.is_empty:
                continue
            tokens = ex.run(plan)
            sched.launched(plan)
        else:
            plan, tokens = in_flight
            in_flight = None
        sched.check_invariants()
        ahead = sched.schedule_ahead(plan)
        if ahead is not None:
            assert all(i.fed_on_device and i.num_tokens == 1 and i.sample for i in ahead.items)
            assert [i.seq_id for i in ahead.items] == [i.seq_id for i in plan.items]
            ahead_tokens = ex.run(ahead)
            sched.launched(ahead)
            sched.check_invariants()
            ahead_steps += 1
        sched.complete(plan, tokens, ahead)
        sched.check_invariants()
        if ahead is not None and any(not sched.seqs[i.seq_id].is_finished for i in ahead.items):
            in_flight = (ahead, ahead_tokens)
    return ahead_steps


@pytest.mark.parametrize("seed", range(12))
def test_running_ahead_gives_the_same_outputs_and_loses_no_page(seed):
    import random
    rng = random.Random(seed)
    n_req = rng.randint(2, 7)
    shapes = [(rng.randint(1, 30), rng.randint(1, 25)) for _ in range(n_req)]
    eos = {i: rng.randint(0, 20) for i in range(n_req) if rng.random() < 0.5}
    late = {rng.randint(3, 30): i for i in range(n_req) if i and rng.random() < 0.4}
    pages, page = rng.choice([(24, 4), (40, 4), (12, 16), (200, 2)])
    window = rng.choice([None, 8])

    def run(ahead):
        sched, cache = make(num_pages=pages, page=page, budget=rng_budget, max_seqs=4, window=window)
        ex = ScriptedExecutor(eos_after=eos)
        reqs = [Request(f"r{i}", list(range(1, n + 1)), SamplingParams(max_tokens=m, stop_token_ids=[2]))
                for i, (n, m) in enumerate(shapes)]
        arrivals = {}
        for i, r in enumerate(reqs):
            if i in late.values():
                arrivals[[k for k, v in late.items() if v == i][0]] = r
            else:
                sched.add_request(r)
        n_ahead = 0
        if ahead:
            n_ahead = run_all_ahead(sched, ex, arrivals)
        else:
            calls = 0
            while sched.has_work or arrivals:
                if calls in arrivals:
                    sched.add_request(arrivals.pop(calls))
                calls += 1
                sched.step(ex)
                sched.check_invariants()
        assert all(p.num_free == p.num_pages for p in cache.pools)
        out = {s.request.request_id: (list(s.output_token_ids), s.finish_reason)
               for s in sched.take_finished()}
        return out, n_ahead

    rng_budget = rng.choice([8, 16, 64])
    plain, _ = run(False)
    ahead, n_ahead = run(True)
    assert ahead == plain
    assert len(plain) == n_req
    AHEAD_STEPS.append(n_ahead)


AHEAD_STEPS = []


def test_running_ahead_was_exercised():
    assert sum(AHEAD_STEPS) > 50


def test_running_ahead_is_used_for_plain_decoding_and_stops_for_arrivals_and_lengths():
    sched, cache = make(num_pages=64, page=4, budget=32, max_seqs=4)
    for i in range(3):
        sched.add_request(req(5 + i, max_tokens=10, rid=f"r{i}"))
    ex = ScriptedExecutor()
    plan = sched.schedule()
    ex.run(plan)
    sched.launched(plan)
    ahead = sched.schedule_ahead(plan)            # all three sample their first token
    assert ahead is not None and [i.start_pos for i in ahead.items] == [5, 6, 7]
    assert [i.rng_offset for i in ahead.items] == [1, 1, 1]
    # asked twice for the same step: the first answer stands, nothing is taken twice
    used = [p.num_used for p in cache.pools]
    sched.launched(ahead)
    sched.complete(plan, {0: 11, 1: 12, 2: 13}, ahead)
    assert used == [p.num_used for p in cache.pools]
    sched.check_invariants()
    # something waits: the next step must be scheduled in the ordinary way
    sched.add_request(req(3, rid="late"))
    assert sched.schedule_ahead(ahead) is None
    sched.complete(ahead, {0: 21, 1: 22, 2: 23})
    sched.check_invariants()
    assert [sched.seqs[i].output_token_ids for i in range(3)] == [[11, 21], [12, 22], [13, 23]]
    # the token in flight is the last one a request may make: no step ahead
    sched2, _ = make()
    sched2.add_request(req(4, max_tokens=2, rid="short"))
    p1 = sched2.schedule()
    sched2.launched(p1)
    p2 = sched2.schedule_ahead(p1)
    assert p2 is not None
    sched2.launched(p2)
    sched2.complete(p1, {0: 7}, p2)
    assert sched2.schedule_ahead(p2) is None      # output 2 of 2 is in flight
    sched2.complete(p2, {0: 8})
    assert sched2.take_finished()[0].output_token_ids == [7, 8]


def test_running_ahead_goes_on_while_those_that_wait_cannot_be_admitted():
    """With every slot taken a waiting request changes nothing about the next step, so the
    step ahead may be made; once a slot is free it may not."""
    sched, cache = make(num_pages=64, page=4, budget=32, max_seqs=2)
    sched.add_request(Request("a", [1, 2, 3], SamplingParams(max_tokens=9, stop_token_ids=[2])))
    sched.add_request(Request("b", [1, 2, 3, 4], SamplingParams(max_tokens=9, stop_token_ids=[2])))
    sched.add_request(Request("c", [1, 2], SamplingParams(max_tokens=3, stop_token_ids=[2])))
    p1 = sched.schedule()
    assert [i.seq_id for i in p1.items] == [0, 1] and len(sched.waiting) == 1
    sched.launched(p1)
    p2 = sched.schedule_ahead(p1)
    assert p2 is not None and [i.seq_id for i in p2.items] == [0, 1]
    sched.launched(p2)
    sched.complete(p1, {0: 40, 1: 2}, p2)         # "b" stops: a slot is free, "c" can come in
    sched.check_invariants()
    assert sched.schedule_ahead(p2) is None
    sched.complete(p2, {0: 41, 1: 99})
    p3 = sched.schedule()
    assert sorted(i.seq_id for i in p3.items) == [0, 2]
    ex = ScriptedExecutor()
    sched.launched(p3)
    sched.complete(p3, ex.run(p3))
    run_all_ahead(sched, ex)
    out = {s.request.request_id: s.output_token_ids for s in sched.take_finished()}
    assert out["b"] == [2] and out["a"][:2] == [40, 41] and len(out["c"]) == 3
    assert all(p.num_free == p.num_pages for p in cache.pools)


def test_a_request_that_stops_on_the_token_in_flight_is_dropped_from_the_step_ahead():
    sched, cache = make(num_pages=16, page=4)
    sched.add_request(Request("a", [1, 2, 3], SamplingParams(max_tokens=9, stop_token_ids=[2])))
    sched.add_request(Request("b", [1, 2, 3, 4, 5], SamplingParams(max_tokens=9, stop_token_ids=[2])))
    p1 = sched.schedule()
    sched.launched(p1)
    p2 = sched.schedule_ahead(p1)
    sched.launched(p2)
    sched.complete(p1, {0: 2, 1: 50}, p2)         # "a" stops
    sched.check_invariants()
    assert sched.seqs[0].finish_reason is FinishReason.STOP and sched.seqs[0].output_token_ids == [2]
    p3 = sched.schedule_ahead(p2)                 # p2 no longer covers exactly the running requests
    assert p3 is None
    sched.complete(p2, {0: 99, 1: 51})            # the token computed for "a" is ignored
    assert sched.seqs[0].output_token_ids == [2] and sched.seqs[1].output_token_ids == [50, 51]
    sched.check_invariants()


def test_sequences_are_entities_not_values():
    """Membership tests on the running list must not compare token lists field by field
    (with hundreds of running requests that made every step quadratic)."""
    sched, _ = make()
    a = sched.add_request(req(5, rid="same"))
    b = sched.add_request(req(5, rid="same"))
    sa, sb = sched.seqs[a], sched.seqs[b]
    assert sa is not sb and sa != sb and sa == sa
    assert sb not in [sa]


def test_token_slice_equals_slicing_the_whole_list():
    sched, _ = make()
    sid = sched.add_request(req(7, rid="s"))
    seq = sched.seqs[sid]
    seq.output_token_ids.extend([101, 102, 103, 104])
    whole = seq.all_token_ids()
    for start in range(0, 12):
        for n in range(0, 13 - start):
            assert seq.token_slice(start, n) == whole[start:start + n], (start, n)


def test_captured_steps_pad_the_request_count_by_less_than_a_quarter():
    """``EngineCore.padded_requests``: never fewer than asked, exact up to 8, the same for a
    count and for what it was padded to, never more than a quarter on top, few distinct sizes."""
    from helios_b200.engine.core import EngineCore

    sizes = set()
    for n in range(1, 1025):
        p = EngineCore.padded_requests(n)
        assert p >= n and EngineCore.padded_requests(p) == p
        assert p == n if n <= 8 else 4 * (p - n) < n
        sizes.add(p)
    assert len(sizes) <= 8 + 4 * 7 and sorted(sizes)[:12] == [1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16]


def test_decode_attention_slices_and_warps_by_the_size_of_the_step(monkeypatch):
    """``ops.decode_splits`` / ``ops.decode_warps`` with the cluster capacities of a device of
    148 SMs: few requests run clusters of eight-warp blocks, eight requests clusters of four
    slices, many requests whole contexts; a slice never has fewer than 128 keys, and eight warps
    only where each has 64 keys."""
    from helios_b200.csrc import ops

    four = {1: 296, 2: 148, 3: 98, 4: 71, 5: 56, 6: 48, 7: 40, 8: 34}
    eight = {1: 148, 2: 74, 3: 48, 4: 35, 5: 28, 6: 24, 7: 20, 8: 16}
    monkeypatch.setattr(ops, "sm_count", lambda device=None: 148)
    monkeypatch.setattr(ops, "decode_cluster_capacity",
                        lambda head_dim, size, warps=4: (eight if warps == 8 else four)[size])

    def plan(requests, kv_heads, context, head_dim=128):
        s = ops.decode_splits(requests, kv_heads, context, head_dim)
        return s, ops.decode_warps(requests * kv_heads, s, head_dim, context)

    assert plan(1, 8, 4096) == (8, 8) and plan(2, 8, 4096) == (8, 8)
    assert plan(4, 8, 4096) == (8, 4)          # 32 clusters of 8 four-warp blocks, no merge kernel
    assert plan(8, 8, 4096) == (4, 4)
    assert plan(64, 8, 4096) == (1, 4) and plan(256, 2, 1024, 64) == (1, 4)
    assert plan(9, 8, 4096)[0] > 1 and plan(9, 8, 4096)[1] == 4     # 72 pairs: no room for clusters of 4
    assert plan(1, 2, 1024, 64)[1] == 4        # 1,024 keys over 6 to 8 slices: too few for eight warps
    for requests in (1, 3, 8, 20, 100):
        for context in (128, 200, 1000, 5000):
            s, w = plan(requests, 8, context)
            assert 1 <= s <= max(1, context // 128)
            assert w == 4 or context >= 64 * 8 * s
    monkeypatch.setattr(ops, "ATTENTION_DECODE_WIDE_BLOCKS", False)
    assert plan(1, 8, 4096)[1] == 4
