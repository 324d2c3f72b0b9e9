"""The cache's bookkeeping (no GPU): no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; reuse is first-freed-first."""
import random

import pytest

from helios_b200.cache import (CacheInvariantError, CacheLayout, GroupLayout, OutOfPages, PagePool)


def test_pool_take_and_give_back():
    pool = PagePool(4)
    a = pool.take(3, "a")
    assert a == [0, 1, 2] and pool.num_free == 1
    with pytest.raises(OutOfPages):
        pool.take(2, "b")
    assert pool.num_free == 1          # nothing was taken
    pool.give_back([1], "a")
    with pytest.raises(CacheInvariantError):
        pool.give_back([1], "a")        # freed twice
    with pytest.raises(CacheInvariantError):
        pool.give_back([0], "b")        # not the holder
    assert pool.take(2, "b") == [3, 1]  # first freed, first reused
    pool.check_invariants()


def test_tables_grow_by_pages_and_release_gives_all_back():
    lay = CacheLayout([GroupLayout(None, 10)], page_size=4, max_slots=2)
    lay.admit("r")
    assert lay.pages_needed("r", 9) == [3]
    lay.extend("r", 9)
    lay.commit("r", 9)
    assert lay.table("r", 0) == [0, 1, 2] and lay.length("r") == 9
    assert lay.pages_needed("r", 3) == [0] and lay.pages_needed("r", 4) == [1]
    lay.extend("r", 4)
    lay.commit("r", 4)
    lay.check_invariants()
    lay.release("r")
    assert lay.pools[0].num_free == 10 and lay.num_free_slots == 2
    with pytest.raises(KeyError):
        lay.release("r")


def test_extend_is_all_or_nothing_across_groups():
    lay = CacheLayout([GroupLayout(None, 8), GroupLayout(None, 2)], page_size=4, max_slots=2)
    lay.admit("r")
    with pytest.raises(OutOfPages):
        lay.extend("r", 12)             # group 1 has only 2 pages
    assert lay.pools[0].num_free == 8 and lay.pools[1].num_free == 2
    lay.check_invariants()


def test_commit_without_pages_is_an_error():
    lay = CacheLayout([GroupLayout(None, 8)], page_size=4, max_slots=1)
    lay.admit("r")
    with pytest.raises(CacheInvariantError):
        lay.commit("r", 3)


def test_window_group_gives_pages_back_as_the_window_passes():
    lay = CacheLayout([GroupLayout(None, 16), GroupLayout(6, 16)], page_size=4, max_slots=1)
    lay.admit("r")
    for _ in range(40):
        lay.extend("r", 1)
        lay.commit("r", 1)
        lay.check_invariants()
        n = lay.length("r")
        first_needed = max(0, n - 6 + 1) // 4       # page of the oldest key the next token sees
        held = [j for j, p in enumerate(lay.table("r", 1)) if p >= 0]
        assert held[0] == first_needed
        assert all(p >= 0 for p in lay.table("r", 0))
    assert lay.pools[1].num_used <= 3
    assert lay.pools[0].num_used == 10
    lay.release("r")
    assert lay.pools[1].num_free == 16


def test_slots_run_out_and_come_back():
    lay = CacheLayout([GroupLayout(None, 8)], page_size=4, max_slots=2)
    assert {lay.admit("a"), lay.admit("b")} == {0, 1}
    with pytest.raises(OutOfPages):
        lay.admit("c")
    with pytest.raises(ValueError):
        lay.admit("a")
    lay.release("a")
    assert lay.admit("c") == 0
    lay.check_invariants()


@pytest.mark.parametrize("seed", range(40))
def test_random_walk_keeps_the_invariants(seed):
    """python/helios/tests: the reference walks its allocator the same way
    (tests/allocator/test_allocator.py:238-308)."""
    rng = random.Random(seed)
    page = rng.choice([1, 4, 16])
    groups = [GroupLayout(None, rng.randint(6, 24))]
    if rng.random() < 0.7:
        groups.append(GroupLayout(rng.randint(1, 40), rng.randint(6, 24)))
    lay = CacheLayout(groups, page, max_slots=4)
    lengths = {}
    next_id = 0
    for _ in range(300):
        op = rng.random()
        if op < 0.25 and lay.num_free_slots:
            lay.admit(next_id)
            lengths[next_id] = 0
            next_id += 1
        elif op < 0.8 and lengths:
            rid = rng.choice(list(lengths))
            n = rng.choice([1, 1, 1, 2, 7, 30])
            free_before = [p.num_free for p in lay.pools]
            try:
                lay.extend(rid, n)
            except OutOfPages:
                assert [p.num_free for p in lay.pools] == free_before
            else:
                lay.commit(rid, n)
                lengths[rid] += n
        elif lengths:
            rid = rng.choice(list(lengths))
            lay.release(rid)
            del lengths[rid]
        lay.check_invariants()
        for rid, n in lengths.items():
            assert lay.length(rid) == n
    for rid in list(lengths):
        lay.release(rid)
    assert all(p.num_free == p.num_pages for p in lay.pools)
    lay.check_invariants()


def test_corruption_is_detected():
    lay = CacheLayout([GroupLayout(None, 8)], page_size=4, max_slots=2)
    lay.admit("a")
    lay.admit("b")
    lay.extend("a", 8)
    lay.extend("b", 4)
    lay.table("b", 0)[0] = lay.table("a", 0)[0]      # the same page in two tables
    with pytest.raises(CacheInvariantError):
        lay.check_invariants()
