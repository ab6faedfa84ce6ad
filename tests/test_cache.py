"""Cache bookkeeping on the host: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import numpy as np
import pytest

from inferllm_b200.cache import CacheError, CacheFull, FixedState, IndexPool, PagedKV, PageLedger, SequenceCache


def test_pool_alloc_free_reuse():
    p = IndexPool(4, "slot")
    a = p.alloc(3)
    assert a == [0, 1, 2] and p.n_free == 1
    p.free([1])
    assert p.alloc(2) == [1, 3]
    with pytest.raises(CacheFull):
        p.alloc(1)
    p.free([0, 1, 2, 3])
    p.check()
    assert p.n_free == 4


def test_pool_double_free_and_foreign():
    p = IndexPool(2, "page")
    (a,) = p.alloc(1)
    p.free([a])
    with pytest.raises(CacheError, match="twice"):
        p.free([a])
    with pytest.raises(CacheError, match="does not exist"):
        p.free([7])


def test_ledger_grows_by_pages_and_rows():
    led = PageLedger(num_pages=8, page_size=4, num_slots=2)
    assert led.pages_needed(0, 9) == 3
    led.reserve(0, 9)
    led.reserve(1, 4)
    led.reserve(0, 12)   # still three pages
    assert led.pool.n_held == 4
    led.reserve(0, 13)
    assert led.pool.n_held == 5
    row = np.empty(6, np.int32)
    led.row(0, 6, row)
    assert list(row) == [0, 1, 2, 4, -1, -1]
    led.check()
    led.release_all(0)
    led.release_all(1)
    assert led.pool.n_free == 8
    led.check()


def test_window_releases_pages_that_left_the_window():
    led = PageLedger(num_pages=16, page_size=4, num_slots=1, window=6)
    led.reserve(0, 20)
    assert led.pool.n_held == 5
    led.release_outside_window(0, 20)      # next query at 20 sees keys 15..20 -> pages 3, 4
    assert sorted(led.pages[0]) == [3, 4]
    led.reserve(0, 21)
    assert sorted(led.pages[0]) == [3, 4, 5]
    row = np.empty(8, np.int32)
    led.row(0, 8, row)
    assert list(row[:3]) == [-1, -1, -1] and row[5] >= 0
    led.check()
    # window 1 with a length that is a multiple of the page: every page can go, none comes back
    led1 = PageLedger(num_pages=4, page_size=4, num_slots=1, window=1)
    led1.reserve(0, 8)
    led1.release_outside_window(0, 8)
    assert led1.pages[0] == {}
    led1.reserve(0, 9)
    assert sorted(led1.pages[0]) == [2]


def _cache(num_slots=3, num_pages=6, page=4, max_len=16, extra=None):
    reqs = {0: PagedKV(2, 8), 1: PagedKV(2, 8)}
    reqs.update(extra or {})
    return SequenceCache(reqs, num_slots, num_pages, page, max_len)


def test_groups_by_need():
    c = _cache(extra={2: PagedKV(2, 8, window=5), 3: FixedState((4,)), 4: None})
    st = c.stats()
    assert len(st["paged"]) == 2 and len(st["states"]) == 1
    assert st["paged"][0]["entries"] == [0, 1] and st["paged"][1]["entries"] == [2] and st["paged"][1]["request"]["window"] == 5
    assert st["states"][0]["entries"] == [3] and st["states"][0]["request"]["shape"] == [4]


def test_step_plan_positions_and_tables():
    c = _cache()
    s0, s1 = c.alloc_slot(), c.alloc_slot()
    plan = c.plan_step([s0, s1], [5, 2])
    assert plan.past == [0, 0] and plan.tables[0].shape == (2, 4)
    assert list(plan.tables[0][0]) == [0, 1, -1, -1] and list(plan.tables[0][1]) == [2, -1, -1, -1]
    c.commit_step(plan)
    assert c.seq_len[s0] == 5 and c.seq_len[s1] == 2
    plan = c.plan_step([s1, s0], [1, 4])
    assert plan.past == [2, 5]
    c.commit_step(plan)
    assert c.seq_len[s0] == 9 and c.pages_free() == [2]
    c.check()


def test_misuse_is_refused():
    c = _cache()
    s = c.alloc_slot()
    with pytest.raises(CacheError, match="not live"):
        c.plan_step([2], [1])
    with pytest.raises(CacheError, match="twice"):
        c.plan_step([s, s], [1, 1])
    with pytest.raises(CacheError, match="at least one token"):
        c.plan_step([s], [0])
    with pytest.raises(CacheError, match="maximum sequence length"):
        c.plan_step([s], [17])
    c.free_slot(s)
    with pytest.raises(CacheError, match="freed twice"):
        c.free_slot(s)


def test_out_of_pages_is_all_or_nothing():
    c = _cache(num_pages=3)
    a, b = c.alloc_slot(), c.alloc_slot()
    with pytest.raises(CacheFull):
        c.plan_step([a, b], [8, 8])       # needs 4 pages
    assert c.pages_free() == [3]          # nothing was taken
    c.commit_step(c.plan_step([a, b], [8, 4]))
    with pytest.raises(CacheFull):
        c.plan_step([b], [1])
    c.free_slot(a)
    c.commit_step(c.plan_step([b], [1]))  # a's pages are used again
    c.check()


def test_out_of_slots():
    c = _cache(num_slots=2)
    c.alloc_slot(), c.alloc_slot()
    with pytest.raises(CacheFull):
        c.alloc_slot()


def test_freed_slots_and_pages_are_used_again():
    c = _cache(num_slots=2, num_pages=4)
    for _ in range(5):
        a, b = c.alloc_slot(), c.alloc_slot()
        assert {a, b} == {0, 1}
        c.commit_step(c.plan_step([a, b], [7, 3]))
        c.commit_step(c.plan_step([a], [1]))
        c.free_slot(b)
        c.commit_step(c.plan_step([a], [1]))
        c.free_slot(a)
        assert c.pages_free() == [4] and c.slots_free == 2
        c.check()


def test_random_walk_keeps_invariants():
    rng = random.Random(3)
    c = _cache(num_slots=5, num_pages=12, page=4, max_len=24, extra={2: PagedKV(1, 8, window=6)})
    live = {}
    for _ in range(600):
        r = rng.random()
        if r < 0.25 and c.slots_free:
            live[c.alloc_slot()] = 0
        elif r < 0.45 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            chosen = rng.sample(list(live), rng.randint(1, len(live)))
            qs = [rng.randint(1, 6) if live[s] == 0 else 1 for s in chosen]
            try:
                plan = c.plan_step(chosen, qs)
            except CacheFull:
                before = c.pages_free()
                assert before == c.pages_free()
                continue
            except CacheError:
                continue  # beyond the longest sequence
            for s, q, past in zip(chosen, qs, plan.past):
                assert past == live[s]
                live[s] += q
            c.commit_step(plan)
            for s in chosen:
                assert c.seq_len[s] == live[s]
                # every position the next query may see has a page
                for gi, g in enumerate(c.stats()["paged"]):
                    w = g["request"]["window"]
                    lo = max(0, live[s] - w + 1) if w else 0
                    held = c.pages_of(gi, s)
                    for pos in range(lo, live[s]):
                        assert pos // 4 in held
        c.check()
    c.reset()
    c.check()
    assert c.slots_free == 5 and c.pages_free() == [12, 12]


def test_a_step_that_failed_gives_its_pages_back():
    """Pages are reserved when a step is planned; if the step does not run, `abandon_step` returns
    what it had reserved and the sequence stands where it stood."""
    c = _cache(num_pages=6)
    s = c.alloc_slot()
    c.commit_step(c.plan_step([s], [3]))
    free = c.pages_free()
    plan = c.plan_step([s], [9])
    assert c.pages_free()[0] == free[0] - 2
    c.abandon_step(plan)
    assert c.pages_free() == free and c.seq_len[s] == 3
    c.check()
    c.commit_step(c.plan_step([s], [9]))
    assert c.seq_len[s] == 12
    c.check()
