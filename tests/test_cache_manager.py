"""The cache manager: no page lost, held twice or freed twice, under random orders of
requests; window release; state slots."""

from __future__ import annotations

import random

import pytest

from emberserve_b200.cache.manager import CacheManager, OutOfPages, PagePool, plan_groups
from emberserve_b200.parts.base import FixedState, PagedKV

FULL = PagedKV(2, 16, None)
WIN = PagedKV(2, 16, 10)
STATE = FixedState((4, 8))


def manager(needs, pages=8, page_size=4, slots=3):
    return CacheManager(plan_groups(needs), pages, page_size, slots)


def test_groups_by_equal_needs():
    groups = plan_groups([FULL, WIN, FULL, STATE, WIN, PagedKV(1, 16, None)])
    assert [g.entries for g in groups] == [(0, 2), (1, 4), (3,), (5,)]
    assert [g.paged for g in groups] == [True, True, False, True]


def test_pages_needed_admit_extend_release():
    m = manager([FULL])
    assert [m.pages_needed(n) for n in (0, 1, 4, 5, 8, 9)] == [0, 1, 1, 2, 2, 3]
    m.admit(1, 9)
    assert m.table(1, 0) == [0, 1, 2] and m.num_free_pages() == 5
    m.extend(1, 12)  # fills the last page: no new page
    assert m.table(1, 0) == [0, 1, 2]
    m.extend(1, 13)
    assert m.table(1, 0) == [0, 1, 2, 3]
    m.admit(2, 16)
    assert m.num_free_pages() == 0 and not m.can_admit(1)
    with pytest.raises(OutOfPages):
        m.extend(1, 17)
    assert m.num_tokens(1) == 13 and m.table(1, 0) == [0, 1, 2, 3]  # untouched by the failure
    with pytest.raises(OutOfPages):
        m.admit(3, 1)
    assert not m.has_sequence(3)
    m.release(1)
    m.release(1)  # idempotent
    # freed pages go to the back and come out again in that order, contents and all
    m.admit(4, 8)
    assert m.table(4, 0) == [0, 1]
    m.check()


def test_double_free_is_caught():
    pool = PagePool(2)
    p = pool.take()
    pool.give(p)
    with pytest.raises(AssertionError):
        pool.give(p)


def test_window_gives_pages_back_once_passed():
    m = manager([FULL, WIN], pages=16, page_size=4)
    m.admit(7, 30)
    assert len(m.table(7, 0)) == 8 and len(m.table(7, 1)) == 8
    m.commit(7, 9)  # next query at 9 reads keys >= 0 (9 - 10 + 1): nothing passed
    assert m.table(7, 1).count(-1) == 0
    m.commit(7, 13)  # reads keys >= 4: page 0 passed
    assert m.table(7, 1)[:2] == [-1, m.table(7, 1)[1]] and m.table(7, 1)[1] >= 0
    m.commit(7, 30)  # reads keys >= 21: pages 0..4 passed
    assert [p < 0 for p in m.table(7, 1)] == [True] * 5 + [False] * 3
    assert m.table(7, 0).count(-1) == 0  # the group that keeps everything keeps everything
    assert m.num_free_pages(1) == 16 - 3
    m.check()
    for n in range(31, 60):
        m.extend(7, n)
        m.commit(7, n)
        live = [p for p in m.table(7, 1) if p >= 0]
        assert len(live) <= 10 // 4 + 2
        m.check()
    m.release(7)
    assert m.num_free_pages(0) == 16 and m.num_free_pages(1) == 16
    m.check()


def test_state_slots():
    m = manager([FULL, STATE], slots=2)
    m.admit(1, 3)
    m.admit(2, 3)
    assert {m.state_slot(1), m.state_slot(2)} == {0, 1}
    assert m.take_fresh_slots() == [0, 1] and m.take_fresh_slots() == []
    assert not m.can_admit(1)
    with pytest.raises(OutOfPages):
        m.admit(3, 1)
    m.release(1)
    m.admit(3, 1)
    assert m.state_slot(3) == 0 and m.take_fresh_slots() == [0]  # handed out again: zero it
    m.check()
    plain = manager([FULL])
    plain.admit(1, 1)
    assert plain.state_slot(1) == -1 and plain.can_admit(1)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_duplicate_a_page(seed):
    rng = random.Random(seed)
    needs = [FULL, WIN, STATE] if seed % 2 else [FULL]
    m = manager(needs, pages=24, page_size=4, slots=5)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.3:
            n = rng.randint(1, 30)
            if m.can_admit(n):
                m.admit(next_id, n)
                live[next_id] = 0
                next_id += 1
            else:
                with pytest.raises(OutOfPages):
                    m.admit(next_id, n)
        elif op < 0.75 and live:
            sid = rng.choice(list(live))
            total = m.num_tokens(sid)
            if live[sid] < total:  # compute a portion of what is reserved
                live[sid] = rng.randint(live[sid] + 1, total)
                m.commit(sid, live[sid])
            else:
                try:
                    m.extend(sid, total + 1)
                except OutOfPages:
                    assert m.num_tokens(sid) == total
        elif live:
            sid = rng.choice(list(live))
            m.release(sid)
            del live[sid]
        m.check()
    for sid in list(live):
        m.release(sid)
    m.check()
    st = m.stats()
    assert st.num_free == st.num_pages and st.free_state_slots == st.num_state_slots
