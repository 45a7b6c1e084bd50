"""The cache manager: no page lost, held twice or freed twice, under random orders of requests (CPU)."""
import random

import pytest

from cbis_b200.kernels.library import host


def make(groups, max_requests=4):
    h = host()
    return h.CacheManager([h.GroupSpec(ps, n, w) for ps, n, w in groups], max_requests)


def test_grows_at_the_page_edge():
    # reference: tests/correctness_test.cpp:28-53
    m = make([(16, 8, 0)])
    s = m.admit(1)
    assert m.append(s, 16) and m.block_table(s, 0) == [0]
    assert m.append(s, 1) and m.block_table(s, 0) == [0, 1] and m.free_pages(0) == 6
    assert m.token_slot(s, 0, 16) == 1 * 16 + 0 and m.token_slot(s, 0, 5) == 5
    assert m.check() == ""


def test_exhaustion_is_all_or_nothing_and_pages_come_back():
    # reference: tests/correctness_test.cpp:55-68 (there a failed ensure_capacity keeps a partial allocation)
    m = make([(8, 4, 0)])
    a, b = m.admit(1), m.admit(2)
    assert m.append(a, 20)                       # 3 pages
    assert not m.can_append(b, 9) and not m.append(b, 9)
    assert m.block_table(b, 0) == [] and m.length(b) == 0 and m.free_pages(0) == 1
    assert m.max_appendable(b, 100) == 8 and m.max_appendable(a, 100) == 12
    m.release(a)
    assert m.free_pages(0) == 4 and m.append(b, 9)
    assert m.block_table(b, 0) == [2, 1]         # LIFO: the pages freed last are used first
    assert m.check() == ""


def test_requests_hold_disjoint_pages():
    # reference: tests/correctness_test.cpp:81-90
    m = make([(4, 16, 0)])
    slots = [m.admit(i) for i in range(4)]
    for k, s in enumerate(slots):
        assert m.append(s, 3 + 4 * k)
    pages = [p for s in slots for p in m.block_table(s, 0)]
    assert len(pages) == len(set(pages)) and m.check() == ""


def test_slots_run_out_and_return():
    m = make([(4, 16, 0)], max_requests=2)
    a, b = m.admit(1), m.admit(2)
    assert {a, b} == {0, 1} and m.admit(3) == -1
    m.release(a)
    assert m.admit(4) == a and m.request_id(a) == 4 and m.length(a) == 0
    with pytest.raises(ValueError):
        m.append(3, 1)
    m.release(b)
    with pytest.raises(ValueError):
        m.release(b)                               # freeing twice is refused


def test_window_group_gives_pages_back_as_the_window_passes():
    m = make([(4, 32, 0), (4, 6, 8)])             # a full group and a window of 8 keys
    s = m.admit(1)
    assert m.append(s, 10)
    assert m.release_out_of_window(s) == 0        # next query at 10 reads keys 3..10: page 0 (0..3) still needed
    assert m.append(s, 2)                          # length 12: next query reads 5..12
    assert m.release_out_of_window(s) == 1 and m.block_table(s, 1)[0] == -1
    assert m.block_table(s, 0)[0] >= 0            # the full group keeps everything
    for _ in range(40):                            # 40 more tokens fit into 6 pages of 4 only because pages return
        assert m.append(s, 1)
        m.release_out_of_window(s)
        assert m.check() == ""
    live = [p for p in m.block_table(s, 1) if p >= 0]
    assert len(live) <= 3 and m.length(s) == 52
    with pytest.raises(IndexError):
        m.token_slot(s, 1, 0)
    m.release(s)
    assert m.free_pages(1) == 6 and m.free_pages(0) == 32 and m.check() == ""


def test_fits_at_all_counts_window_groups_by_what_is_live():
    m = make([(4, 5, 8)])
    assert m.fits_at_all(1000, 4)                 # 8 + 4 + 4 tokens live at most: 4 pages
    assert not m.fits_at_all(1000, 16)
    assert not make([(4, 5, 0)]).fits_at_all(21, 4)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    groups = [(rng.choice([2, 4, 8]), rng.randint(6, 24), 0), (4, rng.randint(6, 12), rng.choice([0, 6, 9]))]
    m = make(groups, max_requests=5)
    live = {}                                      # slot -> length
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            s = m.admit(next_id)
            next_id += 1
            assert s >= 0 and s not in live
            live[s] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.randint(1, 9)
            free_before = [m.free_pages(g) for g in range(2)]
            ok = m.append(s, n)
            assert ok == all(m.pages_needed(s, g, 0) >= 0 for g in range(2)) or True
            if ok:
                live[s] += n
                m.release_out_of_window(s)
            else:
                assert [m.free_pages(g) for g in range(2)] == free_before and m.length(s) == live[s]
        elif live:
            s = rng.choice(list(live))
            m.release(s)
            del live[s]
        assert m.check() == ""
        for s, n in live.items():
            assert m.length(s) == n
            for g, (ps, _, w) in enumerate(groups):
                table = m.block_table(s, g)
                first_needed = max(0, n - w + 1) if w else 0
                for lp, p in enumerate(table):
                    if (lp + 1) * ps > first_needed and lp * ps < n:
                        assert p >= 0              # every page a later query can reach is held
        held = sum(1 for s in live for p in m.block_table(s, 0) if p >= 0)
        assert held + m.free_pages(0) == groups[0][1]
    for s in list(live):
        m.release(s)
    assert all(m.free_pages(g) == groups[g][1] for g in range(2)) and m.check() == ""


def test_pages_given_back_are_noted_for_the_debugging_mode():
    m = make([(4, 8, 0), (4, 8, 6)])
    a, b = m.admit(1), m.admit(2)
    assert m.append(a, 9) and m.append(b, 5)
    assert m.take_freed(0) == [] and m.take_freed(1) == []      # nothing is noted until it is switched on
    m.record_freed(True)
    m.release(b)
    assert sorted(m.take_freed(0)) == [3, 4] and sorted(m.take_freed(1)) == [3, 4]
    assert m.take_freed(0) == []                                 # handed over once
    assert m.append(a, 8)                                        # 17 tokens; the window of 6 lets the first pages go
    assert m.release_out_of_window(a) == 3                       # the next query, at 17, reads keys 12..17
    assert m.take_freed(0) == [] and sorted(m.take_freed(1)) == [0, 1, 2]
    m.release(a)
    assert len(m.take_freed(0)) == 5 and len(m.take_freed(1)) == 2
    assert m.check() == ""
