"""The cache manager: no page lost, held twice or freed twice, under random orders of requests (no GPU)."""
import random

import pytest

from atoma_infer_b200.cache import CacheError, CacheGroup, CacheManager, CacheNeed, OutOfPages


def mgr(pages=8, page_size=4, max_seqs=4, window=None, extra_groups=()):
    groups = [CacheGroup(CacheNeed.kv(2, 16, window), [0, 1], pages + 1)] + list(extra_groups)
    return CacheManager(page_size, groups, max_seqs)


def test_pages_are_lifo_and_page_zero_is_never_handed_out():
    m = mgr()
    assert m.add_request(1) == 0
    m.reserve(1, 10)  # 3 pages of 4 tokens
    assert m.table(1) == [8, 7, 6]  # the highest id first, as the reference's allocator (block_allocator.rs:59-67)
    assert m.num_free_pages() == 5
    m.advance(1, 10)
    assert m.num_tokens(1) == 10
    m.reserve(1, 12)
    assert m.table(1) == [8, 7, 6]  # the third page still has room
    m.reserve(1, 13)
    assert m.table(1) == [8, 7, 6, 5]
    assert m.free_request(1) == 4
    assert m.num_free_pages() == 8 and m.audit() == ""
    m.add_request(2)
    m.reserve(2, 16)
    assert 0 not in m.table(2) and m.table(2) == [5, 6, 7, 8]  # used again, in another physical order


def test_errors_are_told_apart():
    m = mgr(pages=4, max_seqs=2)
    m.add_request(1)
    with pytest.raises(CacheError) as e:
        m.add_request(1)
    assert e.value.code == -4
    m.add_request(2)
    with pytest.raises(CacheError) as e:
        m.add_request(3)
    assert e.value.code == -2  # no state slot left
    m.reserve(1, 12)
    assert m.can_reserve(2, 8) == -1   # not now
    assert m.can_reserve(2, 17) == -6  # never: 5 pages of 4 usable
    with pytest.raises(OutOfPages):
        m.reserve(2, 8)
    assert m.table(2) == [] and m.audit() == ""  # all pools or none
    with pytest.raises(CacheError) as e:
        m.advance(2, 3)
    assert e.value.code == -5
    m.free_request(1)
    with pytest.raises(CacheError) as e:
        m.free_request(1)  # freed twice
    assert e.value.code == -3
    assert m.audit() == ""


def test_state_slots_are_claimed_and_given_back():
    m = mgr(max_seqs=3)
    slots = [m.add_request(r) for r in (10, 11, 12)]
    assert sorted(slots) == [0, 1, 2] and m.num_free_slots() == 0
    m.free_request(11)
    assert m.add_request(13) == slots[1]  # the freed slot is used again
    assert m.state_slot(13) == slots[1] and m.audit() == ""


def test_window_group_gives_pages_back_as_the_window_passes():
    m = mgr(pages=6, page_size=4, window=6)
    m.add_request(1)
    held = []
    for step in range(40):  # one token a step, far beyond 6 pages * 4 tokens
        n = m.num_tokens(1)
        m.reserve(1, n + 1)
        m.advance(1, 1)
        t = m.table(1)
        live = [p for p in t if p >= 0]
        held.append(len(live))
        # the next query sits at n+1 and needs keys n+1-5 .. n+1: their pages must be there
        first_needed = max(0, (n + 1) - 6 + 1) // 4
        assert all(p >= 0 for p in t[first_needed:]) and all(p < 0 for p in t[:first_needed])
        assert m.audit() == ""
    assert max(held) <= 3  # window 6 over pages of 4 never needs more than 3 pages
    m.free_request(1)
    assert m.num_free_pages() == 6 and m.audit() == ""


def test_groups_have_pools_of_their_own():
    m = mgr(pages=8, window=None, extra_groups=[CacheGroup(CacheNeed.kv(1, 32, 8), [2], 4)])
    m.add_request(1)
    m.reserve(1, 12)
    assert len(m.table(1, 0)) == 3 and len(m.table(1, 1)) == 3
    assert m.num_free_pages(0) == 5 and m.num_free_pages(1) == 0
    m.add_request(2)
    assert m.can_reserve(2, 4) == -1  # the small pool is empty although the large one has room
    m.advance(1, 12)                  # window 8: the first page of the window group goes back
    assert m.num_free_pages(1) == 1 and m.can_reserve(2, 4) == 0
    assert m.audit() == ""


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_books(seed):
    rng = random.Random(seed)
    window = None if seed % 2 == 0 else 9
    m = mgr(pages=24, page_size=4, max_seqs=5, window=window)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            m.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 13])
            if m.can_reserve(r, live[r] + n) == 0:
                m.reserve(r, live[r] + n)
                m.advance(r, n)
                live[r] += n
                assert m.num_tokens(r) == live[r]
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(r, live[r] + n)
        elif live:
            r = rng.choice(list(live))
            m.free_request(r)
            del live[r]
            with pytest.raises(CacheError):
                m.free_request(r)
        assert m.audit() == "", m.audit()
        held = sum(sum(p >= 0 for p in m.table(r)) for r in live)
        assert held + m.num_free_pages() == 24
        all_pages = [p for r in live for p in m.table(r) if p >= 0]
        assert len(all_pages) == len(set(all_pages)) and 0 not in all_pages
    for r in list(live):
        m.free_request(r)
    assert m.num_free_pages() == 24 and m.num_free_slots() == 5 and m.audit() == ""
