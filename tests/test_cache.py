"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of requests."""

import random

import pytest
import torch

from akas_b200.cache import CacheManager, OutOfPages, OutOfSlots, PageAllocator
from akas_b200.parts import PagedKVSpec, StateSpec

FULL = PagedKVSpec(2, 16)
WINDOW = PagedKVSpec(1, 32, window=20)
STATE = StateSpec((2, 8))


def _manager(specs=(FULL, STATE, FULL), page=4, tokens=64, requests=3, context=40, storage=False):
    return CacheManager(list(specs), page, tokens, requests, context, storage=storage)


def test_allocator_refuses_double_free_and_foreign_pages():
    a = PageAllocator(3)
    pages = [a.take() for _ in range(3)]
    assert sorted(pages) == [0, 1, 2] and a.free == 0
    with pytest.raises(OutOfPages):
        a.take()
    a.give(1)
    with pytest.raises(RuntimeError):
        a.give(1)
    with pytest.raises(RuntimeError):
        a.give(7)
    assert a.take() == 1


def test_layers_with_the_same_needs_share_a_group():
    m = _manager((FULL, STATE, WINDOW, FULL, None, WINDOW))
    assert len(m.groups) == 2
    assert [getattr(v, "group", None) for v in m.views] == [0, None, 1, 0, None, 1]


def test_pages_follow_tokens_and_come_back():
    m = _manager()
    m.admit("a")
    assert m.pages_needed("a", 9) == [3]
    m.reserve("a", 9)
    m.advance("a", 9)
    assert len(m.blocks("a", 0)) == 3 and m.free_pages() == 13 and m.room("a") == 31  # bounded by the context of 40
    m.reserve("a", 3)  # fits the last page
    assert len(m.blocks("a", 0)) == 3
    m.advance("a", 3)
    with pytest.raises(RuntimeError):
        m.advance("a", 1)  # nothing reserved for it
    with pytest.raises(ValueError):
        m.reserve("a", 100)  # past the context
    m.release("a")
    assert m.free_pages() == 16 and m.free_slots() == 3
    m.check()


def test_out_of_pages_takes_nothing():
    m = _manager((FULL, WINDOW), page=4, tokens=16, requests=3, context=64)
    m.admit("a"), m.admit("b")
    m.reserve("a", 12)
    before = [g.allocator.free for g in m.groups]
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)
    assert [g.allocator.free for g in m.groups] == before and m.blocks("b", 0) == []
    m.check()


def test_slots_run_out_and_are_reused_lowest_first():
    m = _manager()
    assert [m.admit(r) for r in "abc"] == [0, 1, 2]
    with pytest.raises(OutOfSlots):
        m.admit("d")
    with pytest.raises(RuntimeError):
        m.admit("a")
    m.release("b")
    assert m.admit("d") == 1


def test_a_window_gives_back_the_pages_it_has_passed():
    m = _manager((FULL, WINDOW), page=4, tokens=200, requests=2, context=200)
    m.admit("a")
    for _ in range(60):
        m.reserve("a", 1)
        m.advance("a", 1)
        m.check()
    full, win = m.blocks("a", 0), m.blocks("a", 1)
    assert all(p >= 0 for p in full) and len(full) == 15
    # the next query sits at position 60 and sees keys 41..60: blocks 0..9 (positions < 40) are gone
    assert [p >= 0 for p in win] == [False] * 10 + [True] * 5
    assert m.groups[1].allocator.free == 50 - 5
    m.reserve("a", 30)  # a portion: queries at 60..89 still need keys from 41 on
    assert [p >= 0 for p in m.blocks("a", 1)][:10] == [False] * 10 and len(m.blocks("a", 1)) == 23
    m.advance("a", 30)
    assert sum(p >= 0 for p in m.blocks("a", 1)) == 6
    m.release("a")
    assert m.groups[1].allocator.free == 50 and m.groups[0].allocator.free == 50


def test_state_rows_are_zeroed_at_admission():
    m = _manager(storage=True)
    state = m.views[1].state
    state.fill_(3.0)
    slot = m.admit("a")
    assert torch.count_nonzero(state[slot]) == 0 and torch.all(state[slot + 1] == 3.0)
    state[slot].fill_(5.0)
    m.release("a")
    assert m.admit("b") == slot and torch.count_nonzero(state[slot]) == 0
    assert m.views[0].k.shape == (16, 2, 4, 16)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests(seed):
    rng = random.Random(seed)
    m = _manager((FULL, WINDOW, STATE), page=4, tokens=96, requests=4, context=80)
    live, counter = {}, 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and m.free_slots():
            counter += 1
            live[counter] = 0
            m.admit(counter)
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice((1, 1, 1, 2, 5, 11))
            if live[rid] + n > 80:
                continue
            try:
                m.reserve(rid, n)
            except OutOfPages:
                victim = max(live)  # what the scheduler does: the youngest gives everything back
                m.release(victim)
                del live[victim]
                continue
            m.advance(rid, n)
            live[rid] += n
            assert m.length(rid) == live[rid]
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():  # a request holds exactly the pages its tokens need
            assert len(m.blocks(rid, 0)) == -(-n // 4)
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(g.allocator.free == 24 for g in m.groups) and m.free_slots() == 4
