"""The cache manager on the host: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; state slots."""
import random

import pytest

from gollmgo_b200.cache import (CacheManager, FixedStateNeed, OutOfPages, OutOfStateSlots,
                                PagedKVNeed, PagePool, StateSlots)


def test_pool_allocates_all_or_nothing_and_reuses_last_freed():
    p = PagePool(4)
    a = p.allocate(3)
    assert a == [0, 1, 2] and p.num_free == 1
    with pytest.raises(OutOfPages):
        p.allocate(2)
    assert p.num_free == 1                       # nothing was taken
    p.release(1)
    assert p.allocate(1) == [1]                  # last freed, first reused
    with pytest.raises(RuntimeError):
        p.release(3)                             # never allocated
    p.release(0)
    with pytest.raises(RuntimeError):
        p.release(0)                             # freed twice
    assert p.high_water == 3


def test_pool_reference_counts():
    p = PagePool(2)
    (a,) = p.allocate(1)
    p.ref(a)
    p.release(a)
    assert p.num_free == 1 and p.refcount(a) == 1
    p.release(a)
    assert p.num_free == 2
    with pytest.raises(RuntimeError):
        p.ref(a)


def test_state_slots():
    s = StateSlots(2)
    a, b = s.take(), s.take()
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfStateSlots):
        s.take()
    s.give_back(a)
    with pytest.raises(RuntimeError):
        s.give_back(a)
    assert s.take() == a


def make(num_pages=12, page=4, window=None, max_requests=6):
    needs = [PagedKVNeed(2, 8, None), PagedKVNeed(2, 8, None), PagedKVNeed(2, 8, window)] if window \
        else [PagedKVNeed(2, 8, None)] * 3
    return CacheManager(needs, page, num_pages, max_requests)


def test_layers_with_equal_needs_share_a_group():
    cm = make(window=6)
    assert len(cm.groups) == 2
    assert cm.group_of == {0: (0, 0), 1: (0, 1), 2: (1, 0)}
    assert len(make().groups) == 1
    with pytest.raises(TypeError):
        CacheManager(["keys"], 4, 4, 2)
    both = CacheManager([PagedKVNeed(1, 8), FixedStateNeed((5,))], 4, 4, 2)
    assert len(both.groups) == 1 and 1 in both.state_needs


def test_slots_follow_the_block_table():
    cm = make(page=4)
    cm.admit("a")
    a1 = cm.append("a", 6)
    assert a1.start == 0 and list(a1.slots[0]) == [0, 1, 2, 3, 4, 5]
    cm.admit("b")
    assert list(cm.append("b", 1).slots[0]) == [8]
    a2 = cm.append("a", 3)                       # fills page 1, opens page 3
    assert a2.start == 6 and list(a2.slots[0]) == [6, 7, 12]
    assert cm.block_table("a", 0) == [0, 1, 3] and cm.num_tokens("a") == 9
    cm.audit()


def test_out_of_pages_takes_nothing_and_free_returns_everything():
    cm = make(num_pages=3, page=4)
    cm.admit("a")
    cm.append("a", 9)
    cm.admit("b")
    assert cm.pages_short("b", 5) == 2
    with pytest.raises(OutOfPages):
        cm.append("b", 5)
    assert cm.num_tokens("b") == 0 and cm.free_pages() == 0
    cm.audit()
    cm.free("a")
    assert cm.free_pages() == 3
    cm.append("b", 5)
    cm.free("b")
    cm.audit()
    with pytest.raises(KeyError):
        cm.free("b")
    cm.admit("c")
    with pytest.raises(RuntimeError):
        cm.admit("c")                            # admitted twice


def test_window_gives_pages_back_as_it_passes():
    cm = CacheManager([PagedKVNeed(2, 8, 6)], 4, 4, 2)      # window 6, 4 pages of 4 tokens
    cm.admit("a")
    seen = set()
    for step in range(60):                       # 60 tokens through 4 pages: pages come round again
        slots = cm.append("a", 1).slots[0]
        seen.add(slots[0] // 4)
        cm.audit()
        table = cm.block_table("a", 0)
        n = cm.num_tokens("a")
        for idx, page in enumerate(table):
            if idx * 4 + 3 >= n - 6:             # still (partly) inside the window of the last token
                assert page >= 0, f"page {idx} inside the window was given back at {n} tokens"
    assert len(table) == 15 and sum(p >= 0 for p in table) <= 4
    assert seen <= {0, 1, 2, 3} and len(seen) < len(table)      # the same few pages, again and again
    cm.free("a")
    assert cm.free_pages() == 4
    cm.audit()


def test_window_with_portions():
    cm = CacheManager([PagedKVNeed(1, 8, None), PagedKVNeed(1, 8, 5)], 4, 8, 2)
    cm.admit("a")
    cm.append("a", 13)                           # a portion longer than the window keeps all its pages
    assert all(p >= 0 for p in cm.block_table("a", 1))
    cm.append("a", 2)                            # now tokens < 13 - 5 + 1 = 9 are behind: pages 0, 1
    assert cm.block_table("a", 1)[:2] == [-1, -1] and cm.block_table("a", 1)[2] >= 0
    assert all(p >= 0 for p in cm.block_table("a", 0))
    cm.audit()


def test_rollback_returns_the_pages_of_the_abandoned_tokens():
    cm = make(num_pages=6, page=4)
    cm.admit("a")
    cm.append("a", 5)
    before = cm.free_pages()
    cm.append("a", 9)
    cm.rollback("a", 5)
    assert cm.num_tokens("a") == 5 and cm.free_pages() == before
    cm.audit()


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 7])
def test_random_orders_keep_every_page_accounted_for(seed, window):
    rng = random.Random(seed)
    cm = make(num_pages=24, page=4, window=window, max_requests=5)
    live, next_id = {}, 0
    for _ in range(600):
        r = rng.random()
        if (r < 0.25 and len(live) < 5) or not live:
            rid = f"r{next_id}"
            next_id += 1
            cm.admit(rid)
            live[rid] = 0
        elif r < 0.85:
            rid = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 3, 5, 9, 17])
            short = cm.pages_short(rid, n)
            if short:
                with pytest.raises(OutOfPages):
                    cm.append(rid, n)
                victim = max(live, key=lambda k: live[k])      # make room the way a scheduler would
                cm.free(victim)
                del live[victim]
            else:
                got = cm.append(rid, n)
                assert got.start == live[rid]
                for g, slots in enumerate(got.slots):
                    table = cm.block_table(rid, g)
                    for i, s in enumerate(slots):
                        t = got.start + i
                        assert s == table[t // 4] * 4 + t % 4
                live[rid] += n
        else:
            rid = rng.choice(sorted(live))
            cm.free(rid)
            del live[rid]
        cm.audit()
    for rid in list(live):
        cm.free(rid)
    cm.audit()
    assert all(g.pool.num_free == 24 for g in cm.groups) and cm.slots.num_free == 5
