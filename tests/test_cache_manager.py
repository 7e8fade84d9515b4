"""The cache manager: no page lost, held twice or freed twice, under random orders of requests."""

import random

import pytest

from llmserve_b200.cache import RELEASED, CacheManager, KVGroupSpec, OutOfPages, PageAllocator


def groups(window=0, page=4):
    g = [KVGroupSpec((0, 1), 2, 16, 0, page)]
    if window:
        g.append(KVGroupSpec((2,), 1, 16, window, page))
    return g


def test_allocator_fifo_and_double_free():
    a = PageAllocator(3)
    p = [a.allocate() for _ in range(3)]
    assert p == [0, 1, 2] and a.num_free == 0
    with pytest.raises(OutOfPages):
        a.allocate()
    a.release(1)
    a.release(0)
    with pytest.raises(AssertionError):
        a.release(1)
    assert [a.allocate(), a.allocate()] == [1, 0]  # first freed, first reused
    a.check_invariants()


def test_tables_grow_by_pages_and_return_on_release():
    m = CacheManager(groups(), [6], max_requests=2)
    m.admit("a")
    assert m.pages_needed("a", 5) == [2] and m.can_allocate("a", 5)
    m.allocate("a", 5)
    m.commit("a", 5)
    assert m.block_table("a") == [0, 1] and m.num_computed("a") == 5
    m.allocate("a", 3)  # 8 tokens still fit two pages
    assert m.block_table("a") == [0, 1]
    m.commit("a", 3)
    m.allocate("a", 1)
    assert m.block_table("a") == [0, 1, 2]
    m.admit("b")
    assert not m.can_allocate("b", 13) and m.can_allocate("b", 12)
    with pytest.raises(OutOfPages):
        m.allocate("b", 13)
    assert m.block_table("b") == []  # a failed allocation takes nothing
    with pytest.raises(OutOfPages):
        m.admit("c")  # no state slot left
    m.release("a")
    assert m.num_free_pages() == 6 and m.has_free_slot()
    m.allocate("b", 13)
    assert m.block_table("b") == [3, 4, 5, 2]  # freed pages go to the tail, in reverse table order
    m.check_invariants()
    with pytest.raises(KeyError):
        m.release("a")


def test_try_allocate_takes_all_or_nothing():
    m = CacheManager(groups(window=6), [6, 3], max_requests=2)
    m.admit("a")
    assert m.try_allocate("a", 8) and m.block_table("a") == [0, 1] and m.block_table("a", 1) == [0, 1]
    assert m.table_array("a").tolist() == [0, 1]
    assert m.try_allocate("a", 8)  # nothing new is needed
    assert not m.try_allocate("a", 13)  # the second group has no fourth page: the first keeps its own
    assert m.block_table("a") == [0, 1] and m.num_free_pages(0) == 4
    m.commit("a", 8)
    assert m.try_allocate("a", 1)
    m.commit("a", 1)  # the next query reads keys 4 and later: the window group gives page 0 back
    assert m.block_table("a", 1) == [RELEASED, 1, 2] and m.table_array("a", 1).tolist() == [RELEASED, 1, 2]
    assert m.try_allocate("a", 4) and m.block_table("a", 1) == [RELEASED, 1, 2, 0]
    m.check_invariants()
    big = CacheManager(groups(), [100], max_requests=1)  # a table far longer than the array's first room
    big.admit("x")
    assert big.try_allocate("x", 4 * 70)
    assert big.table_array("x").tolist() == big.block_table("x") == list(range(70))
    big.check_invariants()


def test_window_group_gives_pages_back_while_the_request_lives():
    m = CacheManager(groups(window=6), [20, 4], max_requests=1)
    m.admit("a")
    held_max = 0
    for step in range(40):
        n = 1 + step % 3
        assert m.can_allocate("a", n)
        m.allocate("a", n)
        # every key a query of this step may read still has its page
        c = m.num_computed("a")
        t = m.block_table("a", 1)
        for j in range(max(0, c - 6 + 1), c + n):
            assert t[j // 4] != RELEASED
        m.commit("a", n)
        held_max = max(held_max, sum(p != RELEASED for p in m.block_table("a", 1)))
        m.check_invariants()
    assert held_max <= 4 and m.num_computed("a") > 60
    assert sum(p != RELEASED for p in m.block_table("a", 0)) == -(-m.num_computed("a") // 4)
    m.release("a")
    assert m.usage() == 0.0


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    m = CacheManager(groups(window=9, page=rng.choice([1, 4, 16])), [40, 12], max_requests=5)
    live, next_id = {}, 0
    for _ in range(400):
        r = rng.random()
        if r < 0.25 and m.has_free_slot():
            rid = f"r{next_id}"
            next_id += 1
            m.admit(rid)
            live[rid] = 0
        elif r < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 30])
            if m.can_allocate(rid, n):
                m.allocate(rid, n)
                if rng.random() < 0.9:  # sometimes allocated but the step never commits
                    m.commit(rid, n)
                    live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.allocate(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            assert m.num_computed(rid) == n
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert m.usage() == 0.0 and len(m.free_slots) == 5


def test_layers_are_grouped_by_what_they_keep():
    import torch

    from llmserve_b200.cache import group_cache_layers, pages_for_memory
    from llmserve_b200.parts import PagedKVNeed, StateNeed

    needs = {0: PagedKVNeed(2, 64, 0), 1: PagedKVNeed(2, 64, 128), 2: PagedKVNeed(2, 64, 0), 3: None,
             4: StateNeed((4, 8), torch.float32), 5: PagedKVNeed(2, 64, 128)}
    kv, st = group_cache_layers(needs, 16)
    assert [g.cache_ids for g in kv] == [(0, 2), (1, 5)] and [g.window for g in kv] == [0, 128]
    assert [g.cache_ids for g in st] == [(4,)]
    pages = pages_for_memory(kv, 64 << 20, 2, 4096, 512)
    assert pages[0] > pages[1] > 0  # the windowed group needs far fewer pages per request


def test_a_part_may_ask_for_pages_of_another_dtype():
    """Two mixers with the same heads but different page dtypes get groups (and pools) of their
    own, and the memory split counts each group's own element size."""
    import torch

    from llmserve_b200.cache import CachePools, group_cache_layers, pages_for_memory
    from llmserve_b200.parts.base import PagedKVNeed

    needs = {0: PagedKVNeed(2, 16), 1: PagedKVNeed(2, 16, dtype=torch.float32), 2: PagedKVNeed(2, 16)}
    kv, st = group_cache_layers(needs, 8)
    assert [g.cache_ids for g in kv] == [(0, 2), (1,)] and not st
    assert kv[0].bytes_per_token(2) == 2 * 2 * 2 * 16 * 2 and kv[1].bytes_per_token(2) == 2 * 1 * 2 * 16 * 4
    pages = pages_for_memory(kv, 1 << 20, 2, 256, 64)
    assert pages[0] == pages[1]  # the same bytes per token and the same live tokens: the same number of pages
    pools = CachePools(kv, st, pages, 4, torch.bfloat16, "cpu")
    assert pools.view(0, True).k.dtype == torch.bfloat16 and pools.view(1, True).k.dtype == torch.float32
    assert pools.view(1, True).group == 1 and pools.view(2, False).group == 0
