"""The cache manager: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; slots
(pattern of crates/vllm-paged-attention/src/allocator.rs:177-210)."""
import numpy as np
import pytest

from railgun_b200.cache.manager import CacheError, OutOfPages, PageAllocator, PagedKVNeed, StateNeed, group_needs


def test_counts_and_fifo_reuse():
    a = PageAllocator([4], [6], [0], 3)
    assert a.free_pages() == 6 and a.free_slots() == 3
    s = a.add_request(10)
    a.reserve(10, 9)                                   # 3 pages
    assert a.block_table(10).tolist() == [0, 1, 2] and a.free_pages() == 3
    a.reserve(10, 9)                                   # idempotent
    assert a.free_pages() == 3
    a.commit(10, 9)
    assert a.num_computed(10) == 9 and a.slot(10) == s
    a.release(10)
    assert a.free_pages() == 6 and a.free_slots() == 3
    a.add_request(11)
    a.reserve(11, 16)                                  # FIFO: the untouched pages first, then the returned ones
    assert a.block_table(11).tolist() == [3, 4, 5, 0]
    a.check()


def test_errors():
    a = PageAllocator([4], [2], [0], 1)
    a.add_request(1)
    with pytest.raises(CacheError):
        a.add_request(1)                               # duplicate
    with pytest.raises(CacheError):
        a.add_request(2)                               # no slot left
    with pytest.raises(OutOfPages):
        a.reserve(1, 9)
    assert a.free_pages() == 2                         # a failed reserve takes nothing
    with pytest.raises(CacheError):
        a.commit(1, 5)                                 # beyond what is reserved
    with pytest.raises(CacheError):
        a.release(99)
    a.release(1)
    with pytest.raises(CacheError):
        a.release(1)                                   # freed twice
    a.check()


def test_reserve_is_all_groups_or_none():
    a = PageAllocator([4, 4], [8, 2], [0, 0], 2)
    a.add_request(1)
    with pytest.raises(OutOfPages):
        a.reserve(1, 12)                               # group 1 has only 2 pages
    assert a.free_pages(0) == 8 and a.free_pages(1) == 2
    a.check()


def test_window_gives_pages_back():
    a = PageAllocator([4, 4], [32, 32], [0, 6], 2)
    a.add_request(1)
    n = 0
    for step in (3, 5, 1, 1, 7, 2, 1, 1, 1, 9):
        n += step
        a.reserve(1, n)
        a.commit(1, n)
        full, win = a.block_table(1, 0), a.block_table(1, 1)
        assert (full >= 0).all() and len(full) == -(-n // 4)
        first_needed = n - 6 + 1
        for i, p in enumerate(win):
            assert (p < 0) == ((i + 1) * 4 <= first_needed), (n, i, win)
        a.check()
    held = (a.block_table(1, 1) >= 0).sum()
    assert held <= 3 and a.free_pages(1) == 32 - held
    a.release(1)
    assert a.free_pages(1) == 32
    a.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = np.random.default_rng(seed)
    pages, slots = [24, 16], 5
    a = PageAllocator([4, 8], pages, [0, 20], slots)
    live, next_id = {}, 1
    held_at_some_time = set()
    for _ in range(600):
        op = rng.integers(0, 10)
        if op < 2 and len(live) < slots:
            a.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 8 and live:
            rid = int(rng.choice(list(live)))
            new_len = live[rid] + int(rng.integers(1, 12))
            try:
                a.reserve(rid, new_len)
            except OutOfPages:
                victim = int(rng.choice(list(live)))
                a.release(victim)
                del live[victim]
                continue
            a.commit(rid, new_len)
            live[rid] = new_len
        elif live:
            rid = int(rng.choice(list(live)))
            a.release(rid)
            del live[rid]
        a.check()
        # no page is held by two requests
        for g in range(2):
            seen = []
            for rid in live:
                seen += [int(p) for p in a.block_table(rid, g) if p >= 0]
            assert len(seen) == len(set(seen))
            assert len(seen) + a.free_pages(g) == pages[g]
            held_at_some_time |= {(g, p) for p in seen}
        assert a.free_slots() == slots - len(live)
    for rid in list(live):
        a.release(rid)
    a.check()
    assert [a.free_pages(g) for g in range(2)] == pages and a.free_slots() == slots
    assert len(held_at_some_time) > sum(pages) * 0.8          # pages were used again and again


def test_needs_are_sorted_into_groups():
    full = PagedKVNeed(2, 16, 0)
    groups, group_of, states = group_needs({
        0: full, 1: PagedKVNeed(2, 16, 8), 2: full, 3: StateNeed((4, 4)), 4: None, 5: PagedKVNeed(1, 16, 0)})
    assert [(n, c) for n, c in groups] == [(full, [0, 2]), (PagedKVNeed(2, 16, 8), [1]), (PagedKVNeed(1, 16, 0), [5])]
    assert group_of == {0: 0, 2: 0, 1: 1, 5: 2} and list(states) == [3]


def test_groups_get_the_page_geometry_they_ask_for():
    """Needs that say nothing get the engine's page size, pool and precision; a need may ask for its own page
    size, a smaller pool (a windowed group), another precision and another shape of page."""
    import torch
    from railgun_b200.cache.manager import CacheManager, PagedKVNeed, StateNeed
    needs = {0: PagedKVNeed(2, 16), 1: PagedKVNeed(2, 16),                       # one group, two cache ids
             2: PagedKVNeed(1, 32, window=24, page_size=8, pool_tokens=96),      # windowed: small pages, small pool
             3: PagedKVNeed(0, 0, dtype="float32", page_shape=("page", 40)),     # one compressed vector per token
             4: StateNeed((5, 3), "float32"), 5: None}
    cm = CacheManager(needs, page_size=16, max_tokens=256, max_requests=4, dtype=torch.bfloat16, device="cpu")
    assert [(g.page_size, g.num_pages, g.cache_ids) for g in cm.groups] == [(16, 16, [0, 1]), (8, 12, [2]), (16, 16, [3])]
    assert cm.kv[0].shape == (16, 2, 2, 16, 16) and cm.kv[0].dtype == torch.bfloat16
    assert cm.kv[2].shape == (12, 2, 1, 8, 32) and cm.page_size_of(2) == 8
    assert cm.kv[3].shape == (16, 16, 40) and cm.kv[3].dtype == torch.float32
    assert cm.state[4].shape == (4, 5, 3) and 5 not in cm.kv and 5 not in cm.state
    assert cm.bytes_per_token() == 2 * (2 * 2 * 16 * 2) + 2 * 1 * 32 * 2 + 40 * 4
    # the allocator has the groups' own page sizes and pools: 20 tokens take 2, 3 and 2 pages
    cm.alloc.add_request(1)
    cm.alloc.reserve(1, 20)
    assert [len(cm.alloc.block_table(1, g)) for g in range(3)] == [2, 3, 2]
    assert [cm.alloc.free_pages(g) for g in range(3)] == [14, 9, 14]
    cm.alloc.check()
