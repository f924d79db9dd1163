"""The cache manager's host side: no page lost, held twice or freed twice, under random
orders of requests; groups with windows give pages back; state slots (no GPU)."""
import random

import pytest

from sandyrt_b200.cache.pages import (FREED, BlockAllocator, CacheError, CacheLayout, NoFreeSlot,
                                      OutOfPages, PagePool)
from sandyrt_b200.parts.base import PagedKVSpec, StateSpec


def test_pool_hands_out_runs():
    """A fresh pool hands out 0, 1, 2, ...; afterwards always the lowest free pages, in order."""
    pool = PagePool(16)
    a = pool.allocate(6)
    b = pool.allocate(4)
    assert a == [0, 1, 2, 3, 4, 5] and b == [6, 7, 8, 9]
    pool.release(a)
    assert pool.allocate(4) == [0, 1, 2, 3]
    pool.release(b)
    assert pool.allocate(6) == [4, 5, 6, 7, 8, 9]


def _alloc(specs, pages, page_size=16, max_requests=4):
    layout = CacheLayout.from_specs(specs, page_size)
    return BlockAllocator(layout, [pages] * len(layout.groups), max_requests)


def test_pool_reuses_last_freed_first_and_detects_double_free():
    pool = PagePool(4)
    a = pool.allocate(3)
    assert sorted(a) == [0, 1, 2] and pool.free_pages == 1
    pool.release([a[1]])
    assert pool.allocate(1) == [a[1]]              # the page just freed comes back (it is the lowest free one)
    with pytest.raises(OutOfPages):
        pool.allocate(2)
    assert pool.free_pages == 1                    # a failed allocation takes nothing
    pool.release([a[0]])
    with pytest.raises(CacheError, match="freed twice"):
        pool.release([a[0]])
    with pytest.raises(CacheError, match="does not belong"):
        pool.release([17])
    assert pool.high_water == 3


def test_page_size_must_be_a_power_of_two():
    with pytest.raises(CacheError, match="power of two"):
        CacheLayout.from_specs([PagedKVSpec(2, 16)], 24)


def test_layers_with_equal_needs_share_a_group():
    full, local = PagedKVSpec(2, 16), PagedKVSpec(2, 16, window=32)
    layout = CacheLayout.from_specs([full, local, local, full, None, StateSpec((3, 5))], 16)
    assert [g.caches for g in layout.groups] == [[0, 3], [1, 2]]
    assert layout.group_of_cache[3] == (0, 1) and layout.group_of_cache[2] == (1, 1)
    assert list(layout.state_of_cache) == [5]


def test_reserve_commit_release():
    al = _alloc([PagedKVSpec(2, 16)] * 3, pages=6)
    al.admit("a")
    assert al.pages_needed("a", 33) == [3]
    al.reserve("a", 33)
    assert len(al.block_list("a", 0)) == 3 and al.free_pages() == 3
    al.reserve("a", 40)                                  # still inside the third page
    assert al.free_pages() == 3
    al.commit("a", 33)
    with pytest.raises(CacheError, match="not reserved"):
        al.commit("a", 49)
    with pytest.raises(CacheError, match="shrink"):
        al.commit("a", 10)
    al.admit("b")
    with pytest.raises(OutOfPages):
        al.reserve("b", 16 * 4)
    assert al.free_pages() == 3 and al.block_list("b", 0) == []   # all or nothing
    al.release("a")
    al.reserve("b", 16 * 4)
    al.check()
    with pytest.raises(CacheError, match="not live"):
        al.release("a")


def test_slots_run_out_and_come_back():
    al = _alloc([PagedKVSpec(1, 16)], pages=8, max_requests=2)
    s0, s1 = al.admit("a"), al.admit("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(NoFreeSlot):
        al.admit("c")
    with pytest.raises(CacheError, match="already live"):
        al.admit("a")
    al.release("a")
    assert al.admit("c") == s0
    al.check()


def test_window_group_gives_pages_back_as_the_window_passes():
    full, local = PagedKVSpec(2, 16), PagedKVSpec(2, 16, window=20)
    al = _alloc([full, local], pages=10)
    al.admit("a")
    held_local = []
    for new_len in range(1, 150):
        al.reserve("a", new_len)
        al.commit("a", new_len)
        al.check()
        bl = al.block_list("a", 1)
        # the next query sits at position new_len and reads keys >= new_len - 19
        first_needed = max(0, new_len - 19) // 16
        assert all(p == FREED for p in bl[:first_needed])
        assert all(p != FREED for p in bl[first_needed:])
        held_local.append(sum(p != FREED for p in bl))
    assert max(held_local) <= 3                          # window 20 over pages of 16: at most 3 pages
    assert len([p for p in al.block_list("a", 0) if p != FREED]) == 10   # the full group keeps all
    al.release("a")
    assert al.free_pages(0) == 10 and al.free_pages(1) == 10


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests_never_lose_a_page(seed):
    rng = random.Random(seed)
    specs = [PagedKVSpec(2, 16), PagedKVSpec(2, 16, window=rng.choice([8, 24, 40])), PagedKVSpec(2, 16)]
    al = _alloc(specs, pages=rng.choice([6, 9, 16]), page_size=rng.choice([4, 8, 16]), max_requests=4)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and al.free_slots():
            al.admit(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            new_len = live[rid] + rng.choice([1, 1, 1, 2, 5, 17, 40])
            if al.can_reserve(rid, new_len):
                al.reserve(rid, new_len)
                if rng.random() < 0.9:                   # sometimes a reservation is not used at once
                    al.commit(rid, new_len); live[rid] = new_len
            else:
                before = [al.free_pages(g) for g in range(len(al.pools))]
                with pytest.raises(OutOfPages):
                    al.reserve(rid, new_len)
                assert before == [al.free_pages(g) for g in range(len(al.pools))]
        elif live:
            rid = rng.choice(list(live))
            al.release(rid); del live[rid]
        al.check()
    for rid in list(live):
        al.release(rid)
    al.check()
    assert all(p.free_pages == p.num_pages for p in al.pools)
    assert al.free_slots() == 4


def test_decode_splits_avoid_clusters_of_six_and_seven():
    """The splits of a (token, head) pair are one thread-block cluster; sizes 6 and 7 are never asked for."""
    from sandyrt_b200.csrc.ops import decode_splits

    seen = set()
    for tokens in range(1, 80):
        for heads in (1, 2, 12, 16, 25):
            for max_kv in (64, 128, 512, 1024, 8192):
                n = decode_splits(tokens, heads, max_kv, sms=148)
                assert n >= 1 and n not in (6, 7)
                assert n <= max(1, max_kv // 64) or n == 5
                seen.add(n)
    assert {1, 2, 3, 4, 5, 8} <= seen


def test_decode_splits_at_the_measured_points():
    """The rule's answers where whole decode steps were measured (12 heads of 64, 148 SMs): about four blocks
    an SM, to the nearest; more for long ranges, up to eight blocks an SM."""
    from sandyrt_b200.csrc.ops import decode_splits

    at = lambda tokens, ctx, heads=12: decode_splits(tokens, heads, ctx, sms=148)
    assert [at(b, 400) for b in (8, 12, 16, 24, 32, 48, 64)] == [5, 4, 3, 2, 2, 2, 1]
    assert at(32, 965) == 3 and at(8, 965) == 5
    assert at(32, 1024, heads=16) == 2          # GPT-2 medium's mixed workload
    assert at(64, 600, heads=25) == 1           # GPT-2 xl, 64 requests: one block a pair


def test_small_product_rule():
    """Which kernel takes a product of up to 64 rows is a rule of its shape (the kernels add in different
    orders, so it must not depend on a timing)."""
    from sandyrt_b200.csrc.ops import small_gemm_kernel

    # GPT-2 small's four products and the vocabulary
    assert [small_gemm_kernel(8, n, k) for n, k in ((2304, 768), (768, 768), (3072, 768), (768, 3072), (50257, 768))] == ["streaming"] * 5
    assert [small_gemm_kernel(64, n, k) for n, k in ((2304, 768), (768, 768), (3072, 768))] == ["streaming"] * 3
    assert small_gemm_kernel(17, 768, 3072) == "split_k" and small_gemm_kernel(64, 50257, 768) == "split_k"
    # wide models: a long K below 17 rows, any K from 1,280 above 32 rows
    assert small_gemm_kernel(8, 1600, 6400) == "split_k" and small_gemm_kernel(8, 1024, 4096) == "streaming"
    assert small_gemm_kernel(64, 4800, 1600) == "split_k" and small_gemm_kernel(32, 4800, 1600) == "streaming"
    assert small_gemm_kernel(64, 3072, 1024) == "streaming"
