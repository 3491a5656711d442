"""The cache manager's host bookkeeping: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; groups have pools of their own; slots."""
import random

import pytest
from hypothesis import given, settings, strategies as st

import kirai_b200
from kirai_b200.cache import NO_PAGE, CacheError, CacheManager, PagePool, SlotPool
from kirai_b200.parts.base import KVCacheNeed, StateNeed


def manager(page_size=4, num_pages=16, num_slots=4, window=8):
    needs = [KVCacheNeed(2, 16, None), KVCacheNeed(2, 16, window), KVCacheNeed(2, 16, window), StateNeed((3,))]
    return CacheManager(needs, page_size=page_size, num_pages=num_pages, num_slots=num_slots, device=None)


def test_pool_allocates_all_or_nothing_and_refuses_double_free():
    pool = PagePool(4)
    first = pool.allocate(3)
    assert pool.allocate(2) is None and pool.free_pages == 1
    pool.release(first[:1])
    with pytest.raises(CacheError):
        pool.release(first[:1])
    with pytest.raises(CacheError):
        pool.release([99])
    again = pool.allocate(2)
    assert first[0] in again  # a freed page is used again, last freed first
    assert pool.high_water == 4


def test_slots():
    slots = SlotPool(2)
    a, b = slots.allocate(), slots.allocate()
    assert slots.allocate() is None and {a, b} == {0, 1}
    slots.release(a)
    with pytest.raises(CacheError):
        slots.release(a)
    assert slots.allocate() == a


def test_groups_are_formed_by_need():
    cache = manager()
    assert len(cache.groups) == 2 and cache.groups[0].layers == [0] and cache.groups[1].layers == [1, 2]
    assert cache.layer_view(2).group == 1 and cache.layer_view(2).window == 8
    assert cache.bytes_per_token() == 3 * 2 * 2 * 16 * 4


def test_reserve_commit_close_and_block_table():
    cache = manager()
    request = cache.open("r")
    assert cache.reserve(request, 9)  # 3 pages in both groups
    assert [len(t) for t in request.tables] == [3, 3]
    cache.commit(request, 9)
    assert cache.reserve(request, 3) and [len(t) for t in request.tables] == [3, 3]  # still fits: 12 tokens
    cache.commit(request, 3)
    # window 8 at length 12: positions below 5 are dead, so page 0 (positions 0-3) went back in group 1 only
    assert request.tables[0][0] != NO_PAGE and request.tables[1][0] == NO_PAGE and request.tables[1][1] != NO_PAGE
    table = cache.block_table_array([request], 1)
    assert table.shape == (1, 3) and table[0, 0] == NO_PAGE
    cache.tables.check_consistency()
    with pytest.raises(CacheError):
        cache.commit(request, 1)  # no page reserved for a 13th token
    cache.close(request)
    assert cache.free_pages() == [16, 16] and cache.tables.slots.free_slots == 4
    with pytest.raises(CacheError):
        cache.close(request)


def test_window_release_boundaries():
    cache = manager(page_size=4, window=8)
    request = cache.open("w")
    for length in range(1, 40):
        assert cache.reserve(request, 1)
        cache.commit(request, 1)
        first_visible = length - 8 + 1  # the next token (position `length`) reads from here on
        for page, entry in enumerate(request.tables[1]):
            dead = (page + 1) * 4 <= first_visible
            assert (entry == NO_PAGE) == dead, (length, page)
        assert all(entry != NO_PAGE for entry in request.tables[0])
    assert cache.tables.pools[1].used_pages <= 3  # 8 tokens of window span at most 3 pages of 4


def test_out_of_pages_takes_nothing():
    cache = manager(num_pages=4)
    a, b = cache.open("a"), cache.open("b")
    assert cache.reserve(a, 12)
    before = cache.free_pages()
    assert not cache.can_reserve(b, 8) and not cache.reserve(b, 8)
    assert cache.free_pages() == before and b.tables == [[], []]
    assert cache.reserve(b, 4)


def test_no_slot_means_no_admission():
    cache = manager(num_slots=1)
    assert cache.open("a") is not None and cache.open("b") is None
    with pytest.raises(CacheError):
        cache.open("a")


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2**32 - 1), st.sampled_from([1, 4, 8]), st.integers(6, 40), st.sampled_from([None, 5, 16]))
def test_random_orders_keep_every_page_accounted(seed, page_size, num_pages, window):
    rng = random.Random(seed)
    needs = [KVCacheNeed(1, 8, None), KVCacheNeed(1, 8, window)] if window else [KVCacheNeed(1, 8, None)]
    cache = CacheManager(needs, page_size=page_size, num_pages=num_pages, num_slots=3, device=None)
    live, counter = {}, 0
    for _ in range(200):
        action = rng.random()
        if action < 0.25 and len(live) < 3:
            request = cache.open(counter)
            assert request is not None
            live[counter] = request
            counter += 1
        elif action < 0.85 and live:
            request = live[rng.choice(list(live))]
            count = rng.choice([1, 1, 1, 2, 3, 7, 19])
            free_before = cache.free_pages()
            if cache.reserve(request, count):
                cache.commit(request, count)
            else:
                assert cache.free_pages() == free_before
        elif live:
            key = rng.choice(list(live))
            cache.close(live.pop(key))
        cache.tables.check_consistency()
        for pool in cache.tables.pools:
            assert pool.free_pages + pool.used_pages == pool.num_pages
    for request in live.values():
        cache.close(request)
    assert cache.free_pages() == [num_pages] * len(cache.groups)
    assert cache.tables.slots.free_slots == 3


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2**32 - 1), st.sampled_from([1, 4, 16]), st.integers(4, 40), st.sampled_from([None, 3, 20]))
def test_native_tables_follow_the_python_model(seed, page_size, num_pages, window):
    """The native page tables and the Python model, driven by the same random requests, hold the same
    pages in the same places at every step."""
    rng = random.Random(seed)
    needs = [KVCacheNeed(1, 8, None), KVCacheNeed(1, 8, window)] if window else [KVCacheNeed(1, 8, None)]
    native = CacheManager(needs, page_size=page_size, num_pages=num_pages, num_slots=3, device=None, native=True)
    model = CacheManager(needs, page_size=page_size, num_pages=num_pages, num_slots=3, device=None, native=False)
    assert type(native.tables).__name__ == "NativePageTables" and type(model.tables).__name__ == "PageTables"
    live, counter = {}, 0
    for _ in range(150):
        action = rng.random()
        if action < 0.25:
            a, b = native.open(counter), model.open(counter)
            assert (a is None) == (b is None)
            if a is not None:
                assert a.slot == b.slot
                live[counter] = (a, b)
            counter += 1
        elif action < 0.85 and live:
            a, b = live[rng.choice(list(live))]
            count = rng.choice([1, 1, 2, 5, 17])
            assert native.tables.pages_needed(a, count) == model.tables.pages_needed(b, count)
            assert native.can_reserve(a, count) == model.can_reserve(b, count)
            took_a, took_b = native.reserve(a, count), model.reserve(b, count)
            assert took_a == took_b
            if took_a:
                native.commit(a, count)
                model.commit(b, count)
        elif live:
            key = rng.choice(list(live))
            a, b = live.pop(key)
            native.close(a)
            model.close(b)
        for a, b in live.values():
            assert a.length == b.length and a.tables == b.tables
        for group in range(len(needs)):
            requests = list(live.values())
            if requests:
                assert (native.block_table_array([a for a, _ in requests], group) ==
                        model.block_table_array([b for _, b in requests], group)).all()
        assert native.free_pages() == model.free_pages()
        native.tables.check_consistency()
        model.tables.check_consistency()
    assert native.stats() == model.stats()


def test_native_tables_refuse_misuse():
    cache = manager()
    request = cache.open("x")
    cache.reserve(request, 5)
    with pytest.raises(CacheError):
        cache.commit(request, 9)
    cache.close(request)
    for call in (lambda: cache.reserve(request, 1), lambda: cache.commit(request, 1), lambda: cache.close(request)):
        with pytest.raises(CacheError):
            call()
    assert request.closed and request.tables == [[], []]


def test_page_sizes_the_kernels_would_refuse_are_refused_when_the_cache_is_made():
    """The bfloat16 attention kernels read pages by TMA boxes that tile their key tiles; a page size they cannot
    take is refused by the cache manager, with the reason, not by a kernel at the first step.  The 32-bit path and
    head sizes that go to the CUDA-core kernel take any page size."""
    import torch

    from kirai_b200.csrc.ops import page_size_refusal

    need = [KVCacheNeed(2, 128, None)]
    for page_size in (1, 2, 4, 8, 16, 32, 64, 128, 192):
        assert page_size_refusal(torch.bfloat16, 128, page_size) is None
        CacheManager(need, page_size=page_size, num_pages=4, num_slots=1, dtype=torch.bfloat16, device=None)
    for page_size in (3, 12, 24, 48, 96, 100):
        assert "pages of" in page_size_refusal(torch.bfloat16, 128, page_size)
        with pytest.raises(CacheError, match="attention kernels"):
            CacheManager(need, page_size=page_size, num_pages=4, num_slots=1, dtype=torch.bfloat16, device=None)
        CacheManager(need, page_size=page_size, num_pages=4, num_slots=1, dtype=torch.float32, device=None)
        CacheManager([KVCacheNeed(2, 20, None)], page_size=page_size, num_pages=4, num_slots=1, dtype=torch.bfloat16, device=None)
    with pytest.raises(CacheError):
        CacheManager(need, page_size=0, num_pages=4, num_slots=1, dtype=torch.float32, device=None)
