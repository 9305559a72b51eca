"""The cache manager on the host (no GPU): no page is lost, held twice or freed
twice, under random orders of requests; windows give pages back; state slots."""
import random

import pytest
import torch

from llm_serving_engine_b200.cache import CacheFullError, CacheManager, PagePool
from llm_serving_engine_b200.config import CacheConfig
from llm_serving_engine_b200.parts import PagedKV, RequestState


def make(requirements, pages=12, page=4, max_pos=64, slots=4):
    return CacheManager(requirements, CacheConfig(block_size=page, num_blocks=pages), torch.float32, "cpu",
                        max_pos, num_state_slots=slots)


def check_invariants(cache: CacheManager, grown: dict | None = None) -> None:
    """``grown``: per request, tokens whose pages were taken early (``grow``) and not yet reserved."""
    grown = grown or {}
    for index, group in enumerate(cache.groups):
        held = [page for request in cache.requests.values() for page in request.tables[index] if page >= 0]
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) == group.pool.used_pages, "owner map and block tables disagree"
        assert group.pool.used_pages + group.pool.free_pages == group.pool.num_pages, "a page was lost"
        free = list(group.pool._free)
        assert len(free) == len(set(free)) and not set(free) & set(held), "a free page is also held"
        for request in cache.requests.values():
            for page in request.tables[index]:
                if page >= 0:
                    assert group.pool.owner_of(page) == request.request_id
            assert cache.block_table_array(index, request.request_id).tolist() == request.tables[index]
            live = [p for p in request.tables[index] if p >= 0]
            needed = -(-(request.length + grown.get(request.request_id, 0)) // cache.page_size) - request.released[index]
            assert len(live) == needed
    slots = [request.state_slot for request in cache.requests.values()]
    assert len(slots) == len(set(slots)) and len(slots) + len(cache._free_slots) == cache.num_state_slots


def test_pool_reuses_pages_in_fifo_order_and_checks_owners():
    pool = PagePool(3)
    a, b = pool.allocate("x"), pool.allocate("y")
    assert (a, b) == (0, 1)
    with pytest.raises(ValueError, match="belongs to"):
        pool.free(a, "y")
    pool.free(a, "x")
    with pytest.raises(ValueError):
        pool.free(a, "x")               # freed twice
    assert pool.allocate("z") == 2 and pool.allocate("z") == 0   # the freed page comes after older free pages
    with pytest.raises(CacheFullError):
        pool.allocate("w")


def test_layers_are_grouped_by_what_they_need():
    full, windowed = PagedKV(2, 16), PagedKV(2, 16, window=8)
    cache = make([full, windowed, full, None, 0, RequestState((3, 5))])
    assert len(cache.groups) == 2 and cache.groups[0].layers == [0, 2] and cache.groups[1].layers == [1]
    assert cache.groups[0].storage.shape == (2, 2, 12, 2, 4, 16)
    assert cache.layer_view(4).keys.data_ptr() == cache.layer_view(0).keys.data_ptr()   # layer 4 reads layer 0's cache
    assert cache.layer_view(2).keys.data_ptr() != cache.layer_view(0).keys.data_ptr()
    assert cache.layer_view(3).keys is None and cache.layer_view(5).state.shape == (4, 3, 5)


def test_reserve_slots_and_block_tables():
    cache = make([PagedKV(1, 16)], pages=6, page=4)
    cache.create("a")
    assert cache.reserve("a", 5) == 0 and cache.block_table(0, "a") == [0, 1]
    assert cache.slot_mapping(0, "a", 0, 5).tolist() == [0, 1, 2, 3, 4]
    cache.create("b")
    assert cache.reserve("b", 1) == 0 and cache.block_table(0, "b") == [2]
    assert cache.reserve("a", 4) == 5 and cache.block_table(0, "a") == [0, 1, 3]
    assert cache.slot_mapping(0, "a", 5, 4).tolist() == [5, 6, 7, 12]
    assert cache.pages_needed("a", 3) == [0] and cache.pages_needed("a", 4) == [1]
    assert cache.fits([("a", 11), ("b", 3)]) and not cache.fits([("a", 11), ("b", 4)])
    check_invariants(cache)
    cache.free("a")
    assert cache.groups[0].pool.free_pages == 5
    with pytest.raises(KeyError):
        cache.free("a")
    check_invariants(cache)


def test_all_or_nothing_when_pages_run_out_and_the_limit_per_request():
    cache = make([PagedKV(1, 16)], pages=3, page=4, max_pos=64)
    cache.create("a")
    cache.reserve("a", 8)
    cache.create("b")
    with pytest.raises(CacheFullError, match="no free blocks"):
        cache.reserve("b", 5)
    assert cache.requests["b"].length == 0 and cache.block_table(0, "b") == []
    check_invariants(cache)
    small = make([PagedKV(1, 16)], pages=32, page=4, max_pos=10)      # 3 pages per request at most
    small.create("c")
    small.reserve("c", 12)
    with pytest.raises(CacheFullError, match="metadata capacity"):
        small.reserve("c", 1)


def test_window_gives_pages_back_as_it_passes_them():
    cache = make([PagedKV(1, 16, window=6)], pages=4, page=4, max_pos=400)
    cache.create("w")
    for _ in range(100):                     # 100 tokens through a pool of 16 slots
        cache.reserve("w", 1)
        cache.release_passed("w")
        request = cache.requests["w"]
        first_needed = max(0, request.length - 6 + 1)
        table = request.tables[0]
        for page in range(first_needed // 4, len(table)):
            assert table[page] >= 0, "a page inside the window was given back"
        assert all(p == -1 for p in table[:request.released[0]])
        check_invariants(cache)
    assert cache.groups[0].pool.used_pages <= 3
    cache.free("w")
    assert cache.groups[0].pool.free_pages == 4


def test_state_slots_are_zeroed_and_reused():
    cache = make([RequestState((2,)), PagedKV(1, 16)], slots=2)
    a = cache.create("a")
    cache.states.tensors[0][a.state_slot] = 7.0
    cache.create("b")
    with pytest.raises(CacheFullError, match="state slot"):
        cache.create("c")
    cache.free("a")
    c = cache.create("c")
    assert c.state_slot == a.state_slot and float(cache.states.tensors[0][c.state_slot].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_books(seed):
    rng = random.Random(seed)
    cache = make([PagedKV(2, 16), PagedKV(2, 16, window=9), PagedKV(1, 32)], pages=10, page=4, max_pos=200, slots=5)
    live: list[str] = []
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.2 and len(live) < 5:
            counter += 1
            live.append(f"r{counter}")
            cache.create(live[-1])
        elif action < 0.85 and live:
            rid = rng.choice(live)
            count = rng.choice((1, 1, 1, 2, 3, 7, 11))
            before = (cache.requests[rid].length, [list(t) for t in cache.requests[rid].tables])
            try:
                first = cache.reserve(rid, count)
                assert first == before[0]
                cache.release_passed(rid)
            except CacheFullError:
                assert (cache.requests[rid].length, cache.requests[rid].tables) == before
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            cache.free(rid)
        check_invariants(cache)
    for rid in live:
        cache.free(rid)
    assert all(group.pool.free_pages == 10 for group in cache.groups) and len(cache._free_slots) == 5


@pytest.mark.parametrize("seed", range(4))
def test_pages_taken_early_are_found_by_the_next_reserve_or_go_back_with_the_request(seed):
    """``grow`` takes the page of a request's next token before the token is counted in (a decode step
    packed ahead): the next ``reserve`` must give that position in that page and take nothing more;
    a request that ends instead gives the page back; nothing changes when no page is free."""
    rng = random.Random(seed)
    cache = make([PagedKV(2, 16), PagedKV(1, 32)], pages=9, page=4, max_pos=120, slots=4)
    live: list[str] = []
    grown: dict[str, int] = {}
    counter = 0
    for _ in range(500):
        action = rng.random()
        if action < 0.15 and len(live) < 4:
            counter += 1
            live.append(f"r{counter}")
            cache.create(live[-1])
            try:
                cache.reserve(live[-1], rng.randrange(1, 9))
            except CacheFullError:
                pass
        elif action < 0.5 and live:
            rid = rng.choice(live)
            before = [list(t) for t in cache.requests[rid].tables]
            free_before = cache.free_pages()
            if cache.grow(rid, 1):
                grown[rid] = 1
                assert all(len(t) * cache.page_size > cache.requests[rid].length for t in cache.requests[rid].tables)
            else:
                assert [list(t) for t in cache.requests[rid].tables] == before and cache.free_pages() == free_before
        elif action < 0.85 and live:
            rid = rng.choice(live)
            request = cache.requests[rid]
            free_before = cache.free_pages()
            length, tables = request.length, [list(t) for t in request.tables]
            try:
                assert cache.reserve(rid, 1) == length
                if grown.pop(rid, 0):     # the page was there already
                    assert cache.free_pages() == free_before and [list(t) for t in request.tables] == tables
            except CacheFullError:
                assert not grown.get(rid) and request.length == length
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            grown.pop(rid, None)
            cache.free(rid)
        check_invariants(cache, grown)
    for rid in live:
        cache.free(rid)
    assert all(group.pool.free_pages == 9 for group in cache.groups)


def test_stats_report_usage():
    cache = make([PagedKV(1, 16)], pages=8, page=4)
    cache.create("a")
    cache.reserve("a", 6)
    stats = cache.stats(contiguous_max_length=64)
    assert stats["blocks_used"] == 2 and stats["blocks_free"] == 6 and stats["used_tokens"] == 6
    assert stats["paged_waste_tokens"] == 2 and stats["peak_blocks_used"] == 2
    assert cache.kv_bytes_per_token() == 2 * 16 * 4 and cache.capacity_tokens == 32
