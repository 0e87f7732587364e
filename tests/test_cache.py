"""The cache manager's books: no page lost, held twice or freed twice, under random orders
of requests; window groups give pages back while a request lives; state slots."""
import random

import pytest
import torch

from microllm_rocm_b200.cache import CacheManager, PageError, PagePool, RELEASED
from microllm_rocm_b200.parts.base import FixedStateNeed, PagedKVNeed


def manager(num_pages=12, page_size=16, max_requests=4, window=32, with_state=False):
    entries = {"l0": PagedKVNeed(2, 32, None), "l1": PagedKVNeed(2, 32, window), "l2": PagedKVNeed(1, 16, window)}
    if with_state:
        entries["s"] = FixedStateNeed((4, 3))
    return CacheManager(entries, page_size, num_pages, max_requests)


def test_pool_is_lifo_and_refuses_double_free():
    pool = PagePool(4)
    a, b = pool.alloc(), pool.alloc()
    assert (a, b) == (0, 1)
    pool.free(a)
    assert pool.alloc() == a, "a page given back is the next one handed out"
    pool.free(b)
    with pytest.raises(PageError, match="double free"):
        pool.free(b)
    with pytest.raises(PageError):
        pool.free(3)
    for _ in range(3):
        pool.alloc()
    assert pool.alloc() is None and pool.free_count == 0
    pool.check()


def test_layers_with_the_same_need_share_a_group_and_its_table():
    c = manager()
    assert set(c.groups) == {"full", "window32"}
    assert c.entry_group == {"l0": "full", "l1": "window32", "l2": "window32"}


def test_reserve_is_all_or_nothing_across_groups():
    c = manager(num_pages=4)
    c.add("a"); c.add("b")
    assert c.reserve("a", 48) and c.reserve("b", 16)
    before = {k: g.pool.free_count for k, g in c.groups.items()}
    assert not c.reserve("b", 48)                       # needs 2 more, 0 free
    assert {k: g.pool.free_count for k, g in c.groups.items()} == before
    c.check()


def test_window_group_gives_pages_back_while_the_request_lives():
    c = manager(num_pages=12, window=32)
    c.add("a")
    assert c.reserve("a", 100)
    c.commit("a", 100)
    t = c.requests["a"].tables
    assert RELEASED not in t["full"]
    # the next query (position 100) reads keys >= 69: blocks 0..3 (tokens 0..63) are dead
    assert t["window32"][:4] == [RELEASED] * 4 and RELEASED not in t["window32"][4:]
    assert c.groups["window32"].pool.used_count == 3 and c.groups["full"].pool.used_count == 7
    # freed pages are handed out again at once
    c.add("b")
    assert c.reserve("b", 16)
    assert c.requests["b"].tables["window32"][0] in (0, 1, 2, 3)
    c.check()
    c.release("a"); c.release("b")
    c.check()
    assert all(g.pool.used_count == 0 for g in c.groups.values())


def test_commit_without_pages_and_shrinking_are_refused():
    c = manager()
    c.add("a")
    with pytest.raises(PageError):
        c.commit("a", 20)
    c.reserve("a", 20); c.commit("a", 20)
    with pytest.raises(ValueError):
        c.commit("a", 10)
    with pytest.raises(KeyError):
        c.add("a")


def test_state_slots_are_per_request_and_reused():
    c = manager(max_requests=2, with_state=True)
    assert c.add("a") and c.add("b")
    assert not c.add("c"), "no slot left"
    assert {c.slot("a"), c.slot("b")} == {0, 1}
    s = c.slot("a")
    c.release("a")
    assert c.add("c") and c.slot("c") == s
    c.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_duplicate_a_page(seed):
    rng = random.Random(seed)
    c = manager(num_pages=rng.choice([6, 9, 15]), page_size=rng.choice([4, 16]), max_requests=5,
                window=rng.choice([8, 32]), with_state=True)
    live, next_id, refused = {}, 0, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            if c.add(next_id):
                live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            q = rng.choice(list(live))
            n = live[q] + rng.choice([1, 1, 1, 2, 7, 19, 40])
            if c.reserve(q, n):
                c.commit(q, n)
                live[q] = n
            else:
                refused += 1
        elif live:
            q = rng.choice(list(live))
            c.release(q)
            del live[q]
        c.check()
        for q, n in live.items():
            assert c.length(q) == n
            for key, group in c.groups.items():
                table = c.requests[q].tables[key]
                first = 0 if group.window is None else max(0, n - group.window + 1)
                for b in range(first // c.page_size, c.blocks_for(n)):
                    assert table[b] != RELEASED, "a block a later query may read was given back"
    assert refused > 0, "the pool was never tight"
    for q in list(live):
        c.release(q)
    c.check()
    assert all(g.pool.used_count == 0 for g in c.groups.values()) and c.slots.used_count == 0


def test_a_window_group_needs_pages_for_its_window_only():
    """With a promise on how many tokens a request brings per step, the pool of a windowed group is sized for
    the spans that can be live (window - 1 + step tokens per request), not for whole sequences; a request that
    runs far beyond the window never fails to get its pages, and the books stay right."""
    from microllm_rocm_b200.cache.manager import CacheManager
    from microllm_rocm_b200.parts.base import PagedKVNeed
    entries = {"full": PagedKVNeed(2, 32, None), "win": PagedKVNeed(2, 32, 40)}
    cache = CacheManager(entries, page_size=16, num_pages=200, max_requests=3, max_step_tokens=24)
    assert cache.groups["full"].pool.num_pages == 200
    assert cache.groups["window40"].pool.num_pages == 3 * (-(-(39 + 24) // 16) + 1) == 15
    rng = random.Random(5)
    lengths = {}
    for rid in ("a", "b", "c"):
        assert cache.add(rid)
        lengths[rid] = 0
    for _ in range(300):
        rid = rng.choice(list(lengths))
        n = rng.randint(1, 24)
        if lengths[rid] + n > 1000:
            continue
        assert cache.reserve(rid, lengths[rid] + n), (rid, lengths[rid], n)
        lengths[rid] += n
        cache.commit(rid, lengths[rid])
        cache.check()
    assert max(lengths.values()) > 500
    assert cache.groups["window40"].pool.peak_used <= 15
    for rid in lengths:
        cache.release(rid)
    cache.check()
    assert cache.groups["window40"].pool.used_count == 0 and cache.groups["full"].pool.used_count == 0


def test_guard_pages_show_a_store_outside_the_pool():
    """With guard_pages every paged entry has a page of a fixed pattern in front of and behind its pool.  The
    pool's own pages are where they would be without guards (the entry's tensor starts one page in); a value
    written just outside either end is found by check_guards()."""
    import torch
    from microllm_rocm_b200.cache.manager import GUARD_VALUE
    from microllm_rocm_b200.cache.pages import PageError
    entries = {"run0": PagedKVNeed(2, 8), "run1": PagedKVNeed(1, 16, window=24), "run2": FixedStateNeed((4,))}
    cache = CacheManager(entries, page_size=16, num_pages=6, max_requests=2, device=torch.device("cpu"),
                         kv_dtype=torch.bfloat16, guard_pages=True)
    for name in ("run0", "run1"):
        pool, whole = cache.kv_storage[name], cache.guarded[name]
        assert pool.is_contiguous() and pool.shape[0] == whole.shape[0] - 2
        assert pool.data_ptr() == whole.data_ptr() + whole[0].numel() * whole.element_size()
        assert float(whole[0].float().min()) == GUARD_VALUE == float(whole[-1].float().max())
        assert float(pool.float().abs().max()) == 0.0
    cache.check_guards()
    cache.kv_storage["run0"].fill_(1.0)                   # every legal store
    cache.check_guards()
    cache.guarded["run1"][-1, 0, 0, 0, 3] = 0.5            # one element past the last page
    with pytest.raises(PageError, match="run1.*behind"):
        cache.check_guards()
    cache.guarded["run1"][-1].fill_(GUARD_VALUE)
    cache.guarded["run0"][0, 1, 1, 15, 7] = 2.0            # the last element before the first page
    with pytest.raises(PageError, match="run0.*in front"):
        cache.check_guards()
    plain_cache = CacheManager(entries, page_size=16, num_pages=6, max_requests=2, device=torch.device("cpu"))
    assert not plain_cache.guarded
    plain_cache.check_guards()                            # nothing to check, nothing raised
