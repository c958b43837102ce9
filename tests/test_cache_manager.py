"""The page pool and the cache manager on the host (no GPU): order of reuse, reference
counts, prefix hashes, windows, state slots, and invariants under random request orders."""

import random

import pytest

from jax_vllm_b200.cache import CacheManager, OutOfPages, PagePool, chain_hash
from jax_vllm_b200.parts import FixedStateNeed, PagedKVNeed

FULL = PagedKVNeed(2, 16)
WIN = PagedKVNeed(2, 16, window=20)
WIN8 = PagedKVNeed(2, 16, window=8)


def test_alloc_order_and_reversed_release():
    # as the reference's pool behaves (tests/test_paged.py:87-106), minus its sink page
    pool = PagePool(7)
    got = [pool.alloc() for _ in range(3)]
    assert got == [0, 1, 2]
    pool.release(got)
    assert pool.free_pages() == [3, 4, 5, 6, 2, 1, 0]
    pool.check()


def test_out_of_pages_and_double_release():
    pool = PagePool(2)
    a, b = pool.alloc(), pool.alloc()
    with pytest.raises(OutOfPages):
        pool.alloc()
    pool.release([a])
    with pytest.raises(RuntimeError, match="more often"):
        pool.release([a])
    pool.release([b])
    assert pool.num_free == 2
    pool.check()


def test_touch_takes_a_cached_page_off_the_free_list_and_alloc_evicts_hashes():
    pool = PagePool(3)
    p = pool.alloc()
    h = chain_hash(b"", [1, 2, 3])
    pool.register(p, h)
    pool.release([p])
    assert pool.lookup(h) == p and p in pool.free_pages()
    pool.touch(p)
    assert p not in pool.free_pages() and pool.ref[p] == 1
    pool.touch(p)
    pool.release([p]); pool.release([p])
    # p is now at the tail; taking every page drops its hash when p is handed out again
    for _ in range(3):
        pool.alloc()
    assert pool.lookup(h) is None
    pool.check()


def test_first_hash_and_first_page_win():
    pool = PagePool(4)
    a, b = pool.alloc(), pool.alloc()
    h1, h2 = chain_hash(b"", [1]), chain_hash(b"", [2])
    pool.register(a, h1); pool.register(b, h1); pool.register(a, h2)
    assert pool.lookup(h1) == a and pool.lookup(h2) is None and pool.hash_of[b] is None


def test_chain_hash_depends_on_parent_and_tokens():
    h = chain_hash(b"", [1, 2])
    assert h == chain_hash(b"", [1, 2]) and h != chain_hash(b"", [2, 1]) and h != chain_hash(h, [1, 2])


def test_groups_by_need_and_state_layers():
    m = CacheManager([FULL, WIN, FULL, None, FixedStateNeed((4, 3)), WIN], page_size=8, num_pages=10, max_live=2)
    assert [g.layers for g in m.groups] == [[0, 2], [1, 5]]
    assert m.layer_group == {0: 0, 2: 0, 1: 1, 5: 1} and list(m.state_layers) == [4]
    assert m.prefix_cache is False          # fixed state switches prefix reuse off
    assert CacheManager([FULL, WIN], page_size=8, num_pages=10, max_live=2).prefix_cache is True
    assert m.bytes_per_page(2) == 2 * (2 * 2 * 8 * 2 * 16 * 2)


def test_grow_commit_release_and_slots():
    m = CacheManager([FULL, FULL], page_size=4, num_pages=6, max_live=2, prefix_cache=False)
    a = m.admit("a")
    assert a.slot == 0 and m.pages_needed(a, 9) == [3]
    m.grow(a, 9); m.commit(a, list(range(9)))
    b = m.admit("b")
    assert b.slot == 1 and not m.can_admit()
    assert m.max_len_allocatable(b) == 12 and not m.can_grow(b, 13)
    with pytest.raises(OutOfPages):
        m.grow(b, 13)
    assert b.tables == [[]]                  # all or nothing
    m.grow(b, 12); m.check()
    m.release("a"); m.check()
    assert m.groups[0].pool.num_free == 3 and m.can_admit()
    c = m.admit("c")
    assert c.slot == 0
    m.release("b"); m.release("c"); m.check()
    assert m.groups[0].pool.num_free == 6
    with pytest.raises(KeyError):
        m.release("c")


def test_window_pages_are_given_back_as_the_window_passes():
    m = CacheManager([WIN], page_size=8, num_pages=5, max_live=1)
    rc = m.admit("r")
    n = 0
    for step in range(12):
        m.grow(rc, n + 7)
        m.commit(rc, [0] * 7)
        n += 7
        first_needed = max(0, n - 20 + 1)
        assert all((p == -1) == ((i + 1) * 8 <= first_needed) for i, p in enumerate(rc.tables[0]))
        assert sum(p >= 0 for p in rc.tables[0]) <= 4
        m.check()
    assert n == 84                          # far more tokens than the 40 the pool holds
    m.release("r"); m.check()
    assert m.groups[0].pool.num_free == 5


def test_prefix_reuse_hits_full_pages_but_leaves_a_token():
    m = CacheManager([FULL], page_size=4, num_pages=8, max_live=2)
    toks = list(range(100, 112))            # three full pages
    a = m.admit("a", toks)
    assert a.num_tokens == 0
    m.grow(a, 12); m.commit(a, toks)
    assert len(a.hashes) == 3
    b = m.admit("b", toks)                  # same prompt: 2 pages hit, the last page is computed
    assert b.num_tokens == 8 and b.tables[0] == a.tables[0][:2]
    assert [m.groups[0].pool.ref[p] for p in a.tables[0]] == [2, 2, 1]
    m.check()
    m.release("a"); m.release("b"); m.check()
    c = m.admit("c", toks + [7])            # freed pages keep content and hash: 3 pages hit now
    assert c.num_tokens == 12 and m.stats["prefix_hit_pages"] == 5
    d = m.admit("d", [1] + toks)            # different first page: nothing
    assert d.num_tokens == 0
    m.check()


def test_prefix_reuse_with_a_window_takes_only_the_pages_the_window_reaches():
    m = CacheManager([FULL, WIN], page_size=4, num_pages=12, max_live=2)      # the window is 20 positions
    toks = list(range(200, 241))            # ten full pages and a token
    a = m.admit("a", toks)
    m.grow(a, 41); m.commit(a, toks)
    assert a.tables[1][:5] == [-1] * 5 and all(p >= 0 for p in a.tables[1][5:])   # keys before 41 - 20 + 1 = 22 are gone
    b = m.admit("b", toks)
    # ten pages hit; a query at 40 sees keys from 21 on: page 5 (positions 20..23) is the first one needed
    assert b.num_tokens == 40 and b.tables[0] == a.tables[0][:10]
    assert b.tables[1] == [-1] * 5 + a.tables[1][5:10] and b.freed_upto == [0, 5]
    assert m.stats["prefix_hit_pages"] == 10 and m.stats["prefix_hit_tokens"] == 40
    m.check()
    m.grow(b, 41); m.commit(b, toks[40:])
    assert b.tables[1][:6] == [-1] * 5 + [a.tables[1][5]]       # 41 - 20 + 1 = 22: page 5 is still needed
    m.release("a"); m.release("b"); m.check()
    # a shorter prompt with the same start: its window would reach pages that the window group gave back and that
    # have been handed out again since, so the hit shrinks to what every group still has
    c = m.admit("c", [1, 2, 3, 4] * 6); m.grow(c, 24); m.commit(c, [1, 2, 3, 4] * 6); m.release("c")
    d = m.admit("d", toks[:25])
    win_known = [m.groups[1].pool.lookup(h) is not None for h in a.hashes[:6]]
    want = max(n for n in range(7) if all(win_known[max(0, n * 4 - 19) // 4:n]))
    assert d.num_tokens == 4 * want and all((p >= 0) == (i >= max(0, 4 * want - 19) // 4) for i, p in enumerate(d.tables[1]))
    m.check()
    m.release("d"); m.check()
    assert all(g.pool.num_free == 12 for g in m.groups)


def test_prefix_reuse_with_windows_only():
    m = CacheManager([WIN], page_size=4, num_pages=12, max_live=2)
    toks = list(range(300, 333))
    a = m.admit("a", toks); m.grow(a, 33); m.commit(a, toks)
    b = m.admit("b", toks + [5, 6])         # eight pages known by hash; the window reaches back to page 3
    assert b.num_tokens == 32 and b.tables[0] == [-1] * 3 + a.tables[0][3:8] and b.freed_upto == [3]
    m.check()
    c_prompt = toks[:13]                    # a hit of three pages would need pages 0..2, which were given back
    m.release("a"); m.release("b"); m.check()
    c = m.admit("c", c_prompt)
    known = [m.groups[0].pool.lookup(h) is not None for h in a.hashes[:3]]
    assert c.num_tokens == 4 * max(n for n in range(4) if all(known[:n]))
    m.check()


def test_eviction_drops_prefix():
    m = CacheManager([FULL], page_size=2, num_pages=3, max_live=2)
    a = m.admit("a", [1, 2, 3, 4, 5]); m.grow(a, 5); m.commit(a, [1, 2, 3, 4, 5]); m.release("a")
    b = m.admit("b", [9, 9, 9, 9, 9, 9])    # takes all three pages: a's hashes go
    m.grow(b, 6); m.commit(b, [9] * 6); m.release("b")
    c = m.admit("c", [1, 2, 3, 4, 5])
    assert c.num_tokens == 0
    m.check()


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("needs,prefix", [([FULL, FULL], True), ([FULL, WIN], False), ([FULL], False),
                                          ([FULL, WIN], True), ([WIN, WIN8], True)])
def test_random_orders_lose_no_page(seed, needs, prefix):
    rng = random.Random(seed)
    m = CacheManager(needs, page_size=4, num_pages=24, max_live=4, prefix_cache=prefix)
    shared = [rng.randrange(50) for _ in range(32)]
    live, next_id = {}, 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and m.can_admit():
            prompt = (shared[: rng.choice([0, 4, 8, 16, 32])] + [rng.randrange(50) for _ in range(rng.randrange(1, 20))])
            rc = m.admit(next_id, prompt)
            assert rc.num_tokens < len(prompt)
            for g, grp in enumerate(m.groups):      # every page that the first query can see is there
                first = 0 if grp.need.window is None else max(0, rc.num_tokens - grp.need.window + 1) // 4
                assert len(rc.tables[g]) == rc.num_tokens // 4
                assert all((p >= 0) == (i >= first) for i, p in enumerate(rc.tables[g]))
            live[next_id] = (rc, prompt)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            rc, toks = live[rid]
            n = rng.randrange(1, 9)
            new = (toks[rc.num_tokens:rc.num_tokens + n] + [rng.randrange(50) for _ in range(n)])[:n]
            if m.can_grow(rc, rc.num_tokens + n):
                before = rc.num_tokens
                m.grow(rc, before + n)
                m.commit(rc, new)
                assert rc.num_tokens == before + n
            else:
                with pytest.raises(OutOfPages):
                    m.grow(rc, rc.num_tokens + n)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for g in m.groups:                  # no page is in two live tables unless it is a shared prefix page
            seen = {}
            for rc, _ in live.values():
                for p in rc.tables[m.groups.index(g)]:
                    if p >= 0:
                        seen[p] = seen.get(p, 0) + 1
            assert all(n == g.pool.ref[p] for p, n in seen.items())
            if not prefix:
                assert all(n == 1 for n in seen.values())
    for rid in list(live):
        m.release(rid)
    m.check()
    assert (m.stats["prefix_hit_pages"] > 0) == prefix
    assert all(g.pool.num_free == 24 for g in m.groups) and m.slots.num_free == 4


def test_page_table_behaves_like_a_list():
    from jax_vllm_b200.cache.manager import PageTable
    t, ref = PageTable(), []
    for i in range(100):                     # grows past its first allocation
        t.append(3 * i + 1)
        ref.append(3 * i + 1)
    assert len(t) == 100 and list(t) == ref and t == ref and t[:7] == ref[:7] and t[-1] == ref[-1]
    t[5] = -1
    ref[5] = -1
    assert t[5] == -1 and isinstance(t[5], int) and t.array(8).tolist() == ref[:8]
    assert t.array().dtype.name == "int32" and sum(p >= 0 for p in t) == 99
    with pytest.raises(IndexError):
        t[100]
    with pytest.raises(IndexError):
        t[100] = 0
