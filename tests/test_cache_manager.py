"""Page allocator, cache manager (groups, windows, copy-on-write, state slots) and prefix cache,
on the CPU: no page lost, held twice or freed twice, under random orders of requests."""

import random

import pytest

from clockwork_b200.cache import NO_PAGE, CacheManager, OutOfPages, PageAllocator, PrefixCache, PrefixTree
from clockwork_b200.parts import PagedKVNeed, SlotStateNeed

FULL = PagedKVNeed(2, 16, None)


def manager(num_pages=8, page_size=4, needs=None, **kw):
    return CacheManager(needs or {0: FULL, 1: FULL}, num_pages=num_pages, page_size=page_size, **kw)


# ---- allocator (behaviours of the reference's tests/test_block_allocator.py) ---------------------
def test_allocator_order_reuse_and_errors():
    a = PageAllocator(4, 16)
    assert [a.allocate() for _ in range(4)] == [0, 1, 2, 3]
    with pytest.raises(OutOfPages):
        a.allocate()
    a.free(2)
    a.free(0)
    assert a.allocate() == 0 and a.allocate() == 2  # last freed is handed out first
    with pytest.raises(ValueError, match="out of range"):
        a.free(9)
    a.free(3)
    with pytest.raises(ValueError, match="not allocated"):
        a.free(3)
    with pytest.raises(ValueError):
        PageAllocator(0, 4)


def test_allocate_many_is_all_or_nothing():
    a = PageAllocator(4, 16)
    a.allocate()
    with pytest.raises(OutOfPages):
        a.allocate_many(4)
    assert a.num_free == 3
    assert a.allocate_many(3) == [1, 2, 3]


def test_copy_on_write():
    a = PageAllocator(2, 16)
    p = a.allocate()
    assert a.copy_on_write(p) is None
    a.incref(p)
    assert a.is_shared(p)
    assert a.copy_on_write(p) == (p, 1) and a.refcount(p) == 1 and a.refcount(1) == 1
    a.incref(p)
    with pytest.raises(OutOfPages):  # allocation happens before the shared page is let go
        a.copy_on_write(p)
    assert a.refcount(p) == 2
    a.check_invariants()


# ---- manager ----------------------------------------------------------------------------------------
def test_reserve_slots_and_close():
    m = manager()
    r = m.open("a")
    m.reserve(r, 6)
    assert r.tables == [[0, 1]] and m.slots(r, 0, 0, 6) == [0, 1, 2, 3, 4, 5]
    m.reserve(r, 8)
    assert r.tables == [[0, 1]]
    m.reserve(r, 9)
    assert r.tables == [[0, 1, 2]] and m.slots(r, 0, 8, 9) == [8]
    s = m.open("b")
    m.reserve(s, 3)
    assert s.tables == [[3]] and m.slots(s, 0, 1, 3) == [13, 14]
    assert m.close("a") == []
    with pytest.raises(ValueError, match="double free"):
        m.close("a")
    t = m.open("c")
    m.reserve(t, 5)
    assert t.tables == [[2, 1]]  # freed pages are used again, last freed first
    with pytest.raises(ValueError, match="outside the covered range"):
        m.slots(t, 0, 0, 9)
    m.check_invariants()


def test_out_of_pages_leaves_state_intact():
    m = manager(num_pages=3)
    r = m.open("a")
    m.reserve(r, 8)
    with pytest.raises(OutOfPages):
        m.reserve(r, 17)
    assert r.tables == [[0, 1]] and r.num_tokens == 8 and m.num_free_pages() == [1]
    m.check_invariants()


def test_watermark_thresholds():
    m = manager(num_pages=10, page_size=4, watermark=0.2)  # 2 pages stay free at admission
    assert m.watermark_pages == 2
    assert m.can_open(32) and not m.can_open(33)  # 8 pages + 2 free
    assert m.can_open(40, shared_pages=2)
    r = m.open("a")
    m.reserve(r, 32)
    assert m.can_reserve(r, 40) and not m.can_reserve(r, 40, keep_watermark=True)


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    window = PagedKVNeed(2, 16, 6)
    other = PagedKVNeed(1, 32, None)
    m = manager(num_pages=8, page_size=4, needs={0: FULL, 1: window, 2: FULL, 3: other})
    assert [g.cache_layers for g in m.groups] == [[0, 2], [1], [3]]
    assert m.group_of_layer == {0: 0, 2: 0, 1: 1, 3: 2}
    r = m.open("a")
    m.reserve(r, 20)
    assert all(len(t) == 5 for t in r.tables) and m.num_free_pages() == [3, 3, 3]
    r.num_computed = 20
    # a query at position >= 20 reads keys >= 15: pages 0..2 (positions 0..11) are behind the window
    assert m.release_behind_window(r, 20) == 3
    assert r.tables[1] == [NO_PAGE, NO_PAGE, NO_PAGE, 3, 4] and r.tables[0] == [0, 1, 2, 3, 4]
    assert m.num_free_pages() == [3, 6, 3]
    assert m.release_behind_window(r, 20) == 0
    with pytest.raises(ValueError, match="already given back"):
        m.slots(r, 1, 0, 4)
    m.reserve(r, 24)
    assert r.tables[1][-1] == 2  # a page the window gave back is used again
    m.check_invariants()
    m.close("a")
    assert m.num_free_pages() == [8, 8, 8]
    m.check_invariants()


def test_fork_shares_pages_and_first_write_copies():
    m = manager(num_pages=6, page_size=4)
    parent = m.open("p")
    m.reserve(parent, 6)
    parent.num_computed = 6
    child = m.fork(parent, "c")
    assert child.tables == [[0, 1]] and m.groups[0].allocator.refcount(1) == 2
    assert m.pages_needed(child, 7) == [1]  # the shared tail page must be copied
    m.reserve(child, 7)
    assert child.tables == [[0, 2]] and parent.tables == [[0, 1]]
    assert m.groups[0].allocator.refcount(0) == 2 and m.groups[0].allocator.refcount(1) == 1
    m.check_invariants()
    m.close("p")
    m.close("c")
    assert m.num_free_pages() == [6]


def test_state_slots():
    m = manager(needs={0: FULL, 1: SlotStateNeed((3, 2))}, num_state_slots=2)
    a, b = m.open("a"), m.open("b")
    assert {a.state_slot, b.state_slot} == {0, 1}
    assert not m.can_open(1)
    with pytest.raises(OutOfPages, match="state slots"):
        m.open("c")
    assert "c" not in m.requests
    freed = a.state_slot
    m.close("a")
    assert m.can_open(1) and m.open("d").state_slot == freed
    m.check_invariants()
    # a model whose mixers keep no state of their own still has the slot pool: every request takes a
    # slot (the column of its progress and sampling state on the device) and gives it back
    plain = manager()
    assert plain.state.num_free == 64 and plain.open("x").state_slot == 0 and plain.state.num_free == 63
    plain.close("x")
    assert plain.state.num_free == 64


def test_shared_prefix_needs_a_single_full_group():
    m = manager(needs={0: FULL, 1: PagedKVNeed(2, 16, 8)})
    with pytest.raises(ValueError, match="single group"):
        m.open("a", shared_prefix=[0])


def test_manager_fuzz_random_orders():
    rng = random.Random(7)
    window = PagedKVNeed(2, 16, 9)
    m = manager(num_pages=24, page_size=4, needs={0: FULL, 1: window, 2: SlotStateNeed((2,))}, num_state_slots=5)
    live: dict[str, int] = {}
    counter = 0
    for step in range(3000):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{counter}"
            counter += 1
            m.open(rid)
            live[rid] = 0
        elif op < 0.75 and live:
            rid = rng.choice(sorted(live))
            req = m.get(rid)
            new_len = live[rid] + rng.randint(1, 9)
            if m.can_reserve(req, new_len):
                m.reserve(req, new_len)
                req.num_computed = new_len
                live[rid] = new_len
                m.release_behind_window(req, new_len)
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(req, new_len)
        elif op < 0.85 and live and len(live) < 5:
            rid = rng.choice(sorted(live))
            child = f"r{counter}"
            counter += 1
            m.fork(m.get(rid), child)
            live[child] = live[rid]
        elif live:
            rid = rng.choice(sorted(live))
            m.close(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            req = m.get(rid)
            assert len(req.tables[0]) * 4 >= n
            if n:
                m.slots(req, 0, 0, n)  # every position of the full group still has its page
                lo = max(0, n - 9 + 1)
                m.slots(req, 1, lo, n)  # and the window's positions in the windowed group
    for rid in sorted(live):
        m.close(rid)
    assert m.num_free_pages() == [24, 24] and m.state.num_free == 5


# ---- prefix tree and cache (behaviours of the reference's tests/test_radix.py) -------------------
def test_tree_matches_whole_pages_only():
    t = PrefixTree(4)
    assert t.insert(list(range(10)), [7, 8, 9]) == [7, 8]  # two whole pages
    assert t.match(list(range(10))) == [7, 8]
    assert t.match([0, 1, 2, 3, 4, 5, 6, 99]) == [7]  # divergence inside the second page
    assert t.match([0, 1, 2, 99]) == []
    assert t.match([0, 1, 2]) == []
    # same first token, divergence inside the first page: separate branches
    assert t.insert([0, 1, 2, 99, 5, 5, 5, 5], [3, 4]) == [3, 4]
    assert t.match([0, 1, 2, 99, 5, 5, 5, 5]) == [3, 4] and t.match(list(range(8))) == [7, 8]
    # inserting a span the tree already holds adopts only what is new
    assert t.insert(list(range(12)), [20, 21, 22]) == [22]
    assert t.match(list(range(12))) == [7, 8, 22]


def test_tree_eviction_is_lru_over_unlocked_leaves():
    t = PrefixTree(2)
    t.insert([1, 1, 2, 2], [0, 1])
    t.insert([1, 1, 3, 3], [0, 2])
    t.insert([4, 4], [3])
    t.match([1, 1, 2, 2])  # touch branch 2 -> page 2 and 3 are older
    t.lock(3)
    assert t.evictable_pages() == 3
    assert t.evict(1) == [2]
    assert t.evict(5) == [1, 0]  # page 0 becomes a leaf once its children are gone; 3 is locked
    assert t.pages() == [3]
    t.unlock(3)
    assert t.evict(1) == [3] and t.num_pages() == 0


def test_prefix_cache_reference_counts_full_cycle():
    a = PageAllocator(8, 4)
    cache = PrefixCache(a, 4)
    pages = a.allocate_many(3)
    tokens = list(range(10))
    assert cache.match(tokens).num_tokens == 0
    cache.insert(tokens, pages)  # adopts the two whole pages
    assert [a.refcount(p) for p in pages] == [2, 2, 1]
    a.free_many(pages)  # the request ends; the tree keeps its pages
    assert a.num_free == 6
    hit = cache.match(tokens)
    assert hit.num_tokens == 8 and hit.pages == pages[:2] and a.refcount(pages[0]) == 2
    # never the whole sequence: 8 tokens match only one page
    assert cache.match(list(range(8))).num_tokens == 4
    cache.release(pages[:1])
    assert cache.evict(8) == 0  # the deepest matched page is locked, its ancestors are no leaves
    cache.release(hit.pages)
    assert cache.evict(8) == 2 and a.num_free == 8
    assert cache.stats.queries == 3 and cache.stats.hit_tokens == 12
    a.check_invariants()


def test_prefix_cache_disabled_and_reset():
    a = PageAllocator(4, 2)
    off = PrefixCache(a, 2, enabled=False)
    off.insert([1, 2, 3, 4], a.allocate_many(2))
    assert off.match([1, 2, 3, 4, 5]).num_tokens == 0 and off.tree.num_pages() == 0
    on = PrefixCache(a, 2)
    on.insert([1, 2, 3, 4], [0, 1])
    on.reset()
    assert a.refcount(0) == 1 and on.tree.num_pages() == 0


def test_prefix_cache_fuzz_against_a_dictionary():
    """Random inserts, matches, releases and evictions against a model that stores every cached
    page-aligned prefix in a dict (after the reference's tests/test_radix.py:267)."""
    rng = random.Random(3)
    ps = 2
    a = PageAllocator(64, ps)
    cache = PrefixCache(a, ps)
    model: dict[tuple, int] = {}  # page-aligned token prefix -> page
    held: list[list[int]] = []  # matches not yet released
    for _ in range(1500):
        op = rng.random()
        tokens = [rng.randint(0, 2) for _ in range(rng.randint(1, 9))]
        if op < 0.4:
            n = len(tokens) // ps
            # a request: pages for the matched prefix come from the cache, the rest are new
            hit = cache.match(tokens)
            own = []
            try:
                own = a.allocate_many((len(tokens) + ps - 1) // ps - len(hit.pages))
            except OutOfPages:
                cache.release(hit.pages)
                cache.evict(8)
                for key in [k for k, p in model.items() if not cache.tree.holds(p)]:
                    del model[key]
                continue
            table = hit.pages + own
            cache.insert(tokens, table)
            for i in range(n):
                model.setdefault(tuple(tokens[: (i + 1) * ps]), table[i])
            a.free_many(own)
            cache.release(hit.pages)
        elif op < 0.7:
            hit = cache.match(tokens)
            cap = (len(tokens) - 1) // ps
            want = []
            for i in range(cap):
                page = model.get(tuple(tokens[: (i + 1) * ps]))
                if page is None:
                    break
                want.append(page)
            assert hit.pages == want
            held.append(hit.pages)
        elif op < 0.85 and held:
            cache.release(held.pop(rng.randrange(len(held))))
        else:
            cache.evict(rng.randint(1, 4))
            for key in [k for k, p in model.items() if not cache.tree.holds(p)]:
                del model[key]
        a.check_invariants()
        expected = {p: 1 for p in cache.tree.pages()}
        for pages in held:
            for p in pages:
                expected[p] = expected.get(p, 0) + 1
        for p in range(a.num_pages):
            assert a.refcount(p) == expected.get(p, 0)
        # a prefix in the tree always has its parent prefix in the tree
        for key in model:
            if len(key) > ps:
                assert key[:-ps] in model
    for pages in held:
        cache.release(pages)
    cache.reset()
    assert a.num_free == 64
