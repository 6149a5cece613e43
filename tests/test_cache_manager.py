"""Cache manager: no page lost, held twice or freed twice, under random orders of requests."""

import random

import numpy as np
import pytest

from pagedserve_b200.cache import CacheError, CacheFull, CacheManager, KVNeed, PageAllocator, StateNeed


def manager(pages=16, page=4, window=None, slots=4, max_len=64, mixed=False):
    needs = [KVNeed(2, 16, None), KVNeed(2, 16, window)] if mixed else [KVNeed(2, 16, window)] * 2
    return CacheManager(needs, [None, None], page, pages, slots, max_len)


def test_allocator_lifo_and_double_free():
    pool = PageAllocator(4)
    assert [pool.allocate() for _ in range(4)] == [3, 2, 1, 0]      # highest id first
    with pytest.raises(CacheFull, match="KV cache full"):
        pool.allocate()
    pool.release(2)
    assert pool.allocate() == 2                                       # the page just freed comes back first
    pool.release(1)
    with pytest.raises(CacheError, match="freed twice"):
        pool.release(1)
    with pytest.raises(CacheError):
        pool.release(9)
    assert pool.peak_used == 4


def test_extend_commit_free_cycle():
    cache = manager()
    assert cache.admit("a") == 0
    cache.extend("a", 5)
    assert cache.groups[0].tables["a"] == [15, 14]
    with pytest.raises(CacheError, match="not committed"):
        cache.extend("a", 1)
    assert cache.commit("a") == 5
    cache.extend("a", 3)                       # positions 5..7 fit in the second page
    assert cache.groups[0].tables["a"] == [15, 14]
    cache.commit("a")
    cache.extend("a", 1)                       # position 8 opens a third page
    assert cache.groups[0].tables["a"] == [15, 14, 13]
    with pytest.raises(CacheError, match="uncommitted"):
        cache.free("a")
    cache.commit("a")
    row = np.zeros(16, dtype=np.int32)
    cache.table_row(0, "a", row)
    assert row.tolist() == [15, 14, 13] + [-1] * 13
    cache.free("a")
    cache.check_invariants()
    assert cache.free_pages() == 16 and cache.free_slots == 4
    with pytest.raises(CacheError, match="unknown request"):
        cache.free("a")
    with pytest.raises(CacheError, match="nothing to commit"):
        cache.admit("b")
        cache.commit("b")


def test_extend_is_all_or_nothing_and_rollback():
    cache = manager(pages=4, page=4)
    cache.admit("a"); cache.extend("a", 9); cache.commit("a")      # 3 pages
    cache.admit("b")
    with pytest.raises(CacheFull):
        cache.extend("b", 6)                                         # needs 2, only 1 left
    assert cache.free_pages() == 1 and cache.groups[0].tables["b"] == []
    cache.check_invariants()
    cache.extend("b", 4)
    cache.rollback("b")                                              # the step failed
    assert cache.free_pages() == 1 and cache.length("b") == 0
    cache.check_invariants()
    with pytest.raises(CacheError, match="maximum length"):
        cache.extend("b", 65)


def test_slots_run_out_and_are_reused():
    cache = manager(slots=2)
    cache.admit("a"); cache.admit("b")
    with pytest.raises(CacheFull, match="slot"):
        cache.admit("c")
    with pytest.raises(CacheError, match="already live"):
        cache.admit("a")
    cache.free("a")
    assert cache.admit("c") == 0


def test_window_group_gives_pages_back_while_full_group_keeps_them():
    cache = manager(pages=8, page=4, window=6, mixed=True)
    full, windowed = cache.groups
    assert full.need.window is None and windowed.need.window == 6
    cache.admit("a")
    for _ in range(5):
        cache.extend("a", 4)
        cache.commit("a")
    # 20 tokens: the next token (position 20) needs keys 15..20 -> pages 0..2 (positions < 12) passed
    assert windowed.tables["a"] == [-1, -1, -1, 7, 6]      # pages 7 and 6 were passed, freed and handed out again
    assert full.tables["a"] == [7, 6, 5, 4, 3]
    assert windowed.allocator.free_pages == 6 and full.allocator.free_pages == 3
    cache.check_invariants()
    cache.extend("a", 4); cache.commit("a")
    assert windowed.tables["a"][5] == 5           # a page the window had passed is handed out again
    cache.free("a")
    cache.check_invariants()
    assert windowed.allocator.free_pages == 8 and full.allocator.free_pages == 8


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 7])
def test_random_orders_keep_every_page_accounted_for(seed, window):
    rng = random.Random(seed)
    cache = manager(pages=24, page=4, window=window, slots=5, max_len=48, mixed=window is not None)
    live = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and cache.free_slots:
            name = f"r{counter}"; counter += 1
            cache.admit(name); live[name] = 0
        elif action < 0.8 and live:
            name = rng.choice(list(live))
            count = rng.randint(1, 9)
            if live[name] + count > 48:
                continue
            try:
                cache.extend(name, count)
            except CacheFull:
                cache.check_invariants()
                continue
            if rng.random() < 0.1:
                cache.rollback(name)
            else:
                live[name] = cache.commit(name)
                assert live[name] == cache.length(name)
        elif live:
            name = rng.choice(list(live))
            cache.free(name); del live[name]
        cache.check_invariants()
        for group in cache.groups:
            for name, length in live.items():
                table = group.tables[name]
                first = group.first_needed_position(length) // 4
                needed = -(-length // 4)
                assert all(page >= 0 for page in table[first:needed]), "a page still in use was given back"
    for name in list(live):
        cache.free(name)
    cache.check_invariants()
    assert all(g.allocator.free_pages == g.num_pages for g in cache.groups)


def test_state_slots_are_declared_per_layer():
    cache = CacheManager([None, KVNeed(1, 16)], [StateNeed((3, 4)), None], 8, 4, 2, 32)
    assert cache.state == {}                        # no device: bookkeeping only
    assert cache.state_needs[0].shape == (3, 4) and cache.group_of_layer == {1: 0}
    with pytest.raises(CacheError):
        CacheManager([KVNeed(1, 16)], [None], 12, 4, 2, 32)


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 7])
def test_batched_extend_and_commit_equal_one_by_one(seed, window):
    """``extend_many`` / ``commit_many`` leave the manager exactly as the same calls one by one do: same
    pages in the same order, same tables, same lengths; and a batch that does not fit takes nothing."""
    rng = random.Random(100 + seed)
    batched = manager(pages=20, page=4, window=window, slots=6, max_len=48, mixed=window is not None)
    single = manager(pages=20, page=4, window=window, slots=6, max_len=48, mixed=window is not None)
    live = []
    counter = 0
    refused = 0
    for _ in range(300):
        action = rng.random()
        if action < 0.2 and batched.free_slots:
            name = f"r{counter}"; counter += 1
            batched.admit(name); single.admit(name); live.append(name)
        elif action < 0.9 and live:
            chosen = rng.sample(live, rng.randint(1, len(live)))
            counts = [1 if rng.random() < 0.6 else rng.randint(2, 9) for _ in chosen]
            if any(single.length(name) + count > 48 for name, count in zip(chosen, counts)):
                continue
            free_before = [g.allocator.free_pages for g in batched.groups]
            try:
                batched.extend_many(chosen, counts)
            except CacheFull:
                refused += 1
                assert [g.allocator.free_pages for g in batched.groups] == free_before    # all or nothing
                assert not batched.pending.any()
                batched.check_invariants()
                continue
            for name, count in zip(chosen, counts):
                single.extend(name, count)
            if rng.random() < 0.1:
                for name in chosen:
                    batched.rollback(name); single.rollback(name)
            else:
                batched.commit_many(chosen)
                for name in chosen:
                    single.commit(name)
        elif live:
            name = live.pop(rng.randrange(len(live)))
            batched.free(name); single.free(name)
        batched.check_invariants()
        assert (batched.lengths == single.lengths).all() and (batched.pending == single.pending).all()
        for g_batched, g_single in zip(batched.groups, single.groups):
            assert g_batched.tables == g_single.tables
            assert (g_batched.rows == g_single.rows).all()
            assert g_batched.allocator._free == g_single.allocator._free
    assert refused > 0                                   # the pool was small enough to run out


def test_batched_extend_refuses_what_extend_refuses():
    cache = manager(pages=8, page=4, slots=3, max_len=16)
    cache.admit("a"); cache.admit("b")
    with pytest.raises(CacheError, match="only once"):
        cache.extend_many(["a", "a"], [1, 1])
    with pytest.raises(CacheError, match="positive"):
        cache.extend_many(["a", "b"], [1, 0])
    with pytest.raises(CacheError, match="unknown request"):
        cache.extend_many(["a", "zz"], [1, 1])
    with pytest.raises(CacheError, match="maximum length"):
        cache.extend_many(["a", "b"], [3, 17])
    cache.extend_many(["a", "b"], [3, 5])
    with pytest.raises(CacheError, match="not committed"):
        cache.extend_many(["b"], [1])
    cache.commit_many([])
    cache.commit_many(["a", "b"])
    assert cache.length("a") == 3 and cache.length("b") == 5
    with pytest.raises(CacheError, match="nothing to commit"):
        cache.commit_many(["a"])
    cache.check_invariants()


# ------------------------------------------------------------------ the slot store (device copy of per-request state)
def _corrections(cache):
    offsets, values = cache.slots.drain()
    return dict(zip(offsets.tolist(), values.tolist()))


def test_slot_store_queues_a_table_entry_only_when_a_page_boundary_is_crossed():
    """What a step uploads of the block tables: nothing while the new tokens stay inside the request's last
    page, one entry per group when they start a new page, and the -1s when pages go back."""
    cache = CacheManager([KVNeed(2, 16), KVNeed(2, 16)], [None, None], page_size=4, num_pages=12, max_slots=3,
                         max_model_len=32)
    store = cache.slots
    assert store.pending == 0
    slot = cache.admit("a")
    assert store.pending == 0                                   # a free slot's row is already all -1
    cache.extend("a", 3)                                        # positions 0-2: the first page
    base = store.tables[0] + slot * store.table_widths[0]
    assert _corrections(cache) == {base: cache.groups[0].tables["a"][0]}
    cache.commit("a")
    for _ in range(1):                                          # position 3: still the first page
        cache.extend("a", 1)
        assert store.pending == 0 and _corrections(cache) == {}
        cache.commit("a")
    cache.extend("a", 1)                                        # position 4 starts the second page
    assert _corrections(cache) == {base + 1: cache.groups[0].tables["a"][1]}
    cache.commit("a")
    cache.extend_many(["a"], [2])                               # positions 5, 6: inside it
    assert store.pending == 0
    cache.rollback("a")
    assert store.pending == 0                                   # nothing had been taken, nothing goes back
    cache.extend_many(["a"], [9])                               # positions 5-13: two more pages
    got = _corrections(cache)
    assert got == {base + 2: cache.groups[0].tables["a"][2], base + 3: cache.groups[0].tables["a"][3]}
    cache.rollback("a")                                         # the step failed: its pages go back on the host;
    assert cache.groups[0].rows[slot, 2:4].tolist() == [-1, -1]
    assert _corrections(cache) == {}                            # the device's stale entries lie beyond every length
    cache.extend_many(["a"], [9])                               # the same pages come back (the free list is LIFO):
    assert _corrections(cache) == {}                            # the device has them already
    cache.commit("a")
    cache.free("a")
    assert _corrections(cache) == {}                            # a free slot's row is read by nobody
    cache.check_invariants()                                    # live requests' entries equal the host's throughout


def test_slot_store_corrections_carry_the_latest_value_once():
    cache = CacheManager([KVNeed(1, 16)], [None], page_size=2, num_pages=8, max_slots=2, max_model_len=16)
    store = cache.slots
    slot = cache.admit("r")
    cache.extend("r", 2)
    first = cache.groups[0].tables["r"][0]
    cache.rollback("r")                                         # taken back before any step drained it
    other = cache.admit("s")
    cache.extend("s", 2)                                        # the page goes to another request ...
    assert cache.groups[0].tables["s"] == [first]
    cache.extend("r", 2)                                        # ... and "r" gets a different one
    page = cache.groups[0].tables["r"][0]
    assert page != first
    got = _corrections(cache)                                   # each entry once, with its latest value
    assert got == {store.tables[0] + slot * store.table_widths[0]: page,
                   store.tables[0] + other * store.table_widths[0]: first}
    # lengths and sampling parameters: queued only where the device's copy differs
    assert store.set_lengths(np.asarray([slot]), np.asarray([0])) == 0
    assert store.set_lengths(np.asarray([slot]), np.asarray([5])) == 1
    assert store.set_sampling(np.asarray([slot]), [0.0], [0]) == 0
    assert store.set_sampling(np.asarray([slot]), [0.5], [2 ** 63 + 1]) == 3
    got = _corrections(cache)                                   # the step's upload takes them ...
    assert got[store.len + slot] == 5
    store.device_advanced(np.asarray([slot]), 3)                # ... and the device moves the length on itself
    assert store.lengths_of(np.asarray([slot])).tolist() == [8]
    assert store.set_lengths(np.asarray([slot]), np.asarray([8])) == 0 and store.pending == 0
    assert np.asarray([got[store.temp + slot]], dtype=np.int32).view(np.float32)[0] == 0.5
    words = np.asarray([got[store.seed + 2 * slot], got[store.seed + 2 * slot + 1]], dtype=np.int32)
    assert int(words.view(np.uint64)[0]) == 2 ** 63 + 1
    drained = np.asarray(list(got), dtype=np.int64)
    store.requeue(drained)                                      # a step that was prepared and dropped
    assert set(_corrections(cache)) == set(got)
    assert store.take_all() is store.mirror and store.pending == 0
