"""Page and slot allocators and the cache manager: no page lost, held twice or
freed twice, under random orders of requests (no GPU)."""
import random

import pytest

from prelude_b200.cache.manager import CacheManager
from prelude_b200.cache.pages import CacheAccountingError, OutOfPages, PageAllocator, SlotAllocator
from prelude_b200.parts.registry import KvPagesNeed, StateNeed


def test_allocator_basics():
    a = PageAllocator(4)
    p = a.allocate(3)
    assert sorted(p) == [0, 1, 2] and a.num_free == 1
    with pytest.raises(OutOfPages):
        a.allocate(2)
    assert a.num_free == 1                               # all-or-nothing
    a.incref(p[:1])
    a.free(p)
    assert a.num_free == 3 and a.refcount(p[0]) == 1     # still held once
    a.free(p[:1])
    assert a.num_free == 4
    with pytest.raises(CacheAccountingError):
        a.free(p[:1])                                    # freed twice
    with pytest.raises(CacheAccountingError):
        a.free([99])
    a.check()


def test_pages_come_back_first_in_first_out():
    a = PageAllocator(3)
    x = a.allocate(3)
    a.free([x[1]])
    a.free([x[0]])
    assert a.allocate(2) == [x[1], x[0]]


def test_slots():
    s = SlotAllocator(2)
    a, b = s.allocate(), s.allocate()
    with pytest.raises(OutOfPages):
        s.allocate()
    s.free(a)
    with pytest.raises(CacheAccountingError):
        s.free(a)
    assert s.allocate() == a
    s.check()


def _manager(num_pages=8, page=4, window=None, slots=4):
    needs = [KvPagesNeed(2, 16), KvPagesNeed(2, 16), None, KvPagesNeed(2, 16, window) if window else KvPagesNeed(2, 16)]
    return CacheManager(needs, page, num_pages, slots, device=None)


def test_groups_by_need():
    m = CacheManager([KvPagesNeed(2, 16), KvPagesNeed(2, 16, 8), KvPagesNeed(2, 16), StateNeed((3, 4)), None,
                      KvPagesNeed(4, 16)], 4, 8, 2, device=None)
    assert [g.members for g in m.groups] == [[0, 2], [1], [5]]
    assert m.layer_cache(0).group == 0 and m.layer_cache(1).group == 1 and m.layer_cache(5).group == 2
    assert m.layer_cache(3).kind == "state" and m.layer_cache(4).kind is None
    assert CacheManager.bytes_per_page([KvPagesNeed(2, 16), None, KvPagesNeed(4, 8)], 4, 2) == 2 * 4 * 2 * (2 * 16 + 4 * 8)


def test_grow_release_reuse():
    m = _manager()
    m.add_request("a")
    m.grow("a", 9)                                       # 3 pages
    assert m.requests["a"].tables[0] == [0, 1, 2] and m.free_pages() == 5
    m.grow("a", 12)                                      # still 3 pages
    assert m.free_pages() == 5
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.grow("b", 21)                                  # 6 pages, 5 free
    assert m.requests["b"].tables[0] == [] and m.free_pages() == 5      # nothing taken
    m.grow("b", 20)
    assert m.free_pages() == 0
    m.release("a")
    m.add_request("c")
    m.grow("c", 5)
    assert m.requests["c"].tables[0] == [0, 1]           # a's pages, used again
    with pytest.raises(CacheAccountingError):
        m.release("a")                                   # released twice
    with pytest.raises(CacheAccountingError):
        m.add_request("c")
    with pytest.raises(CacheAccountingError):
        m.grow("c", 2)                                   # cannot shrink
    m.check()


def test_window_pages_are_given_back_when_the_window_has_passed():
    m = CacheManager([KvPagesNeed(1, 16), KvPagesNeed(1, 16, window=6)], 4, 8, 2, device=None)
    m.add_request("a")
    m.grow("a", 16)
    assert m.trim("a") == 2                              # next query at 16 reads keys from 11 on: pages 0, 1 have passed
    assert m.requests["a"].tables[1] == [-1, -1, 2, 3] and m.requests["a"].tables[0] == [0, 1, 2, 3]
    assert m.groups[1].allocator.num_free == 6 and m.groups[0].allocator.num_free == 4
    m.grow("a", 32)                                      # four more pages in each group
    assert m.requests["a"].tables[0] == [0, 1, 2, 3, 4, 5, 6, 7]
    assert m.requests["a"].tables[1] == [-1, -1, 2, 3, 4, 5, 6, 7]
    assert m.trim("a") == 4                              # keys from 27 on: pages 0..5 have passed
    m.check()
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.grow("b", 1)                                   # the group that keeps all keys is full
    m.release("a")
    m.grow("b", 4)
    assert m.groups[1].allocator.num_free == 7
    m.check()


def test_reset_request_keeps_the_slot_and_marks_it_fresh():
    m = _manager()
    slot = m.add_request("a")
    assert m.take_fresh_slots() == [slot]
    m.grow("a", 10)
    m.reset_request("a")
    assert m.tokens_of("a") == 0 and m.free_pages() == 8 and m.take_fresh_slots() == [slot]
    m.check()


def test_every_request_holds_a_slot_even_without_state_layers():
    m = _manager(slots=2)
    m.add_request("a")
    m.add_request("b")
    assert m.slot_of("a") != m.slot_of("b")
    with pytest.raises(OutOfPages):
        m.add_request("c")
    m.release("a")
    m.add_request("c")
    m.check()


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 7])
def test_random_orders_keep_the_books(seed, window):
    rng = random.Random(seed)
    m = _manager(num_pages=24, page=4, window=window, slots=5)
    live = {}
    for step in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{step}"
            m.add_request(rid)
            live[rid] = 0
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            n = live[rid] + rng.choice([1, 1, 1, 2, 5, 9])
            try:
                m.grow(rid, n)
                live[rid] = n
                m.trim(rid)
            except OutOfPages:
                before = {g.gid: g.allocator.num_free for g in m.groups}
                assert m.tokens_of(rid) == live[rid]
                assert before == {g.gid: g.allocator.num_free for g in m.groups}
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            m.reset_request(rid)
            live[rid] = 0
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            rc = m.requests[rid]
            for g in m.groups:
                table = rc.tables[g.gid]
                assert len(table) == -(-n // 4)
                lo = 0 if g.need.window is None else max(0, n - g.need.window + 1)
                for i, p in enumerate(table):            # every position a later query can read has a page
                    if (i + 1) * 4 > lo:
                        assert p >= 0
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(g.allocator.num_free == 24 for g in m.groups) and m.slots.num_free == 5


def test_device_table_updates_write_every_cell_once_and_follow_the_host_tables():
    """The writes queued for the device-resident block tables: applied flush by flush (at random moments, so that
    requests end, start over and get their slot used again between two flushes), a mirror of the device tables
    agrees with the host tables of every live request, and no flush holds a cell twice (the scatter kernel
    writes its entries side by side, so a second entry for a cell would race with the first)."""
    import numpy as np
    rng = random.Random(7)
    page, slots, width_tokens = 4, 3, 64
    needs = [KvPagesNeed(2, 16), KvPagesNeed(2, 16, 8)]            # all keys; a window of them (pages are trimmed)
    m = CacheManager(needs, page, 40, slots, device=None, max_request_tokens=width_tokens)
    assert m.table_width == width_tokens // page and not m.device_tables
    mirror = {g.gid: np.full((slots, m.table_width), -1, np.int64) for g in m.groups}

    def flush():
        for gid, arr in m.take_table_updates().items():
            assert len(set(arr[0].tolist())) == arr.shape[1], "a cell is written twice in one flush"
            mirror[gid].reshape(-1)[arr[0]] = arr[1]
        for rc in m.requests.values():
            for gid, table in rc.tables.items():
                assert mirror[gid][rc.slot, :len(table)].tolist() == table

    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.3 and len(live) < slots:
            m.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            n = min(width_tokens, live[rid] + rng.randint(1, 9))
            m.grow(rid, n)
            live[rid] = n
            m.trim(rid)
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            m.reset_request(rid)                                       # starts over in the same slot
            live[rid] = 0
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)                                             # its slot goes to whoever comes next
            del live[rid]
        if rng.random() < 0.3:
            flush()
        m.check()
    flush()
