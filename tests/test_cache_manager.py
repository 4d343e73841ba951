"""The cache manager on the host: pages, tables, windows, slots (no GPU)."""
import numpy as np
import pytest

from bitwise_b200.cache import FREED, CacheError, CacheManager, GroupSpec, PagePool, groups_from_needs
from bitwise_b200.parts.base import PagedKVNeed, SlotStateNeed


def test_pool_hands_out_low_ids_first_and_counts_references():
    p = PagePool(3)
    assert [p.allocate(), p.allocate(), p.allocate(), p.allocate()] == [0, 1, 2, None]  # src/block_manager.cpp:28-48
    p.fork(1)
    p.release(1)
    assert p.available() == 0 and p.refcount(1) == 1
    p.release(1)
    assert p.available() == 1 and p.allocate() == 1
    with pytest.raises(CacheError):
        p.release(0), p.release(0)  # the second release is of a page nobody holds
    with pytest.raises(CacheError):
        p.fork(0)


def test_tables_grow_page_by_page_and_keep_the_partial_gain():
    m = CacheManager([GroupSpec(None, (0, 1))], [4], 16, 2)
    m.begin("a")
    assert m.ensure("a", 17) and m.get("a").tables[0] == [0, 1]
    m.begin("b")
    assert not m.ensure("b", 16 * 3)           # needs 3, only 2 left: keeps the 2 (src/engine.cpp:146-153)
    assert m.get("b").tables[0] == [2, 3] and m.available() == 0
    m.release("b")
    assert m.available() == 2 and not m.has("b")
    with pytest.raises(CacheError):
        m.advance("a", 33)                      # more tokens than its pages hold
    m.advance("a", 32)
    m.release("a")
    assert m.all_free()


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([GroupSpec(None, (0,)), GroupSpec(20, (1,))], [8, 8], 16, 1)
    m.begin("r")
    assert m.ensure("r", 70)
    m.advance("r", 35)   # next query at >= 35 reads keys from 16 on: page 0 (keys 0..15) is passed
    assert m.get("r").tables[1][:2] == [FREED, 1] and m.available(1) == 8 - 5 + 1
    m.advance("r", 36)
    assert m.get("r").tables[1][1] == 1
    m.advance("r", 52)   # reads from 33 on: pages 0 and 1 are passed
    assert m.get("r").tables[1][:3] == [FREED, FREED, 2]
    assert m.get("r").tables[0] == [0, 1, 2, 3, 4]  # the full group keeps everything
    m.check_consistency()
    m.release("r")
    assert m.all_free()


def test_slots_and_fork():
    m = CacheManager([GroupSpec(None, (0,))], [6], 16, 2)
    a = m.begin("a")
    m.ensure("a", 40)
    m.advance("a", 40)
    b = m.fork("a", "b")
    assert a.slot != b.slot and b.tables[0] == a.tables[0] and b.length == 40
    with pytest.raises(CacheError):
        m.begin("c")        # no slot left
    m.release("a")
    assert m.available() == 3  # still held by b
    m.check_consistency()
    m.release("b")
    assert m.all_free()
    with pytest.raises(CacheError):
        m.release("b")


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_lose_nothing(seed):
    rng = np.random.default_rng(seed)
    m = CacheManager([GroupSpec(None, (0,)), GroupSpec(int(rng.integers(5, 60)), (1,))], [24, 12], 8, 5)
    live = {}
    for step in range(600):
        op = rng.integers(0, 5)
        if op == 0 and len(live) < 5:
            rid = f"r{step}"
            m.begin(rid)
            live[rid] = 0
        elif op in (1, 2) and live:
            rid = list(live)[rng.integers(len(live))]
            want = live[rid] + int(rng.integers(1, 30))
            if m.ensure(rid, want):
                m.advance(rid, want)
                live[rid] = want
        elif op == 3 and live:
            rid = list(live)[rng.integers(len(live))]
            m.release(rid)
            del live[rid]
        elif op == 4 and live and len(live) < 5:
            src = list(live)[rng.integers(len(live))]
            m.fork(src, f"f{step}")
            live[f"f{step}"] = live[src]
        m.check_consistency()
        for rid, n in live.items():
            assert m.length(rid) == n
    for rid in list(live):
        m.release(rid)
    m.check_consistency()
    assert m.all_free()


def test_groups_from_needs():
    needs = [PagedKVNeed(2, 16), PagedKVNeed(2, 16, 128), SlotStateNeed((8,)), PagedKVNeed(1, 32), PagedKVNeed(2, 16, 128)]
    assert groups_from_needs(needs) == [GroupSpec(None, (0, 3)), GroupSpec(128, (1, 4))]
