"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; groups; windows; slots (no GPU)."""
import random

import pytest

from reinfer_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from reinfer_b200.parts.base import PagedKVSpec, SlotStateSpec

FULL = PagedKVSpec(kv_heads=2, head_dim=16)
WIN = PagedKVSpec(kv_heads=2, head_dim=16, window=20)


def test_pool_conservation_and_double_free():
    p = PagePool(4)
    got = [p.alloc() for _ in range(4)]
    assert got == [0, 1, 2, 3] and p.free_count == 0
    with pytest.raises(OutOfPages):
        p.alloc()
    p.free(2)
    with pytest.raises(CacheError):
        p.free(2)
    with pytest.raises(CacheError):
        p.free(9)
    assert p.alloc() == 2                     # LIFO: the page given back last is used again first
    p.check()


def test_groups_by_need_and_one_table_per_group():
    paged = {"l0": FULL, "l1": WIN, "l2": FULL, "l3": WIN}
    cm = CacheManager(paged, {}, page_size=8, num_pages=16, max_seqs=2)
    assert [g.layers for g in cm.groups] == [("l0", "l2"), ("l1", "l3")]
    cm.admit("a")
    cm.reserve("a", 17)
    assert len(cm.table("a", 0)) == 3 and len(cm.table("a", 1)) == 3
    cm.check()


def test_reserve_is_all_or_nothing_and_release_returns_everything():
    cm = CacheManager({"l0": FULL}, {}, page_size=4, num_pages=5, max_seqs=3)
    cm.admit("a"); cm.reserve("a", 9); cm.commit("a", 9)           # 3 pages
    cm.admit("b")
    with pytest.raises(OutOfPages):
        cm.reserve("b", 12)                                         # needs 3, 2 free
    assert cm.table("b", 0) == [] and cm.free_pages() == 2
    cm.reserve("b", 8)
    assert cm.free_pages() == 0
    with pytest.raises(CacheError):
        cm.commit("b", 9)                                           # beyond what is reserved
    with pytest.raises(CacheError):
        cm.reserve("a", 3)                                          # shrinking
    cm.release("a")
    assert cm.free_pages() == 3
    with pytest.raises(CacheError):
        cm.release("a")
    cm.release("b")
    assert cm.free_pages() == 5 and cm.free_slots() == 3
    cm.check()


def test_pages_are_used_again_in_reverse_order():
    cm = CacheManager({"l0": FULL}, {}, page_size=4, num_pages=6, max_seqs=2)
    cm.admit("a"); cm.reserve("a", 12)
    first = list(cm.table("a", 0))
    cm.release("a")
    cm.admit("b"); cm.reserve("b", 12)
    assert cm.table("b", 0) == first                                # deterministic reuse
    assert cm.write_slots("b", 0, 3, 3) == [first[0] * 4 + 3, first[1] * 4 + 0, first[1] * 4 + 1]


def test_window_gives_pages_back_when_passed():
    cm = CacheManager({"l0": FULL, "l1": WIN}, {}, page_size=8, num_pages=12, max_seqs=1)
    cm.admit("a")
    for n in range(1, 70):
        cm.reserve("a", n)
        cm.commit("a", n)
        cm.check()
        t = cm.table("a", 1)
        first_needed = max(0, n - 20 + 1) // 8                      # the next token (position n) reads keys >= n-19
        assert all(p < 0 for p in t[:first_needed]) and all(p >= 0 for p in t[first_needed:])
        assert all(p >= 0 for p in cm.table("a", 0))
    assert cm.groups[1].pool.in_use <= 4 and cm.groups[0].pool.in_use == 9
    with pytest.raises(CacheError):
        cm.write_slots("a", 1, 0, 1)                                # a position whose page went back
    cm.release("a")
    assert all(g.pool.in_use == 0 for g in cm.groups)


def test_slots_and_fixed_state_specs():
    cm = CacheManager({}, {"l0": SlotStateSpec((4, 8))}, page_size=16, num_pages=1, max_seqs=2)
    assert cm.admit("a") == 0 and cm.admit("b") == 1
    with pytest.raises(OutOfPages):
        cm.admit("c")
    with pytest.raises(CacheError):
        cm.admit("a")
    cm.reserve("a", 1000)                                           # no paged group: nothing to hold
    cm.release("a")
    assert cm.admit("c") == 0
    cm.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rnd = random.Random(seed)
    cm = CacheManager({"l0": FULL, "l1": WIN, "l2": FULL}, {"l1": SlotStateSpec((3,))}, page_size=rnd.choice([4, 8, 16]),
                      num_pages=rnd.randrange(8, 40), max_seqs=4)
    live = {}
    n_ok = n_refused = 0
    for i in range(600):
        op = rnd.random()
        if op < 0.25 and cm.free_slots():
            rid = f"r{i}"
            cm.admit(rid)
            live[rid] = 0
        elif op < 0.85 and live:
            rid = rnd.choice(list(live))
            new = live[rid] + rnd.randrange(1, 40)
            before = [list(cm.table(rid, g)) for g in range(len(cm.groups))]
            free_before = [g.pool.free_count for g in cm.groups]
            try:
                cm.reserve(rid, new)
                cm.commit(rid, new)
                live[rid] = new
                n_ok += 1
            except OutOfPages:
                n_refused += 1
                assert [list(cm.table(rid, g)) for g in range(len(cm.groups))] == before
                assert [g.pool.free_count for g in cm.groups] == free_before
        elif live:
            rid = rnd.choice(list(live))
            cm.release(rid)
            del live[rid]
        cm.check()
    for rid in list(live):
        cm.release(rid)
    cm.check()
    assert all(g.pool.in_use == 0 and g.pool.allocs == g.pool.frees for g in cm.groups)
    assert cm.free_slots() == 4 and n_ok > 50


def test_snapshot_and_restore_undo_admissions_and_reservations():
    """What a failed step needs: the requests it admitted leave, the ones that were live keep what they held."""
    from reinfer_b200.cache import CacheManager
    from reinfer_b200.parts.base import PagedKVSpec
    cm = CacheManager({"a0": PagedKVSpec(2, 16), "w0": PagedKVSpec(2, 16, window=8)}, {}, 4, 12, 3)
    cm.admit("x"); cm.reserve("x", 10); cm.commit("x", 10)
    before = ([list(cm.table("x", g)) for g in range(2)], cm.free_pages(), cm.free_slots(), cm.length("x"))
    snap = cm.snapshot(["x", "y"])
    cm.admit("y"); cm.reserve("y", 7); cm.reserve("x", 19)
    assert cm.free_pages() < before[1]
    cm.restore(snap)
    cm.check()
    assert "y" not in cm
    assert ([list(cm.table("x", g)) for g in range(2)], cm.free_pages(), cm.free_slots(), cm.length("x")) == before
    cm.reserve("x", 19); cm.commit("x", 19)                 # and life goes on
    cm.release("x")
    cm.check()
    assert cm.free_pages() == 12 and cm.free_slots() == 3
