"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; prefixes are found again."""
import os

import numpy as np
import pytest
import torch

from coheryn_ai_studio_b200.cache import CacheError, CacheManager, PagePool, SlotPool
from coheryn_ai_studio_b200.parts import FixedState, PagedKV

CPU = torch.device("cpu")


def manager(needs, pages=8, page=4, cache_from=None, **kw):
    return CacheManager(needs, cache_from or [None] * len(needs), torch.float32, CPU, page_size=page,
                        num_pages=pages, max_requests=kw.pop("max_requests", 4), **kw)


def test_pool_basics():
    p = PagePool(3)
    a = p.allocate(2)
    assert a == [0, 1] and p.available == 1 and p.allocate(2) is None and p.available == 1
    p.release(1)
    assert p.allocate(1) == [1]          # last freed, first reused
    p.release(0)
    with pytest.raises(CacheError, match="nobody holds"):
        p.release(0)
    with pytest.raises(CacheError, match="not in the pool"):
        p.release(7)
    p.check()


def test_hashed_pages_wait_and_are_evicted_last():
    p = PagePool(3)
    a, b, c = p.allocate(3)
    p.set_hash(a, b"A"); p.set_hash(b, b"B")
    p.release(a); p.release(b); p.release(c)
    assert p.available == 3 and p.lookup(b"A") == a
    p.retain(a)                                   # revived from the idle list
    assert p.refcount(a) == 1 and p.available == 2
    got = p.allocate(2)                           # the plain free page first, then the idle one
    assert got == [c, b] and p.lookup(b"B") is None
    p.check({a: 1, b: 1, c: 1})
    with pytest.raises(CacheError):
        p.check({a: 2, b: 1, c: 1})


def test_slots():
    s = SlotPool(2)
    a, b = s.allocate(), s.allocate()
    assert s.allocate() is None
    s.release(a)
    with pytest.raises(CacheError):
        s.release(a)
    s.check()


def test_groups_by_need_and_shared_cache():
    full, win = PagedKV(2, 8, None), PagedKV(2, 8, 6)
    m = manager([full, win, full, None, FixedState((3,))], cache_from=[None, None, None, 0, None])
    assert [g.entries for g in m.groups] == [[0, 2], [1]]
    assert m.groups[0].tensor.shape == (2, 2, 8 + 1, 2, 4, 8)      # 8 pages of the pool and the spare one
    assert m.spare_page == 8 and m.has_fixed_state
    lc = m.layer_caches()
    assert lc[3].kind == "paged" and not lc[3].writes and lc[3].k.data_ptr() == lc[0].k.data_ptr()
    assert lc[2].k.data_ptr() != lc[0].k.data_ptr() and lc[1].group == 1
    assert lc[4].kind == "state" and lc[4].state.shape == (4, 3)
    assert not m.prefix_reuse


def test_reserve_is_all_or_nothing_and_window_returns_pages():
    full, win = PagedKV(1, 4, None), PagedKV(1, 4, 6)
    m = manager([full, win], pages=5, page=4)
    m.admit("a")
    assert m.reserve("a", list(range(10)))        # 3 pages in both groups
    assert m.slot_ids("a", 0) == [m.block_table("a", 0)[p // 4] * 4 + p % 4 for p in range(10)]
    m.commit("a")
    # next query sits at position 10 and sees keys 5..10: block 0 (positions 0..3) is passed
    assert m.block_table("a", 1)[0] == -1 and m.block_table("a", 0)[0] >= 0
    assert m.available_pages() == [2, 3]
    m.admit("b")
    assert not m.reserve("b", list(range(9)))     # group 0 has 2 pages, 3 are needed
    assert m.available_pages() == [2, 3] and m.length("b") == 0
    assert m.reserve("b", list(range(8)))
    m.rollback("b")
    assert m.available_pages() == [2, 3]
    m.check()
    m.free("a"); m.free("b")
    assert m.available_pages() == [5, 5]
    with pytest.raises(CacheError):
        m.free("a")
    m.check()


def test_state_slot_is_zeroed_on_admission():
    m = manager([FixedState((2,))], pages=0)
    m.admit("a")
    slot = m.state_slot("a")
    m.layer_caches()[0].state[slot] += 5
    m.free("a")
    m.admit("b")
    assert m.state_slot("b") == slot and not m.layer_caches()[0].state[slot].any()
    for r in "cde":
        assert m.admit(r) is not None
    assert m.admit("f") is None                   # four slots


def test_prefix_is_found_again_and_last_token_is_recomputed():
    m = manager([PagedKV(1, 4, None)], pages=8, page=4)
    prompt = list(range(100, 112))                # three full pages
    assert m.admit("a", prompt) == 0
    m.reserve("a", prompt); m.commit("a")
    pages_a = list(m.block_table("a", 0))
    assert m.admit("b", prompt) == 8              # (12 - 1) // 4 = 2 pages: the last token is recomputed
    assert m.block_table("b", 0) == pages_a[:2] and m.groups[0].pool.refcount(pages_a[0]) == 2
    m.reserve("b", prompt[8:]); m.commit("b")
    assert m.block_table("b", 0)[2] != pages_a[2]
    m.check()
    m.free("a")
    assert m.admit("c", prompt[:8] + [7, 7, 7, 7, 7]) == 8
    m.free("b"); m.free("c")
    assert m.available_pages() == [8]
    assert m.admit("d", prompt + [1]) == 12       # idle hashed pages are still found
    assert m.admit("e", [5] + prompt) == 0
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = np.random.default_rng(seed)
    needs = [PagedKV(1, 4, None), PagedKV(1, 4, 9 if seed % 2 else None)]
    m = manager(needs, pages=12, page=4, max_requests=5)
    live, counter = {}, 0
    for _ in range(400):
        action = rng.integers(0, 4)
        if action == 0 and len(live) < 5:
            rid = f"r{counter}"; counter += 1
            prompt = rng.integers(0, 3, size=int(rng.integers(1, 20))).tolist()
            assert m.admit(rid, prompt) is not None
            live[rid] = prompt[m.length(rid):]
        elif action in (1, 2) and live:
            rid = list(live)[int(rng.integers(len(live)))]
            n = int(rng.integers(1, 9))
            toks = (live[rid][:n] + rng.integers(0, 3, size=n).tolist())[:n]
            before = m.available_pages()
            if m.reserve(rid, toks):
                if rng.random() < 0.15:
                    m.rollback(rid)
                    assert m.available_pages() == before
                else:
                    m.commit(rid)
                    live[rid] = live[rid][n:]
            else:
                assert m.available_pages() == before
        elif action == 3 and live:
            rid = list(live)[int(rng.integers(len(live)))]
            m.free(rid); del live[rid]
        m.check()
    for rid in list(live):
        m.free(rid)
    m.check()
    assert m.available_pages() == [12] * len(m.groups) and m.slots.available == 5


def test_the_pools_are_the_native_ones():
    """The books are kept by the C++ host library, not by Python containers."""
    pool = PagePool(4)
    assert pool._lib.coheryn_library_path.endswith(".so") and "host" in os.path.basename(pool._lib.coheryn_library_path)
    a = pool.allocate(3)
    pool.set_hash(a[0], b"x" * 32); pool.set_hash(a[1], b"y" * 32)
    pool.release(a[0]); pool.release(a[1])                 # idle, a[0] least recently used
    assert pool.available == 3 and pool.lookup(b"x" * 32) == a[0]
    got = pool.allocate(2)                                  # the free page first, then the LRU idle one
    assert got[1] == a[0] and pool.lookup(b"x" * 32) is None and pool.lookup(b"y" * 32) == a[1]
    pool.retain(a[1])                                       # revived by its hash
    pool.check({a[1]: 1, a[2]: 1, got[0]: 1, got[1]: 1})
    with pytest.raises(CacheError):
        pool.release(99)
    with pytest.raises(CacheError):
        pool.check({a[1]: 2, a[2]: 1, got[0]: 1, got[1]: 1})


def test_native_step_layout_equals_the_tables():
    """The native book lays a step out (position, request and slot of every reserved token, offsets,
    lengths, state slots, serials); the same numbers follow from the block tables."""
    import ctypes
    import numpy as np
    m = manager([PagedKV(1, 4, None)], pages=16, page=4)
    m.admit("a"); m.admit("b"); m.admit("c")
    assert m.reserve("a", list(range(9))); m.commit("a")
    assert m.reserve("a", [1]) and m.reserve("b", list(range(6))) and m.reserve("c", [7, 8])
    ids = ["b", "a", "c"]
    counts = [6, 1, 2]
    T = sum(counts)
    keys = (ctypes.c_char_p * 3)(*[i.encode() for i in ids])
    pos, req, slots = np.empty(T, np.int32), np.empty(T, np.int32), np.empty(T, np.int32)
    cu, kv, st, ser = np.empty(4, np.int32), np.empty(3, np.int32), np.empty(3, np.int32), np.empty(3, np.int64)
    ip = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))
    got = m._lib.coheryn_book_layout(m.book_handle, 3, keys, ip(pos), ip(req), ip(slots), T, ip(cu), ip(kv), ip(st),
                                     ser.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong)))
    assert got == T and cu.tolist() == [0, 6, 7, 9] and kv.tolist() == [6, 10, 2]
    assert pos.tolist() == [0, 1, 2, 3, 4, 5, 9, 0, 1] and req.tolist() == [0] * 6 + [1] + [2, 2]
    want = []
    for rid in ids:
        want += m.slot_ids(rid, 0)
    assert slots.tolist() == want
    for i, rid in enumerate(ids):
        table = m.block_table(rid, 0)
        for t in range(cu[i], cu[i + 1]):
            assert slots[t] == table[pos[t] // 4] * 4 + pos[t] % 4
    assert st.tolist() == [m.state_slot(r) for r in ids] and ser.tolist() == [m.serial(r) for r in ids]
    assert m._lib.coheryn_book_layout(m.book_handle, 3, keys, ip(pos), ip(req), ip(slots), T - 1, ip(cu), ip(kv), ip(st),
                                      ser.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))) == -1     # buffer too small
