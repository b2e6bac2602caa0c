"""Page allocator and per-request page tables through the C ABI (no GPU).

Re-expression of the reference's portable unit tests, tests/test_paged_kv.cpp:18-207 and
597-619 (same capacities, page sizes and expected sequences), plus a differential check
against the C oracle and - where it is available - against the reference's own PagePool /
RequestKVState compiled from its sources.
"""
import ctypes as C

import numpy as np
import pytest

from mlcompiler_b200.host import PagePool, RequestKVState


def test_alloc_release_single():
    pool = PagePool(16)
    assert pool.capacity() == 16 and pool.pages_in_use() == 0 and pool.pages_free() == 16
    pid = pool.allocate()
    assert pid is not None
    assert pool.pages_in_use() == 1 and pool.pages_free() == 15
    assert pool.release(pid)
    assert pool.pages_in_use() == 0 and pool.pages_free() == 16


def test_alloc_ascending_from_fresh_pool():
    pool = PagePool(8)
    assert [pool.allocate() for _ in range(8)] == list(range(8))
    assert pool.pages_in_use() == 8


def test_exhaustion_returns_nullopt():
    pool = PagePool(2)
    assert pool.allocate() is not None and pool.allocate() is not None
    assert pool.allocate() is None
    assert pool.pages_free() == 0 and pool.pages_in_use() == 2


def test_released_page_reused_lifo():
    pool = PagePool(4)
    a, b, c, d = (pool.allocate() for _ in range(4))
    pool.release(b)
    assert pool.allocate() == b


def test_bulk_alloc_atomic():
    pool = PagePool(10)
    ids = []
    assert pool.allocate_n(7, ids)
    assert len(ids) == 7 and len(set(ids)) == 7
    assert pool.pages_in_use() == 7 and pool.pages_free() == 3
    pool = PagePool(5)
    first, second = [], []
    assert pool.allocate_n(3, first)
    assert not pool.allocate_n(3, second)      # only 2 left
    assert second == [] and pool.pages_in_use() == 3 and pool.pages_free() == 2


def test_release_of_a_bad_id_is_refused():
    pool = PagePool(4)
    assert not pool.release(0)        # nothing in use
    pid = pool.allocate()
    assert not pool.release(99)       # outside the pool
    assert pool.release(pid)


def test_empty_total_is_zero():
    assert RequestKVState(64).total_tokens() == 0


def test_reserve_allocates_enough_pages():
    pool, st = PagePool(32), RequestKVState(64)
    assert st.reserve(pool, 100)
    assert len(st.page_table) == 2 and pool.pages_in_use() == 2
    assert st.reserve(pool, 50)                # never shrinks
    assert len(st.page_table) == 2
    assert st.reserve(pool, 200)
    assert len(st.page_table) == 4 and pool.pages_in_use() == 4


def test_reserve_failure_keeps_table_unchanged():
    pool, st = PagePool(2), RequestKVState(64)
    assert not st.reserve(pool, 200)
    assert st.page_table == [] and pool.pages_in_use() == 0


def test_extend_one_token_across_page_boundary():
    pool, st = PagePool(8), RequestKVState(4)
    writes = [st.extend_one_token(pool) for _ in range(10)]
    assert all(w is not None for w in writes)
    assert st.total_tokens() == 10 and len(st.page_table) == 3 and st.tokens_in_last_page == 2
    assert [w[1] for w in writes] == [0, 1, 2, 3, 0, 1, 2, 3, 0, 1]


def test_extend_exhausts_pool():
    pool, st = PagePool(2), RequestKVState(4)
    for _ in range(8):
        assert st.extend_one_token(pool) is not None
    assert st.extend_one_token(pool) is None
    assert st.total_tokens() == 8 and len(st.page_table) == 2 and st.tokens_in_last_page == 4


def test_locate_round_trips_extension_writes():
    pool, st = PagePool(8), RequestKVState(4)
    writes = [st.extend_one_token(pool) for _ in range(10)]
    assert [st.locate(i) for i in range(10)] == writes
    assert st.locate(10) is None and st.locate(100) is None


def test_release_returns_all_pages():
    pool, st = PagePool(8), RequestKVState(4)
    for _ in range(6):
        assert st.extend_one_token(pool) is not None
    assert pool.pages_in_use() == 2
    st.release_all(pool)
    assert st.total_tokens() == 0 and st.page_table == [] and st.tokens_in_last_page == 0
    assert pool.pages_in_use() == 0 and pool.pages_free() == 8


def test_multiple_requests_share_same_pool():
    pool = PagePool(16)
    a, b = RequestKVState(4), RequestKVState(4)
    for _ in range(10):
        assert a.extend_one_token(pool) is not None
        assert b.extend_one_token(pool) is not None
    assert set(a.page_table).isdisjoint(b.page_table)
    assert pool.pages_in_use() == len(a.page_table) + len(b.page_table)
    a.release_all(pool)
    b.release_all(pool)
    assert pool.pages_in_use() == 0


def _random_script(seed, steps=400):
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(0, 3)), int(rng.integers(0, 4))) for _ in range(steps)]


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_allocator_matches_oracle_and_reference(oracle_mod, seed):
    """Same random script of extend / release operations on 4 requests: identical
    (page, slot) sequences from the product, the C oracle and the reference's classes."""
    cap, P = 12, 4
    port = oracle_mod.port()
    ref = oracle_mod.ref()
    pool = PagePool(cap)
    states = [RequestKVState(P) for _ in range(4)]
    opool = port.orc_pool_create(cap)
    ostate = [dict(pages=(C.c_uint32 * 64)(), n=C.c_size_t(0), last=C.c_uint32(0)) for _ in range(4)]
    rpool = ref.ref_pool_create(cap) if ref else None
    rstate = [ref.ref_kvstate_create(P) for _ in range(4)] if ref else None
    for op, r in _random_script(seed):
        if op < 2:   # extend
            got = states[r].extend_one_token(pool)
            pg, sl = C.c_uint32(0), C.c_uint32(0)
            ok = port.orc_kvstate_extend(opool, P, ostate[r]["pages"], C.byref(ostate[r]["n"]),
                                         C.byref(ostate[r]["last"]), C.byref(pg), C.byref(sl))
            want = (pg.value, sl.value) if ok else None
            assert got == want
            if ref:
                pg2, sl2 = C.c_uint32(0), C.c_uint32(0)
                ok2 = ref.ref_kvstate_extend(rstate[r], rpool, C.byref(pg2), C.byref(sl2))
                assert got == ((pg2.value, sl2.value) if ok2 else None)
        else:        # release everything the request holds
            states[r].release_all(pool)
            for i in range(ostate[r]["n"].value):
                port.orc_pool_release(opool, ostate[r]["pages"][i])
            ostate[r]["n"].value, ostate[r]["last"].value = 0, 0
            if ref:
                ref.ref_kvstate_release(rstate[r], rpool)
        assert pool.pages_in_use() == port.orc_pool_in_use(opool)
        if ref:
            assert pool.pages_in_use() == ref.ref_pool_in_use(rpool)
            assert states[r].total_tokens() == ref.ref_kvstate_total(rstate[r])
    port.orc_pool_destroy(opool)
    if ref:
        for s in rstate:
            ref.ref_kvstate_destroy(s)
        ref.ref_pool_destroy(rpool)
