"""GPU parity (bit-exact) of the paged KV writers/readers against the CPU oracle.

Patterns and shapes follow tests/test_paged_kv.cpp:219-595 of the reference:
page*100000 + slot*1000 + head*10 + dim storage pattern, scatter->gather round trips
with out-of-order page tables {5,1} / {7,2,11} / {3,0,6}, start_slot 3, fp32 and fp16.
"""
import numpy as np
import pytest

from mlcompiler_b200 import synth

pytestmark = pytest.mark.gpu


def dev(a):
    import torch
    a = np.ascontiguousarray(a)
    view = {2: np.int16, 4: np.int32}[a.dtype.itemsize]
    return torch.from_numpy(a.view(view)).cuda()


def host(t, dtype):
    return t.cpu().numpy().view(dtype)


def paged_pattern(capacity, P, KVH, D):
    p, s, h, d = np.meshgrid(np.arange(capacity), np.arange(P), np.arange(KVH), np.arange(D), indexing="ij")
    return (p * 100000.0 + s * 1000.0 + h * 10.0 + d).astype(np.float32)


def proj_pattern(KVH, tokens, D, scale=1.0):
    kv, t, d = np.meshgrid(np.arange(KVH), np.arange(tokens), np.arange(D), indexing="ij")
    return (scale * (kv * 1000.0 + t * 10.0 + d)).astype(np.float32)


def test_gather_f32_pattern(executor, oracle_mod):
    import torch
    cap, P, KVH, D = 16, 8, 4, 16
    ref = paged_pattern(cap, P, KVH, D)
    table, n = [7, 2, 11], 20
    dst = torch.zeros(KVH * n * D, dtype=torch.int32, device="cuda")
    assert executor.gatherKVPages(dev(ref), table, P, KVH, D, n, dst, 4, capacity_pages=cap)
    got = host(dst, np.float32).reshape(KVH, n, D)
    want = oracle_mod.gather_kv_pages(ref, table, P, KVH, D, n)
    assert np.array_equal(got, want)
    # the closed form the reference test checks (tests/test_paged_kv.cpp:246-267)
    for t in (0, 7, 8, 19):
        assert got[2, t, 5] == table[t // P] * 100000.0 + (t % P) * 1000.0 + 2 * 10.0 + 5


def test_gather_f16_pattern(executor, oracle_mod):
    import torch
    cap, P, KVH, D = 8, 8, 4, 16
    ref = (paged_pattern(cap, P, KVH, D) * 1e-3).astype(np.float16)
    table, n = [3, 0, 6], 17
    dst = torch.zeros(KVH * n * D, dtype=torch.int16, device="cuda")
    assert executor.gatherKVPages(dev(ref), table, P, KVH, D, n, dst, 2, capacity_pages=cap)
    want = oracle_mod.gather_kv_pages(ref.view(np.uint16), table, P, KVH, D, n)
    assert np.array_equal(host(dst, np.uint16).reshape(KVH, n, D), want)


@pytest.mark.parametrize("dtype,tokens,start,table", [(np.float32, 11, 3, [5, 1]), (np.float16, 7, 0, [2]),
                                                       (np.float16, 40, 5, [4, 0, 7, 3, 6, 1])])
def test_scatter_round_trip_with_gather(executor, oracle_mod, dtype, tokens, start, table):
    import torch
    cap, P, KVH, D = 8, 8, 4, 16
    item = np.dtype(dtype).itemsize
    tdt = torch.int32 if item == 4 else torch.int16
    udt = np.uint32 if item == 4 else np.uint16
    src = proj_pattern(KVH, tokens, D, 1.0 if item == 4 else 1e-3).astype(dtype)
    storage = torch.zeros(cap * P * KVH * D, dtype=tdt, device="cuda")
    assert executor.scatterKVPaged(storage, table, P, KVH, D, tokens, start, dev(src), item, capacity_pages=cap)
    want_pool = np.zeros(cap * P * KVH * D, udt)
    oracle_mod.scatter_kv_paged(src.view(udt), want_pool, table, P, KVH, D, tokens, start)
    assert np.array_equal(host(storage, udt), want_pool)
    n = len(table) * P
    dst = torch.zeros(KVH * n * D, dtype=tdt, device="cuda")
    assert executor.gatherKVPages(storage, table, P, KVH, D, n, dst, item, capacity_pages=cap)
    got = host(dst, dtype).reshape(KVH, n, D)
    expect = np.zeros((KVH, n, D), dtype)
    expect[:, start:start + tokens, :] = src  # slots before start_slot stay zero (test_paged_kv.cpp:449-467)
    assert np.array_equal(got, expect)


def test_scatter_rejects_bad_args(executor):
    """tests/test_paged_kv.cpp:541-595."""
    import torch
    a = torch.zeros(256, dtype=torch.int32, device="cuda")
    b = torch.zeros(256, dtype=torch.int32, device="cuda")
    assert not executor.scatterKVPaged(a, [0], 8, 4, 16, 1, 8, b, 4)     # start_slot out of range
    assert not executor.scatterKVPaged(a, [0], 8, 4, 16, 12, 3, b, 4)    # page table too short
    assert not executor.scatterKVPaged(a, [0], 8, 4, 16, 4, 0, b, 8)     # bad dtype
    assert not executor.gatherKVPages(a, [0], 8, 4, 16, 20, b, 4)        # oversized request
    assert not executor.scatterKVPaged(None, [0], 8, 4, 16, 4, 0, b, 4)
    assert not executor.scatterKVPaged(a, [0], 8, 4, 16, 0, 0, b, 4)     # tokens == 0


@pytest.mark.parametrize("shape", [synth.SHAPE_A, synth.SHAPE_B, dict(H=6, KVH=3, D=20)])
@pytest.mark.parametrize("encode", [False, True])
def test_scatter_batched_bit_exact(executor, oracle_mod, shape, encode):
    """scatter_kv_paged_batched_f16 (metal_runtime.mm:405-424): one row per request."""
    import torch
    lens = [1, 64, 65, 700, 2048, 129, 33, 512]
    case = synth.make_case(21, lens, P=64, **shape)
    pool = dev(case.k_pool)
    src = dev(case.k_new)
    args = (pool, case.page_ids, case.slots, case.P, case.KVH, case.D, case.N, src)
    if encode:
        assert executor.beginForwardPassCB()
        assert executor.encodeScatterKVPagedBatched(*args, capacity_pages=case.capacity)
        assert executor.flushForwardPassCB()
    else:
        assert executor.scatterKVPagedBatched(*args, capacity_pages=case.capacity)
    torch.cuda.synchronize()
    want = case.k_pool.view(np.uint16).copy().reshape(-1)
    oracle_mod.scatter_kv_paged_batched_f16(case.k_new, want, case.page_ids, case.slots, case.P, case.KVH, case.D)
    got = host(pool, np.uint16).reshape(-1)
    assert np.array_equal(got, want)
    assert (got != case.k_pool.view(np.uint16).reshape(-1)).sum() > 0


def test_scatter_pair_bit_exact(executor, oracle_mod):
    import torch
    case = synth.config_case(2)
    kp, vp = dev(case.k_pool), dev(case.v_pool)
    assert executor.beginForwardPassCB()
    assert executor.encodeScatterKVPairPagedBatched(kp, vp, case.page_ids, case.slots, case.P, case.KVH, case.D,
                                                    case.N, dev(case.k_new), dev(case.v_new),
                                                    capacity_pages=case.capacity)
    assert executor.flushForwardPassCB()
    torch.cuda.synchronize()
    for pool, new, orig in ((kp, case.k_new, case.k_pool), (vp, case.v_new, case.v_pool)):
        want = orig.view(np.uint16).copy().reshape(-1)
        oracle_mod.scatter_kv_paged_batched_f16(new, want, case.page_ids, case.slots, case.P, case.KVH, case.D)
        assert np.array_equal(host(pool, np.uint16).reshape(-1), want)


def test_scatter_batched_rejects(executor):
    """metal_runtime.mm:7240-7243 plus bounds checks."""
    import torch
    pool = torch.zeros(4 * 8 * 4 * 16, dtype=torch.int16, device="cuda")
    src = torch.zeros(2 * 4 * 16, dtype=torch.int16, device="cuda")
    assert executor.scatterKVPagedBatched(pool, [0, 1], [0, 7], 8, 4, 16, 2, src, capacity_pages=4)
    assert not executor.scatterKVPagedBatched(pool, [0], [0, 7], 8, 4, 16, 2, src)        # size mismatch
    assert not executor.scatterKVPagedBatched(None, [0, 1], [0, 7], 8, 4, 16, 2, src)
    assert not executor.scatterKVPagedBatched(pool, [0, 1], [0, 7], 0, 4, 16, 2, src)
    assert not executor.scatterKVPagedBatched(pool, [0, 4], [0, 7], 8, 4, 16, 2, src, capacity_pages=4)
    assert executor.last_status == 4
    assert not executor.scatterKVPagedBatched(pool, [0, 1], [0, 8], 8, 4, 16, 2, src, capacity_pages=4)
    assert not executor.encodeScatterKVPagedBatched(pool, [0, 1], [0, 7], 8, 4, 16, 2, src)  # no open pass
    assert executor.last_status == 2


def test_scatter_then_attention_order(executor, oracle_mod):
    """One decode step: the new row must be visible to attention (batched_walker.cpp:299-331)."""
    import torch
    from mlcompiler_b200.capi import MLC_F16
    from tests.util import DeviceCase, assert_attention_close
    case = synth.config_case(1)
    dc = DeviceCase(case)
    o = dc.out()
    assert executor.beginForwardPassCB()
    assert executor.encodeScatterKVPairPagedBatched(dc.k_pool, dc.v_pool, case.page_ids, case.slots, case.P,
                                                    case.KVH, case.D, case.N, dc.k_new, dc.v_new,
                                                    capacity_pages=case.capacity)
    assert executor.encodePagedFlashAttention(dc.q, dc.k_pool, dc.v_pool, o, case.pt_flat, case.pt_off,
                                              case.seq_lens, case.q_pos, case.N, case.H, case.KVH, case.D, case.P,
                                              True, scale=case.scale, q_dtype=MLC_F16, o_dtype=MLC_F16,
                                              capacity_pages=case.capacity)
    assert executor.flushForwardPassCB(), executor.last_error()
    kp = case.k_pool.view(np.uint16).copy().reshape(-1)
    vp = case.v_pool.view(np.uint16).copy().reshape(-1)
    oracle_mod.scatter_kv_paged_batched_f16(case.k_new, kp, case.page_ids, case.slots, case.P, case.KVH, case.D)
    oracle_mod.scatter_kv_paged_batched_f16(case.v_new, vp, case.page_ids, case.slots, case.P, case.KVH, case.D)
    want = oracle_mod.paged_attention(case.q.astype(np.float32), kp, vp, case.pt_flat, case.pt_off, case.seq_lens,
                                      case.q_pos, case.H, case.KVH, case.D, case.P, scale=case.scale)
    assert_attention_close(o.float().cpu().numpy(), want)
