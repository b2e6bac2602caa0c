"""Fused QKV split + rotary + cast (+ scatter) kernel against the CPU restatement: bit-exact.

Reference step: MetalExecutor::encodeQkvSplitRopeCast (compiler/runtime/metal_runtime.mm:7915-8025)
followed by the two scatter_kv_paged_batched_f16 dispatches (batched_walker.cpp:299-309).
"""
import numpy as np
import pytest

import oracle
from mlcompiler_b200 import capi
from mlcompiler_b200.synth import make_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ex():
    e = capi.Executor(0)
    yield e
    e.close()


def _tables(ex, positions, rotary_dim, base=10000.0, scale=1.0):
    cos = np.zeros((len(positions), rotary_dim // 2), np.float32)
    sin = np.zeros_like(cos)
    for i, p in enumerate(positions):
        if rotary_dim:
            cos[i], sin[i] = ex.computeRotaryCoefficients(int(p), rotary_dim, base, scale)
    return cos, sin


@pytest.mark.parametrize("H,KVH,D,rd,pad", [
    (32, 4, 64, 64, 0),      # TinyLlama head shape, full rotation
    (32, 8, 128, 128, 0),    # wide GQA shape
    (8, 2, 64, 32, 0),       # partial rotary_dim: the tail of every head passes through
    (4, 4, 80, 80, 6),       # odd-ish head_dim, padded row stride
    (8, 2, 64, 0, 0),        # rotary_dim = 0: split + cast only
])
def test_split_rope_cast_is_bit_exact(ex, H, KVH, D, rd, pad):
    import torch
    rng = np.random.default_rng(H * 1000 + D + rd)
    batch = 33
    q_rows, k_rows = H * D, KVH * D
    qkv_rows = q_rows + 2 * k_rows + pad
    qkv = (rng.standard_normal((batch, qkv_rows)) * 3).astype(np.float32)
    positions = rng.integers(0, 4096, size=batch)
    cos, sin = _tables(ex, positions, rd)
    want = oracle.qkv_split_rope_cast(qkv, cos, sin, H, KVH, D, rd)
    dev = torch.device("cuda:0")
    d_qkv = torch.from_numpy(qkv).to(dev)
    d_cos = torch.from_numpy(cos if rd else np.zeros((batch, 1), np.float32)).to(dev)
    d_sin = torch.from_numpy(sin if rd else np.zeros((batch, 1), np.float32)).to(dev)
    q = torch.full((batch, q_rows), float("nan"), device=dev)
    k = torch.full((batch, k_rows), float("nan"), device=dev)
    v = torch.full((batch, k_rows), float("nan"), device=dev)
    k16 = torch.zeros((batch, k_rows), dtype=torch.int16, device=dev)
    v16 = torch.zeros((batch, k_rows), dtype=torch.int16, device=dev)
    assert ex.beginForwardPassCB()
    l0 = ex.launchCount()
    assert ex.encodeQkvSplitRopeCast(d_qkv, q, k, v, k16, v16, d_cos, d_sin, batch, H, KVH, D, qkv_rows, q_rows,
                                     k_rows, k_rows, rd), ex.last_error()
    assert ex.launchCount() - l0 == 1   # the reference encodes 7 dispatches here
    assert ex.flushForwardPassCB(), ex.last_error()
    for got, w in zip((q, k, v), want[:3]):
        assert np.array_equal(got.cpu().numpy().view(np.uint32), w.view(np.uint32))
    assert np.array_equal(k16.cpu().numpy().view(np.uint16), want[3])
    assert np.array_equal(v16.cpu().numpy().view(np.uint16), want[4])


@pytest.mark.parametrize("q_dtype", ["f32", "f16"])
def test_split_rope_scatter_writes_the_pages(ex, q_dtype):
    import torch
    H, KVH, D, P, rd = 32, 4, 64, 64, 64
    case = make_case(77, [1, 64, 65, 300, 1000, 129], H=H, KVH=KVH, D=D)
    batch = case.N
    rng = np.random.default_rng(5)
    qkv_rows = H * D + 2 * KVH * D
    qkv = rng.standard_normal((batch, qkv_rows)).astype(np.float32)
    cos, sin = _tables(ex, case.q_pos, rd)
    q_w, k_w, v_w, k16_w, v16_w = oracle.qkv_split_rope_cast(qkv, cos, sin, H, KVH, D, rd)
    kp_w = case.k_pool.view(np.uint16).copy()
    vp_w = case.v_pool.view(np.uint16).copy()
    oracle.scatter_kv_paged_batched_f16(k16_w, kp_w.reshape(-1), case.page_ids, case.slots, P, KVH, D)
    oracle.scatter_kv_paged_batched_f16(v16_w, vp_w.reshape(-1), case.page_ids, case.slots, P, KVH, D)
    dev = torch.device("cuda:0")
    kp = torch.from_numpy(case.k_pool.view(np.int16)).to(dev)
    vp = torch.from_numpy(case.v_pool.view(np.int16)).to(dev)
    d_qkv, d_cos, d_sin = (torch.from_numpy(a).to(dev) for a in (qkv, cos, sin))
    q = torch.zeros((batch, H * D), dtype=torch.float32 if q_dtype == "f32" else torch.float16, device=dev)
    plan = ex.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, batch, H, KVH, D, P, True,
                         case.capacity, page_ids=case.page_ids, slots_in_page=case.slots)
    assert ex.beginForwardPassCB()
    l0 = ex.launchCount()
    assert ex.encodeQkvSplitRopeScatterPlanned(plan, d_qkv, q, capi.MLC_F32 if q_dtype == "f32" else capi.MLC_F16,
                                               kp, vp, d_cos, d_sin, qkv_rows, rd), ex.last_error()
    assert ex.launchCount() - l0 == 1   # 7 + 2 dispatches in the reference
    assert ex.flushForwardPassCB(), ex.last_error()
    assert np.array_equal(kp.cpu().numpy().view(np.uint16), kp_w)     # every other page byte untouched
    assert np.array_equal(vp.cpu().numpy().view(np.uint16), vp_w)
    if q_dtype == "f32":
        assert np.array_equal(q.cpu().numpy().view(np.uint32), q_w.view(np.uint32))
    else:
        assert np.array_equal(q.cpu().numpy().view(np.uint16), q_w.astype(np.float16).view(np.uint16))
    plan.destroy()


@pytest.mark.parametrize("H,KVH,D,rd,hidden,lens", [
    (32, 4, 64, 64, 2048, [700 + 31 * i for i in range(32)]),      # the 1.1B shape at 32 requests
    (4, 2, 64, 32, 256, [1, 64, 65]),                              # partial rotation, a row short of a tile
    (8, 2, 128, 128, 512, [5, 200, 129, 64, 1000]),
])
def test_projection_with_rope_epilogue_equals_projection_then_kernel(ex, H, KVH, D, rd, hidden, lens):
    """mlc_encode_matmul_qkv_rope_scatter_planned against mlc_encode_matmul_quant_fused followed by
    mlc_encode_qkv_split_rope_scatter_planned: the same sums, the same rotation - equal bits in Q and in both pools."""
    import torch
    from mlcompiler_b200 import synth
    P = 64
    case = make_case(91, lens, H=H, KVH=KVH, D=D)
    batch = case.N
    rng = np.random.default_rng(hidden)
    qkv_rows = (H + 2 * KVH) * D
    w = synth.random_q4_0(rng, qkv_rows, hidden)
    x = (rng.standard_normal((batch, hidden)) * 2).astype(np.float32)
    cos, sin = _tables(ex, case.q_pos, rd)
    dev = torch.device("cuda:0")
    dw, dx, d_cos, d_sin = (torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (w, x, cos, sin))
    pools = [[torch.from_numpy(a.view(np.int16).copy()).to(dev) for a in (case.k_pool, case.v_pool)] for _ in range(2)]
    q = [torch.zeros((batch, H * D), dtype=torch.float16, device=dev) for _ in range(2)]
    qkv = torch.zeros((batch, qkv_rows), device=dev)
    plan = ex.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, batch, H, KVH, D, P, True,
                         case.capacity, page_ids=case.page_ids, slots_in_page=case.slots)
    stride = w.shape[1]
    assert ex.beginForwardPassCB()
    l0 = ex.launchCount()
    assert ex.encodeMatMulQuantFused(0, dw, dx, hidden, 0, None, batch, qkv_rows, hidden, stride, qkv), ex.last_error()
    assert ex.encodeQkvSplitRopeScatterPlanned(plan, qkv, q[0], capi.MLC_F16, pools[0][0], pools[0][1], d_cos, d_sin,
                                               qkv_rows, rd), ex.last_error()
    l1 = ex.launchCount()
    assert ex.encodeMatMulQkvRopeScatterPlanned(plan, 0, dw, dx, hidden, 0, hidden, stride, q[1], pools[1][0], pools[1][1],
                                                d_cos, d_sin, rd), ex.last_error()
    assert (l1 - l0, ex.launchCount() - l1) == (2, 1)
    assert ex.flushForwardPassCB(), ex.last_error()
    assert torch.equal(q[0], q[1]) and bool(q[0].float().abs().sum() > 0)
    assert torch.equal(pools[0][0], pools[1][0]) and torch.equal(pools[0][1], pools[1][1])
    assert not np.array_equal(pools[1][0].cpu().numpy(), case.k_pool.view(np.int16))      # rows were written
    plan.destroy()


def test_split_rope_cast_argument_rules(ex):
    import torch
    dev = torch.device("cuda:0")
    z = torch.zeros(4096, device=dev)
    assert not ex.encodeQkvSplitRopeCast(z, z, z, z, z, z, z, z, 1, 4, 2, 8, 64, 32, 16, 16, 8)  # no open pass (mm:7935)
    assert ex.beginForwardPassCB()
    assert not ex.encodeQkvSplitRopeCast(z, z, z, z, z, z, z, z, 1, 4, 2, 8, 64, 33, 16, 16, 8)  # q_rows != H * D
    assert not ex.encodeQkvSplitRopeCast(z, z, z, z, z, z, z, z, 1, 4, 2, 8, 60, 32, 16, 16, 8)  # row shorter than q+k+v
    assert not ex.encodeQkvSplitRopeCast(z, z, z, z, z, z, z, z, 1, 4, 2, 8, 64, 32, 16, 16, 10)  # rotary_dim > head_dim
    assert ex.encodeQkvSplitRopeCast(z, z[0:32], z[64:80], z[128:144], z[256:264], z[512:520], z[1024:], z[2048:], 1,
                                     4, 2, 8, 64, 32, 16, 16, 8), ex.last_error()
    assert ex.flushForwardPassCB()
