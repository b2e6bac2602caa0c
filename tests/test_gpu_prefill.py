"""Chunked causal paged attention (tcgen05 kernel and the any-shape route) against the oracle.

The oracle's orc_paged_prefill restates the reference's definition of multi-token attention
(compiler/runtime/operator_backend.cpp:906-968: query i at position q_start + i, mask
kv_pos > q_pos) over paged fp16 K/V. Tolerance: the attention parity bar of tests/util.py
(max-abs 2e-3, per-row cosine 0.99999) - fp16 operands and fp16 P on the tensor cores,
fp32 accumulation.
"""
import numpy as np
import pytest

import oracle
from mlcompiler_b200 import capi
from mlcompiler_b200.synth import make_case
from tests.util import assert_attention_close

pytestmark = pytest.mark.gpu


def _run(ex, case, q_start, q_len, q, dtype="f16"):
    import torch
    dev = torch.device("cuda:0")
    kp = torch.from_numpy(case.k_pool.view(np.int16)).to(dev)
    vp = torch.from_numpy(case.v_pool.view(np.int16)).to(dev)
    if dtype == "f16":
        qd = torch.from_numpy(q.view(np.int16)).to(dev)
        o = torch.full(q.shape, float("nan"), dtype=torch.float16, device=dev)
        dt = capi.MLC_F16
    else:
        qd = torch.from_numpy(q.astype(np.float32)).to(dev)
        o = torch.full(q.shape, float("nan"), dtype=torch.float32, device=dev)
        dt = capi.MLC_F32
    ok = ex.runPagedPrefillAttention(qd, kp, vp, o, case.pt_flat, case.pt_off, case.seq_lens, q_start, q_len,
                                     case.N, case.H, case.KVH, case.D, case.P, case.scale, dt, dt, case.capacity)
    assert ok, ex.last_error()
    torch.cuda.synchronize()
    return o.float().cpu().numpy()


def _want(case, q_start, q_len, q):
    return oracle.paged_prefill(q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                case.seq_lens, q_start, q_len, case.H, case.KVH, case.D, case.P, case.scale)


def _make(seed, seq_lens, q_len, H, KVH, D, q_start=None):
    case = make_case(seed, seq_lens, H=H, KVH=KVH, D=D)
    q_len = np.asarray(q_len, np.uint32)
    if q_start is None:
        q_start = (case.seq_lens - q_len).astype(np.uint32)
    q_start = np.asarray(q_start, np.uint32)
    rng = np.random.default_rng(seed + 1)
    q = rng.standard_normal((int(q_len.sum()), H, D), dtype=np.float32).astype(np.float16)
    return case, q_start, q_len, q


@pytest.fixture(scope="module")
def ex():
    e = capi.Executor(0)
    yield e
    e.close()


@pytest.mark.parametrize("seq,qn", [
    ([64], [64]),            # one page, pure causal
    ([128], [128]),          # one full query tile, two pages
    ([256], [64]),           # cached prefix + chunk
    ([200], [100]),          # ragged: partial last page, partial query tile
    ([700, 333], [300, 333]),  # several query tiles, two requests
    ([130, 64, 1000], [1, 64, 129]),  # single-token chunk, full chunk, tile + 1
])
def test_tcgen05_prefill_matches_oracle(ex, seq, qn):
    case, qs, ql, q = _make(11, seq, qn, H=8, KVH=2, D=128)
    got = _run(ex, case, qs, ql, q)
    assert ex.lastAttentionKernel() == 3
    assert_attention_close(got, _want(case, qs, ql, q))


def test_tcgen05_prefill_mid_sequence_chunk(ex):
    # the chunk is not the end of the sequence: later tokens exist in the pages and must be masked
    case, qs, ql, q = _make(12, [512, 300], [128, 100], H=8, KVH=8, D=128, q_start=[100, 0])
    got = _run(ex, case, qs, ql, q)
    assert ex.lastAttentionKernel() == 3
    assert_attention_close(got, _want(case, qs, ql, q))


def test_tcgen05_prefill_zero_length_request(ex):
    case, qs, ql, q = _make(13, [256, 192, 64], [64, 0, 64], H=4, KVH=1, D=128)
    got = _run(ex, case, qs, ql, q)
    assert_attention_close(got, _want(case, qs, ql, q))


def test_tcgen05_prefill_ignores_garbage_past_the_sequence(ex):
    # NaN in the unused tail of the last page must not leak (the kernel zeroes those V rows)
    case, qs, ql, q = _make(14, [100], [100], H=4, KVH=2, D=128)
    last = case.pt_flat[case.pt_off[0] + 1]
    case.k_pool[last, 36:] = np.float16(np.nan)
    case.v_pool[last, 36:] = np.float16(np.nan)
    got = _run(ex, case, qs, ql, q)
    assert_attention_close(got, _want(case, qs, ql, q))  # the oracle never reads past seq_len


def test_tcgen05_prefill_config5_shape_sample(ex):
    # the benchmark's head shape (H32 / KVH8 / D128) with cached prefixes, at a size the oracle
    # finishes in seconds
    case, qs, ql, q = _make(15, [2048, 1100], [256, 128], H=32, KVH=8, D=128)
    got = _run(ex, case, qs, ql, q)
    assert ex.lastAttentionKernel() == 3
    want = _want(case, qs, ql, q)
    assert_attention_close(got, want)


@pytest.mark.parametrize("H,KVH,D,dtype", [(8, 2, 64, "f16"), (4, 4, 80, "f32"), (8, 2, 128, "f32")])
def test_prefill_other_shapes_use_the_any_shape_kernel(ex, H, KVH, D, dtype):
    case, qs, ql, q = _make(16, [150, 64], [70, 64], H=H, KVH=KVH, D=D)
    got = _run(ex, case, qs, ql, q, dtype=dtype)
    assert ex.lastAttentionKernel() == 1
    assert_attention_close(got, _want(case, qs, ql, q))


def test_prefill_equals_token_by_token_decode(ex):
    """The reference's own definition: a paged prefill is q_len decode passes
    (compiler/runtime/batched_executor.cpp:450-467)."""
    import torch
    case, qs, ql, q = _make(17, [300], [140], H=8, KVH=2, D=128)
    got = _run(ex, case, qs, ql, q)
    dev = torch.device("cuda:0")
    kp = torch.from_numpy(case.k_pool.view(np.int16)).to(dev)
    vp = torch.from_numpy(case.v_pool.view(np.int16)).to(dev)
    for i in (0, 1, 63, 64, 127, 128, 139):
        qi = torch.from_numpy(q[i:i + 1].view(np.int16)).to(dev)
        o = torch.zeros((1, 8, 128), dtype=torch.float16, device=dev)
        pos = int(qs[0]) + i
        ok = ex.runPagedFlashAttention(qi, kp, vp, o, case.pt_flat, case.pt_off, np.array([pos + 1], np.uint32),
                                       np.array([pos], np.uint32), 1, 8, 2, 128, 64, True, case.scale,
                                       capi.MLC_F16, capi.MLC_F16, case.capacity)
        assert ok, ex.last_error()
        torch.cuda.synchronize()
        assert_attention_close(got[i:i + 1], o.float().cpu().numpy())


def test_prefill_rejects_chunk_past_the_sequence(ex):
    import torch
    case, qs, ql, q = _make(18, [128], [64], H=4, KVH=2, D=128)
    dev = torch.device("cuda:0")
    z = torch.zeros(q.shape, dtype=torch.float16, device=dev)
    kp = torch.from_numpy(case.k_pool.view(np.int16)).to(dev)
    ok = ex.runPagedPrefillAttention(z, kp, kp, z, case.pt_flat, case.pt_off, case.seq_lens,
                                     np.array([100], np.uint32), ql, 1, 4, 2, 128, 64, case.scale,
                                     capi.MLC_F16, capi.MLC_F16, case.capacity)
    assert not ok
    assert "exceeds" in ex.last_error()


def test_prefill_many_back_to_back_launches(ex):
    """Several waves of CTAs per launch and launches queued back to back: the softmax warps get
    a page ahead of the MMA warp here, which a single-phase P barrier once turned into a
    lost wake-up (reported as MLC_DEVERR_WAIT_TIMEOUT, not a hang)."""
    import torch
    H, KVH, D, P = 32, 8, 128, 64
    case = make_case(19, [2048] * 8, H=H, KVH=KVH, D=D, fill=False)
    dev = torch.device("cuda:0")
    kp = torch.randn((case.capacity, P, KVH, D), device=dev, dtype=torch.float16)
    vp = torch.randn((case.capacity, P, KVH, D), device=dev, dtype=torch.float16)
    q = torch.randn((8 * 512, H, D), device=dev, dtype=torch.float16)
    o = torch.zeros_like(q)
    qs, ql = np.full(8, 1536, np.uint32), np.full(8, 512, np.uint32)
    torch.cuda.synchronize()
    for _ in range(4):
        assert ex.beginForwardPassCB()
        for _ in range(25):
            assert ex.encodePagedPrefillAttention(q, kp, vp, o, case.pt_flat, case.pt_off, case.seq_lens, qs, ql,
                                                  8, H, KVH, D, P, case.scale, capi.MLC_F16, capi.MLC_F16,
                                                  case.capacity), ex.last_error()
        assert ex.flushForwardPassCB(), ex.last_error()
    assert torch.isfinite(o.float()).all()
