"""The allocation-free attention entry point against the regular planned one.

Some callers cannot allocate device memory when they call into the library - a server
whose own pool already owns the whole GPU, or a decode loop that must not pay the
device-wide synchronisation of cudaMalloc. mlc_encode_paged_flash_attention_planned_static
serves them: its split-KV scratch is a fixed array inside the library. This test calls it
through the C ABI twice in a row (the second call reuses the array with whatever the first
left in it) and checks each result against mlc_encode_paged_flash_attention_planned on the
same inputs, within the attention parity tolerance (in fact the bits are expected to match:
same kernel, same plan). It lives in a file of its own that pytest collects last.
"""
import numpy as np
import pytest

from mlcompiler_b200 import synth
from mlcompiler_b200.capi import MLC_F16
from tests.util import MAX_ABS, DeviceCase

pytestmark = pytest.mark.gpu


CASES = [
    ("cfg2", lambda: synth.config_case(2)),
    # one request dwarfs the rest: its (request, head) units are cut over CTAs, so the partials and the
    # arrival counters in the fixed array are really used (and must be left at zero for the second call)
    ("longtail", lambda: synth.make_case(11, [12000, 300, 64, 700], 32, 4, 64)),
    ("longtail_d128", lambda: synth.make_case(12, [7000, 90], 32, 8, 128)),
]


@pytest.mark.parametrize("name,build", CASES, ids=[c[0] for c in CASES])
def test_static_scratch_matches_planned_attention_twice(executor, name, build):
    import torch
    case = build()
    dc = DeviceCase(case)
    plan = executor.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH,
                               case.D, case.P, True, case.capacity)
    assert executor.staticScratchBytes() == 8 << 20
    rng = np.random.default_rng(7)
    for call in range(2):
        if call == 1:   # fresh queries for the second call
            dc.q.copy_(torch.from_numpy(rng.standard_normal(case.q.shape).astype(np.float16).view(np.int16)).cuda())
        want, got = dc.out(), dc.out()
        assert executor.beginForwardPassCB()
        assert executor.encodePagedFlashAttentionPlanned(plan, dc.q, dc.k_pool, dc.v_pool, want, case.scale,
                                                         MLC_F16, MLC_F16), executor.last_error()
        assert executor.flushForwardPassCB(), executor.last_error()
        assert executor.beginForwardPassCB()
        assert executor.encodePagedFlashAttentionPlannedStatic(plan, dc.q, dc.k_pool, dc.v_pool, got, case.scale,
                                                               MLC_F16, MLC_F16), executor.last_error()
        assert executor.flushForwardPassCB(), executor.last_error()
        torch.cuda.synchronize()
        assert executor.lastAttentionKernel() == 2
        w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.isfinite(g).all()
        assert np.abs(g - w).max() <= MAX_ABS
        assert torch.equal(want, got)
    plan.destroy()


def test_static_scratch_rejects_oversized_batches(executor):
    """More split pieces than the fixed array holds: a clear error, nothing launched."""
    import torch
    # ~150 requests get cut at CTA boundaries; with 16 query heads per KV head at head_dim 128
    # every piece's partial is 32 KiB, so the batch needs ~9 MiB: more than a 4 MiB half
    lens = np.full(600, 96, np.uint32)
    case = synth.make_case(3, lens, 32, 2, 128, fill=False)
    dev = torch.device("cuda")
    pool = torch.zeros((case.capacity, case.P, case.KVH, case.D), dtype=torch.float16, device=dev)
    q = torch.zeros((case.N, case.H, case.D), dtype=torch.float16, device=dev)
    o = torch.zeros_like(q)
    # the split decomposition is the one that needs scratch (the planner's other form keeps every
    # request inside one CTA and needs none): ask for it while this plan is built
    import os
    prev = os.environ.get("MLC_B200_DECODE_MODE")
    os.environ["MLC_B200_DECODE_MODE"] = "1"
    try:
        plan = executor.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH,
                                   case.D, case.P, True, case.capacity)
    finally:
        if prev is None:
            del os.environ["MLC_B200_DECODE_MODE"]
        else:
            os.environ["MLC_B200_DECODE_MODE"] = prev
    assert executor.beginForwardPassCB()
    before = executor.launchCount()
    ok = executor.encodePagedFlashAttentionPlannedStatic(plan, q, pool, pool, o, case.scale, MLC_F16, MLC_F16)
    assert not ok
    assert executor.last_status == 5 and "scratch" in executor.last_error()
    assert executor.launchCount() == before
    # the regular entry point takes the same batch
    assert executor.encodePagedFlashAttentionPlanned(plan, q, pool, pool, o, case.scale, MLC_F16, MLC_F16)
    assert executor.flushForwardPassCB(), executor.last_error()
    plan.destroy()
