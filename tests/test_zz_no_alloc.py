"""The allocation-free attention entry point against the regular planned one and the oracle.

Some callers cannot allocate device memory when they call into the library - a server
whose own pool already owns the whole GPU, or a decode loop that must not pay the
device-wide synchronisation of cudaMalloc. mlc_encode_paged_flash_attention_planned_static
serves them: its split-KV scratch is a fixed array inside the library, shared by every call
on the GPU and never cleared between calls. These tests call it through the C ABI several
times in a row - the later calls find whatever the earlier ones left in the array - and check
each result against mlc_encode_paged_flash_attention_planned on the same inputs (the bits are
expected to match: same kernel, same plan) and against the CPU oracle. The file is collected
last by pytest.
"""
import os

import numpy as np
import pytest

from mlcompiler_b200 import synth
from mlcompiler_b200.capi import MLC_F16
from tests.util import MAX_ABS, DeviceCase, assert_attention_close

pytestmark = pytest.mark.gpu


CASES = [
    ("cfg2", lambda: synth.config_case(2)),
    # one request dwarfs the rest: its (request, head) units are cut over CTAs, so the partials and the
    # arrival counters in the fixed array are really used (and must be left at zero for the second call)
    ("longtail", lambda: synth.make_case(11, [12000, 300, 64, 700], 32, 4, 64)),
    ("longtail_d128", lambda: synth.make_case(12, [7000, 90], 32, 8, 128)),
]


class _Env:
    """Sets environment switches the planner reads while a plan is built."""

    def __init__(self, **kv):
        self.kv, self.prev = kv, {}

    def __enter__(self):
        for k, v in self.kv.items():
            self.prev[k] = os.environ.get(k)
            os.environ[k] = v

    def __exit__(self, *exc):
        for k, v in self.prev.items():
            if v is None:
                del os.environ[k]
            else:
                os.environ[k] = v


def _plan(ex, case):
    return ex.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH,
                         case.D, case.P, True, case.capacity)


def _oracle(oracle_mod, case, q):
    return oracle_mod.paged_attention(q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                      case.seq_lens, case.q_pos, case.H, case.KVH, case.D, case.P, scale=case.scale)


def _static_call(ex, plan, dc, out):
    case = dc.case
    assert ex.beginForwardPassCB()
    assert ex.encodePagedFlashAttentionPlannedStatic(plan, dc.q, dc.k_pool, dc.v_pool, out, case.scale,
                                                     MLC_F16, MLC_F16), ex.last_error()
    assert ex.flushForwardPassCB(), ex.last_error()


def _regular_call(ex, plan, dc, out):
    case = dc.case
    assert ex.beginForwardPassCB()
    assert ex.encodePagedFlashAttentionPlanned(plan, dc.q, dc.k_pool, dc.v_pool, out, case.scale,
                                               MLC_F16, MLC_F16), ex.last_error()
    assert ex.flushForwardPassCB(), ex.last_error()


@pytest.mark.parametrize("name,build", CASES, ids=[c[0] for c in CASES])
def test_static_scratch_matches_planned_attention_twice(executor, oracle_mod, name, build):
    import torch
    case = build()
    dc = DeviceCase(case)
    plan = _plan(executor, case)
    assert executor.staticScratchBytes() == 8 << 20
    rng = np.random.default_rng(7)
    q_host = case.q
    for call in range(2):
        if call == 1:   # fresh queries for the second call
            q_host = rng.standard_normal(case.q.shape).astype(np.float16)
            dc.q.copy_(torch.from_numpy(q_host.view(np.int16)).cuda())
        want, got = dc.out(), dc.out()
        _regular_call(executor, plan, dc, want)
        _static_call(executor, plan, dc, got)
        torch.cuda.synchronize()
        assert executor.lastAttentionKernel() == 2
        w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.isfinite(g).all()
        assert np.abs(g - w).max() <= MAX_ABS
        assert torch.equal(want, got)
        assert_attention_close(g, _oracle(oracle_mod, case, q_host))
    plan.destroy()


def test_static_scratch_survives_plans_of_different_size(executor, oracle_mod):
    """Calls of this entry point back to back, nothing else in between, with plans whose partials differ in
    size: a large one twice (both halves of the array then hold its partials), a small cut-unit one twice
    (its arrival counters must still read zero), the large one again, then the small one from a second
    context on the same GPU. Every output is compared with the oracle and, bit for bit, with the regular
    entry point's. Nothing may be allocated by any of these calls."""
    import torch
    import mlcompiler_b200
    big = synth.config_case(2)
    small = synth.make_case(11, [12000, 300, 64, 700], 32, 4, 64)
    with _Env(MLC_B200_DECODE_MODE="1"):      # the split form: ~150 request pieces, > 1 MiB of partials
        plan_big = _plan(executor, big)
    with _Env(MLC_B200_DECODE_MODE="2", MLC_B200_DECODE_UNIT_CUT_FORCE="1"):   # units cut over CTAs: counters in use
        plan_small = _plan(executor, small)
    dc_big, dc_small = DeviceCase(big), DeviceCase(small)
    want_big, want_small = dc_big.out(), dc_small.out()
    _regular_call(executor, plan_big, dc_big, want_big)
    _regular_call(executor, plan_small, dc_small, want_small)
    ref_big, ref_small = _oracle(oracle_mod, big, big.q), _oracle(oracle_mod, small, small.q)
    assert_attention_close(want_big.float().cpu().numpy(), ref_big)
    assert_attention_close(want_small.float().cpu().numpy(), ref_small)
    # one call of each kind up front: the first call on a device resolves the array's address
    _static_call(executor, plan_small, dc_small, dc_small.out())
    torch.cuda.synchronize()

    allocs_before = executor.allocCount()
    free_before = torch.cuda.mem_get_info()[0]
    sequence = [(plan_big, dc_big, want_big, ref_big)] * 2 + [(plan_small, dc_small, want_small, ref_small)] * 2 + \
               [(plan_big, dc_big, want_big, ref_big), (plan_small, dc_small, want_small, ref_small)]
    outs = [dc.out() for (_, dc, _, _) in sequence]     # torch allocates here, before the calls under test
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for (plan, dc, _, _), got in zip(sequence, outs):
        _static_call(executor, plan, dc, got)
    torch.cuda.synchronize()
    assert executor.allocCount() == allocs_before, "the allocation-free entry point allocated"
    assert torch.cuda.mem_get_info()[0] == free_before, "free device memory moved across allocation-free calls"
    for i, ((_, _, want, ref), got) in enumerate(zip(sequence, outs)):
        g = got.float().cpu().numpy()
        assert np.isfinite(g).all(), f"call {i}: rows left unwritten"
        assert torch.equal(want, got), f"call {i} differs from the regular entry point"
        assert_attention_close(g, ref)

    # a second context on the same GPU, used strictly after the first has flushed, shares the array
    other = mlcompiler_b200.Executor(0)
    try:
        with _Env(MLC_B200_DECODE_MODE="2", MLC_B200_DECODE_UNIT_CUT_FORCE="1"):
            plan_other = _plan(other, small)
        for _ in range(2):
            got = dc_small.out()
            _static_call(other, plan_other, dc_small, got)
            torch.cuda.synchronize()
            assert torch.equal(want_small, got)
        plan_other.destroy()
    finally:
        other.close()
    plan_big.destroy()
    plan_small.destroy()


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
    with _Env(MLC_B200_DECODE_MODE="1"):
        plan = _plan(executor, case)
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
