"""A bounded device wait that runs out: the kernel returns an error status, nothing faults.

Every wait in the library's kernels is bounded; when one runs out the kernel records
MLC_DEVERR_WAIT_TIMEOUT in the device error word, writes no output and returns, and the context
stays usable. The only wait that depends on somebody else is the peer exchange's wait for the other
ranks' flags, so that is where a test can make a wait run out without any fault: a two-rank exchange
whose second rank never runs (a flag that nothing sets), with the poll limit lowered to about a
millisecond through mlc_ctx_set_wait_limit.
"""
import numpy as np
import pytest

from mlcompiler_b200 import synth
from mlcompiler_b200.capi import MLC_F16, MLC_F32, PeerExchange
from tests.util import DeviceCase, assert_attention_close

pytestmark = pytest.mark.gpu

MLC_ERR_DEVICE_FLAG = 8
MLC_DEVERR_WAIT_TIMEOUT = 0x1


def test_status_codes_match_header():
    import re
    from pathlib import Path
    text = (Path(__file__).resolve().parents[1] / "include" / "mlc_b200.h").read_text()
    assert int(re.search(r"MLC_ERR_DEVICE_FLAG\s*=\s*(\d+)", text).group(1)) == MLC_ERR_DEVICE_FLAG
    m = re.search(r"#define\s+MLC_DEVERR_WAIT_TIMEOUT\s+(\w+)", text)
    assert int(m.group(1).rstrip("u"), 0) == MLC_DEVERR_WAIT_TIMEOUT


def test_exchange_wait_runs_out_and_context_stays_usable(executor, oracle_mod):
    import torch
    rows, D = 33, 64            # an odd row count: the slots of the gather buffer stay 16-byte aligned
    ex0 = PeerExchange(executor, 0, 2, rows, D)
    ex1 = PeerExchange(executor, 1, 2, rows, D)    # stands for the absent rank: its kernel is never launched
    ex0.attach_pointers([0, ex1.local_buffer()])
    o_part = torch.randn((rows, D), dtype=torch.float32, device="cuda")
    ml_part = torch.rand((rows, 2), dtype=torch.float32, device="cuda")
    out = torch.full((rows, D), float("nan"), dtype=torch.float32, device="cuda")
    assert executor.setWaitLimit(1000)           # about a millisecond instead of about a second
    try:
        assert executor.beginForwardPassCB()
        assert ex0.encodeLseCombine(o_part, ml_part, rows, out, MLC_F32), executor.last_error()
        assert not executor.flushForwardPassCB()
        assert executor.last_status == MLC_ERR_DEVICE_FLAG, executor.last_error()
        assert "0x" in executor.last_error()
        word = int(executor.last_error().split("0x")[1].split()[0], 16)
        assert word & MLC_DEVERR_WAIT_TIMEOUT
        assert (word >> 16) & 0xFF == 1, "the wait that ran out was the one for rank 1's flag"
        torch.cuda.synchronize()
        assert torch.isnan(out).all(), "a step whose wait ran out must not write output"
        assert executor.deviceErrorWord() == 0, "the flush clears the error word"
    finally:
        assert executor.setWaitLimit(0)
        ex0.destroy()
        ex1.destroy()

    # the context is still good for ordinary work
    case = synth.make_case(5, [700, 64, 1, 2048, 333], **synth.SHAPE_A)
    dc = DeviceCase(case)
    o = dc.out()
    assert executor.runPagedFlashAttention(dc.q, dc.k_pool, dc.v_pool, o, case.pt_flat, case.pt_off, case.seq_lens,
                                           case.q_pos, case.N, case.H, case.KVH, case.D, case.P, True,
                                           scale=case.scale, q_dtype=MLC_F16, o_dtype=MLC_F16), executor.last_error()
    want = oracle_mod.paged_attention(case.q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                      case.seq_lens, case.q_pos, case.H, case.KVH, case.D, case.P, scale=case.scale)
    assert_attention_close(o.float().cpu().numpy(), want)


def test_fused_exchange_wait_runs_out_and_context_stays_usable(executor, oracle_mod):
    """The same with the fused attention + exchange kernel: rank 1 never runs, so the CTAs that finish a
    (request, head) wait for its flag in vain, record the timeout and skip their combine."""
    import torch
    case = synth.make_case(6, [300, 64, 1000], **synth.SHAPE_A)
    dc = DeviceCase(case)
    rows = case.N * case.H
    ex0 = PeerExchange(executor, 0, 2, rows, case.D)
    ex1 = PeerExchange(executor, 1, 2, rows, case.D)    # the absent rank
    ex0.attach_pointers([0, ex1.local_buffer()])
    plan = executor.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, case.H, case.KVH, case.D,
                               case.P, True, case.capacity)
    out = dc.out()
    assert executor.setWaitLimit(1000)
    try:
        assert executor.beginForwardPassCB()
        assert ex0.encodeAttentionExchange(plan, dc.q, dc.k_pool, dc.v_pool, out, case.scale, MLC_F16, MLC_F16), \
            executor.last_error()
        assert not executor.flushForwardPassCB()
        assert executor.last_status == MLC_ERR_DEVICE_FLAG, executor.last_error()
        word = int(executor.last_error().split("0x")[1].split()[0], 16)
        assert word & MLC_DEVERR_WAIT_TIMEOUT and (word >> 8) & 0xFF == 0x51
        torch.cuda.synchronize()
        assert torch.isnan(out.float()).all(), "no combine may have written output"
    finally:
        assert executor.setWaitLimit(0)
        ex0.destroy()
        ex1.destroy()
        plan.destroy()
    o = dc.out()
    assert executor.runPagedFlashAttention(dc.q, dc.k_pool, dc.v_pool, o, case.pt_flat, case.pt_off, case.seq_lens,
                                           case.q_pos, case.N, case.H, case.KVH, case.D, case.P, True,
                                           scale=case.scale, q_dtype=MLC_F16, o_dtype=MLC_F16), executor.last_error()
    want = oracle_mod.paged_attention(case.q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                      case.seq_lens, case.q_pos, case.H, case.KVH, case.D, case.P, scale=case.scale)
    assert_attention_close(o.float().cpu().numpy(), want)
