"""Two ranks on two GPUs over NCCL: sequence-sharded attention (partials, all-gather,
combine) equals attention over the whole sequence; request-sharded ranks are independent.
Skipped on a box with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

H, KVH, D, P = 32, 4, 64, 64


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case():
    from mlcompiler_b200 import synth
    return synth.make_case(91, [64 * 9 + 5, 64 * 4, 3, 64 * 20 + 1], H, KVH, D, P=P)


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from mlcompiler_b200 import Executor, sharding
    from mlcompiler_b200.capi import MLC_F16, MLC_F32
    case = _case()
    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream(device=dev)
    ex = Executor(rank, stream=stream.cuda_stream)
    flat, off, lens, _ = sharding.slice_tables_for_rank(case.pt_flat, case.pt_off, case.seq_lens, P, rank, world)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev)
    q, kp, vp = up(case.q), up(case.k_pool), up(case.v_pool)       # every rank holds the pool; it reads its slice only
    o_part = torch.zeros((case.N, H, D), dtype=torch.float32, device=dev)
    ml_part = torch.zeros((case.N, H, 2), dtype=torch.float32, device=dev)
    out = torch.zeros((case.N, H, D), dtype=torch.float32, device=dev)
    plan = ex.createPlan(flat, off, lens, np.zeros(case.N, np.uint32), case.N, H, KVH, D, P, False, case.capacity)
    assert ex.beginForwardPassCB()
    assert ex.encodePagedAttentionPartialPlanned(plan, q, kp, vp, o_part, ml_part, case.scale, MLC_F16), ex.last_error()
    with torch.cuda.stream(stream):
        o_all, ml_all = sharding.gather_partials(o_part, ml_part)
    assert ex.encodeLseCombine(o_all, ml_all, world, case.N * H, D, out, MLC_F32), ex.last_error()
    assert ex.flushForwardPassCB(), ex.last_error()
    np.save(os.path.join(out_dir, f"rank{rank}.npy"), out.cpu().numpy())
    dist.barrier()
    plan.destroy()
    ex.close()
    dist.destroy_process_group()


def _exchange_worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # host channel for the 64-byte handles only
    from mlcompiler_b200 import Executor, sharding
    from mlcompiler_b200.capi import MLC_F16, MLC_F32, PeerExchange
    case = _case()
    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream(device=dev)
    ex = Executor(rank, stream=stream.cuda_stream)
    flat, off, lens, _ = sharding.slice_tables_for_rank(case.pt_flat, case.pt_off, case.seq_lens, P, rank, world)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev)
    q, kp, vp = up(case.q), up(case.k_pool), up(case.v_pool)
    o_part = torch.zeros((case.N, H, D), dtype=torch.float32, device=dev)
    ml_part = torch.zeros((case.N, H, 2), dtype=torch.float32, device=dev)
    out = torch.zeros((case.N, H, D), dtype=torch.float32, device=dev)
    plan = ex.createPlan(flat, off, lens, np.zeros(case.N, np.uint32), case.N, H, KVH, D, P, False, case.capacity)
    xc = PeerExchange(ex, rank, world, case.N * H, D)
    xc.attach_with_torch_distributed()
    outs = []
    for step in range(5):   # several steps: both parities of the double buffer, and their reuse
        assert ex.beginForwardPassCB()
        assert ex.encodePagedAttentionPartialPlanned(plan, q, kp, vp, o_part, ml_part, case.scale, MLC_F16), ex.last_error()
        assert xc.encodeLseCombine(o_part, ml_part, case.N * H, out, MLC_F32), ex.last_error()
        assert ex.flushForwardPassCB(), ex.last_error()
        outs.append(out.cpu().numpy().copy())
        out.zero_()
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])
    np.save(os.path.join(out_dir, f"xrank{rank}.npy"), outs[0])
    dist.barrier()          # nobody frees its buffer while a peer may still push into it
    xc.destroy()
    plan.destroy()
    ex.close()
    dist.destroy_process_group()


def _fused_worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # host channel for the 64-byte handles only
    from mlcompiler_b200 import Executor, sharding
    from mlcompiler_b200.capi import MLC_F16, MLC_F32, PeerExchange
    case = _case()
    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream(device=dev)
    ex = Executor(rank, stream=stream.cuda_stream)
    flat, off, lens, _ = sharding.slice_tables_for_rank(case.pt_flat, case.pt_off, case.seq_lens, P, rank, world)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev)
    q, kp, vp = up(case.q), up(case.k_pool), up(case.v_pool)
    out = torch.zeros((case.N, H, D), dtype=torch.float32, device=dev)
    xc = PeerExchange(ex, rank, world, case.N * H, D)
    xc.attach_with_torch_distributed()
    results = {}
    for form, env in (("planner", {}), ("cut", {"MLC_B200_DECODE_MODE": "2", "MLC_B200_DECODE_UNIT_CUT_FORCE": "1"}),
                      ("split", {"MLC_B200_DECODE_MODE": "1"})):
        os.environ.update(env)
        plan = ex.createPlan(flat, off, lens, np.zeros(case.N, np.uint32), case.N, H, KVH, D, P, False, case.capacity)
        for k in env:
            del os.environ[k]
        outs = []
        for step in range(4):   # several steps: both parities of the double buffer, and their reuse
            assert ex.beginForwardPassCB()
            before = ex.launchCount()
            assert xc.encodeAttentionExchange(plan, q, kp, vp, out, case.scale, MLC_F16, MLC_F32), ex.last_error()
            launches = ex.launchCount() - before
            assert ex.flushForwardPassCB(), ex.last_error()
            outs.append(out.cpu().numpy().copy())
            out.fill_(float("nan"))
        assert launches == (1 if form != "split" else 3), (form, launches)   # the split form falls back to partial + merge + exchange
        for o in outs[1:]:
            assert np.array_equal(o, outs[0])
        results[form] = outs[0]
        dist.barrier()
        plan.destroy()
    np.savez(os.path.join(out_dir, f"frank{rank}.npz"), **results)
    dist.barrier()          # nobody frees its buffer while a peer may still push into it
    xc.destroy()
    ex.close()
    dist.destroy_process_group()


def test_fused_attention_and_exchange_on_two_gpus(oracle_mod, tmp_path):
    """One launch per step and rank: partial attention over the rank's slice, rows pushed to the peer as each
    (request, head) finishes, flags, combine - with whole units, units cut over CTAs, and the fall-back for
    the split form. Request 2 has 3 tokens, so the second rank holds none of it (rows that weigh nothing)."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tests.util import assert_attention_close
    world = 2
    mp.spawn(_fused_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    case = _case()
    whole = oracle_mod.paged_attention(case.q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                       case.seq_lens, np.zeros(case.N, np.uint32), H, KVH, D, P, causal=False,
                                       scale=case.scale)
    for rank in range(world):
        got = np.load(tmp_path / f"frank{rank}.npz")
        for form in ("planner", "cut", "split"):
            assert_attention_close(got[form], whole)


FUSED_CASES = [
    ("ragged", [64 * 9 + 5, 64 * 4, 3, 64 * 20 + 1, 0, 1], 32, 4, 64, {}),
    ("cut_units", [9000, 100, 64], 32, 4, 64, {"MLC_B200_DECODE_MODE": "2", "MLC_B200_DECODE_UNIT_CUT_FORCE": "1"}),
    ("d128_g4", [700, 64, 2500], 32, 8, 128, {}),
    ("g16", [300, 1200], 32, 2, 64, {"MLC_B200_DECODE_MODE": "2"}),
]


@pytest.mark.parametrize("name,lens,h,kvh,d,env", FUSED_CASES, ids=[c[0] for c in FUSED_CASES])
def test_fused_attention_and_exchange_single_rank(oracle_mod, name, lens, h, kvh, d, env):
    """world = 1: every finished (request, head) is pushed to this rank's own buffer, flagged, waited for and
    normalised in the same launch - the result is plain attention, on every step (both buffer parities) and
    from a CUDA graph."""
    import torch
    from mlcompiler_b200 import Executor, synth
    from mlcompiler_b200.capi import MLC_F16, PeerExchange
    from tests.util import DeviceCase, assert_attention_close
    case = synth.make_case(93, lens, h, kvh, d, P=P)
    ex = Executor(0)
    dc = DeviceCase(case)
    os.environ.update(env)
    try:
        plan = ex.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, case.N, h, kvh, d, P, True, case.capacity)
    finally:
        for k in env:
            del os.environ[k]
    xc = PeerExchange(ex, 0, 1, case.N * h, d)
    want = oracle_mod.paged_attention(case.q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                      case.seq_lens, case.q_pos, h, kvh, d, P, scale=case.scale)
    out = dc.out()
    for _ in range(3):
        out.fill_(float("nan"))
        assert ex.beginForwardPassCB()
        before = ex.launchCount()
        assert xc.encodeAttentionExchange(plan, dc.q, dc.k_pool, dc.v_pool, out, case.scale, MLC_F16, MLC_F16), ex.last_error()
        assert ex.launchCount() - before == 1
        assert ex.flushForwardPassCB(), ex.last_error()
        assert_attention_close(out.float().cpu().numpy(), want)
    assert ex.beginForwardPassCB()
    assert ex.beginCapture()
    assert xc.encodeAttentionExchange(plan, dc.q, dc.k_pool, dc.v_pool, out, case.scale, MLC_F16, MLC_F16), ex.last_error()
    graph = ex.endCapture()
    for _ in range(3):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        graph.launch()
        assert ex.flushForwardPassCB(), ex.last_error()
        assert ex.beginForwardPassCB()
        assert_attention_close(out.float().cpu().numpy(), want)
    assert ex.flushForwardPassCB(), ex.last_error()
    graph.destroy()
    xc.destroy()
    plan.destroy()
    ex.close()


def test_sequence_sharded_attention_over_peer_memory(oracle_mod, tmp_path):
    """The NCCL-free path: partials pushed into the peers' gather buffers, flags, combine - one kernel."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tests.util import assert_attention_close
    world = 2
    mp.spawn(_exchange_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    case = _case()
    whole = oracle_mod.paged_attention(case.q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                       case.seq_lens, np.zeros(case.N, np.uint32), H, KVH, D, P, causal=False,
                                       scale=case.scale)
    for rank in range(world):
        assert_attention_close(np.load(tmp_path / f"xrank{rank}.npy"), whole)


def test_peer_exchange_single_rank_equals_lse_combine(oracle_mod):
    """world = 1: the kernel pushes to itself, waits on its own flag and normalises - the same numbers
    as mlc_encode_lse_combine over one part, on every step (both buffer parities)."""
    import torch
    from mlcompiler_b200 import Executor
    from mlcompiler_b200.capi import MLC_F32, PeerExchange
    dev = torch.device("cuda:0")
    ex = Executor(0)
    rows, Dh = 200, 64
    g = torch.Generator(device="cpu").manual_seed(4)
    o_part = torch.randn((rows, Dh), generator=g).to(dev)
    ml = torch.stack([torch.randn(rows, generator=g), torch.rand(rows, generator=g) + 0.5], dim=1).contiguous().to(dev)
    ml[7, 0] = float("-inf")   # an empty slice: weight 0
    ml[7, 1] = 0.0
    want = torch.zeros((rows, Dh), device=dev)
    got = torch.zeros((rows, Dh), device=dev)
    xc = PeerExchange(ex, 0, 1, 256, Dh)
    assert ex.beginForwardPassCB()
    assert ex.encodeLseCombine(o_part, ml, 1, rows, Dh, want, MLC_F32), ex.last_error()
    assert ex.flushForwardPassCB(), ex.last_error()
    for _ in range(3):
        got.zero_()
        assert ex.beginForwardPassCB()
        assert xc.encodeLseCombine(o_part, ml, rows, got, MLC_F32), ex.last_error()
        assert ex.flushForwardPassCB(), ex.last_error()
        assert torch.equal(got, want)
    ref = oracle_mod.lse_combine(o_part.cpu().numpy()[None], ml.cpu().numpy()[None])
    assert np.allclose(got.cpu().numpy(), ref, rtol=1e-6, atol=1e-7)
    xc.destroy()
    ex.close()


def test_sequence_sharded_attention_over_nccl(oracle_mod, tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tests.util import assert_attention_close
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    case = _case()
    whole = oracle_mod.paged_attention(case.q.astype(np.float32), case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                       case.seq_lens, np.zeros(case.N, np.uint32), H, KVH, D, P, causal=False,
                                       scale=case.scale)
    for rank in range(world):
        assert_attention_close(np.load(tmp_path / f"rank{rank}.npy"), whole)
