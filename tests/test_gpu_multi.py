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
