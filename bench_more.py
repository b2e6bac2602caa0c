#!/usr/bin/env python3
"""Secondary workloads of the paged-attention path (bench.py holds the headline one).

    python bench_more.py --workload cfg3 [--steps K]          # long-context split-KV
    python bench_more.py --workload cfg4 [--steps K]          # wide GQA, requests sharded by KV bytes
    python bench_more.py --workload cfg5 [--steps K]          # chunked prefill on tcgen05
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        bench_more.py --workload cfg3|cfg4|cfg5

cfg3: 4 requests of 32768 tokens (512 pages each), H32/KVH4/D64. With N ranks every rank holds
a contiguous 1/N of every request's pages, computes the un-normalised partial (o, m, l), the
partials are all-gathered with NCCL and combined by mlc_encode_lse_combine.
cfg4: 128 requests, H32/KVH8/D128, contexts U[512, 8192], requests assigned to ranks by greedy
longest-first packing on KV bytes; no collective.
cfg5: 8 requests, each a 512-token chunk on top of 1536 cached tokens, H32/KVH8/D128, causal; requests
are dealt round-robin to ranks, no collective. Metric: attention TFLOP/s (4*D flops per visible
(query, key) pair), against the measured dense bf16 tensor peak.
Prints one JSON line (rank 0). Pools rotate so that consecutive steps never re-read L2-resident data.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def measured_peak_tflops():
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


def run_cfg5(args):
    import torch
    import torch.distributed as dist
    from mlcompiler_b200 import Executor, synth
    from mlcompiler_b200.capi import MLC_F16

    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    stream = torch.cuda.Stream(device=dev)
    ex = Executor(local, stream=stream.cuda_stream)
    P, H, KVH, D = 64, 32, 8, 128
    n_req, new, cached = 8, 512, 1536
    mine = list(range(rank, n_req, world))
    N = len(mine)
    seq = np.full(N, new + cached, np.uint32)
    case = synth.make_case(0xBEEF + 5 + rank, seq, P=P, fill=False, H=H, KVH=KVH, D=D)
    q_start = np.full(N, cached, np.uint32)
    q_len = np.full(N, new, np.uint32)
    cap = case.capacity
    # visible (query, key) pairs per (request, head): sum_i (cached + i + 1)
    pairs = new * cached + new * (new + 1) // 2
    flops_local = 4.0 * D * pairs * H * N
    kv_bytes = case.kv_bytes
    copies = max(2, int(np.ceil(300e6 / max(kv_bytes + 2 * N * new * H * D * 2, 1))))
    with torch.cuda.stream(stream):
        kp = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16) for _ in range(copies)]
        vp = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16) for _ in range(copies)]
        q = [torch.randn((N * new, H, D), device=dev, dtype=torch.float16) for _ in range(copies)]
        out = [torch.zeros((N * new, H, D), device=dev, dtype=torch.float16) for _ in range(copies)]

    def step(i):
        c = i % copies
        ok = ex.encodePagedPrefillAttention(q[c], kp[c], vp[c], out[c], case.pt_flat, case.pt_off, case.seq_lens,
                                            q_start, q_len, N, H, KVH, D, P, case.scale, MLC_F16, MLC_F16, cap)
        assert ok, ex.last_error()

    def barrier():
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    assert ex.beginForwardPassCB()
    for i in range(max(args.warmup, 3)):
        step(i)
    assert ex.flushForwardPassCB(), ex.last_error()
    assert ex.lastAttentionKernel() == 3, "the tcgen05 kernel did not run"
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = ex.launchCount()
    assert ex.beginForwardPassCB()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    assert ex.flushForwardPassCB(), ex.last_error()
    launches = ex.launchCount() - l0
    sec = e0.elapsed_time(e1) * 1e-3 / args.steps
    flops = flops_local
    if world > 1:
        t = torch.tensor([sec, flops_local], device=dev, dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        sec, flops = float(tmax[0].item()), float(t[1].item())
    burst, sustained, kind = measured_peak_tflops()
    if rank == 0:
        value = flops / sec / 1e12
        print(json.dumps({
            "metric": "paged_prefill_attn_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": {"workload": "cfg5: 8 requests x (512 new + 1536 cached tokens), H32/KVH8/D128, causal chunked prefill",
                       "parallelism": f"request-sharded x{world}", "pool_copies_rotated": copies},
            "tokens_per_s": n_req * new / sec,
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": burst, "unit": "TFLOP/s",
                         "frac": value / world / burst, "peak_source": kind, "peak_sustained": sustained,
                         "note": "per GPU; dense bf16 cuBLAS burst peak"},
            "gpu_launches": int(launches)}))
    ex.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=["cfg3", "cfg4", "cfg5"], required=True)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="cfg3 on several GPUs: peer-memory exchange kernel (default) or NCCL all-gather + combine")
    args = ap.parse_args()
    if args.workload == "cfg5":
        return run_cfg5(args)

    import torch
    import torch.distributed as dist
    from bench import measured_peak_gbs
    from mlcompiler_b200 import Executor, sharding, synth
    from mlcompiler_b200.capi import MLC_F16, MLC_F32, PeerExchange

    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    stream = torch.cuda.Stream(device=dev)
    ex = Executor(local, stream=stream.cuda_stream)
    P = 64

    def barrier():
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(x, op):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return float(t.item())

    if args.workload == "cfg3":
        shape = synth.SHAPE_A
        H, KVH, D = shape["H"], shape["KVH"], shape["D"]
        case = synth.make_case(0xBEEF + 3, synth.config_lengths(3), P=P, fill=False, **shape)
        N = case.N
        flat, off, lens, _ = sharding.slice_tables_for_rank(case.pt_flat, case.pt_off, case.seq_lens, P, rank, world)
        # local pool: only this rank's pages, renumbered densely
        remap = {int(p): i for i, p in enumerate(flat)}
        flat_local = np.array([remap[int(p)] for p in flat], np.uint32)
        cap = len(flat_local)
        local_bytes = int(lens.astype(np.int64).sum()) * 2 * KVH * D * 2
        copies = max(2, int(np.ceil(300e6 / max(local_bytes, 1))))       # rotate over > 2x L2 worth of pools
        with torch.cuda.stream(stream):
            kp = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16) for _ in range(copies)]
            vp = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16) for _ in range(copies)]
            q = torch.randn((N, H, D), device=dev, dtype=torch.float16)
            o_part = torch.zeros((N, H, D), device=dev, dtype=torch.float32)
            ml_part = torch.zeros((N, H, 2), device=dev, dtype=torch.float32)
            out = torch.zeros((N, H, D), device=dev, dtype=torch.float16)
        plan = ex.createPlan(flat_local, off, lens, np.zeros(N, np.uint32), N, H, KVH, D, P, False, cap)
        use_peer = world > 1 and args.exchange == "peer"
        xc = None
        if use_peer:
            xc = PeerExchange(ex, rank, world, N * H, D)
            xc.attach_with_torch_distributed()
        graphs = None

        def step(i):
            if graphs is not None:
                graphs[i % copies].launch()
                return
            assert ex.beginForwardPassCB()
            if world == 1:
                ok = ex.encodePagedFlashAttentionPlanned(plan, q, kp[i % copies], vp[i % copies], out, case.scale, MLC_F16, MLC_F16)
                assert ok, ex.last_error()
            elif use_peer:
                ok = ex.encodePagedAttentionPartialPlanned(plan, q, kp[i % copies], vp[i % copies], o_part, ml_part, case.scale, MLC_F16)
                assert ok, ex.last_error()
                assert xc.encodeLseCombine(o_part, ml_part, N * H, out, MLC_F16), ex.last_error()
            else:
                ok = ex.encodePagedAttentionPartialPlanned(plan, q, kp[i % copies], vp[i % copies], o_part, ml_part, case.scale, MLC_F16)
                assert ok, ex.last_error()
                with torch.cuda.stream(stream):
                    o_all, ml_all = sharding.gather_partials(o_part, ml_part)
                assert ex.encodeLseCombine(o_all, ml_all, world, N * H, D, out, MLC_F16), ex.last_error()
            ex._lib.mlc_pass_is_open(ex.handle)  # keep the pass open across steps: one flush at the end

        for i in range(max(args.warmup, 3)):
            step(i)
        assert ex.flushForwardPassCB(), ex.last_error()
        barrier()
        if world == 1 or use_peer:
            # only this library's kernels in a step: replay them as CUDA graphs, one per pool copy
            built = []
            for c in range(copies):
                assert ex.beginForwardPassCB()
                assert ex.beginCapture()
                step(c)
                built.append(ex.endCapture())
            graphs = built
            for i in range(copies * 2):     # every rank replays the same sequence: the exchange stays in step
                step(i)
            assert ex.flushForwardPassCB(), ex.last_error()
            barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = ex.launchCount()
        assert ex.beginForwardPassCB()
        e0.record(stream)
        for i in range(args.steps):
            step(i)
        e1.record(stream)
        assert ex.flushForwardPassCB(), ex.last_error()
        launches = ex.launchCount() - l0
        sec = reduce(e0.elapsed_time(e1) * 1e-3, dist.ReduceOp.MAX if world > 1 else None) / args.steps
        total_bytes = case.kv_bytes
        how = ("one GPU" if world == 1 else "partials pushed to the peers' memory, flags, combine - one kernel" if use_peer
               else "NCCL all-gather of (o,m,l), LSE combine")
        workload = "cfg3: 4 requests x 32768 tokens, H32/KVH4/D64, KV sequence split over ranks, " + how
        extra = {"parallelism": f"sequence-sharded x{world}", "pool_copies_rotated": copies, "cuda_graph": graphs is not None,
                 "gather_bytes_per_rank": int((o_part.numel() + ml_part.numel()) * 4) if world > 1 else 0}
        n_req = N
    else:
        shape = synth.SHAPE_B
        H, KVH, D = shape["H"], shape["KVH"], shape["D"]
        all_lens = synth.config_lengths(4)
        shards = synth.shard_requests_by_kv_bytes(all_lens, world)
        mine = all_lens[shards[rank]]
        case = synth.make_case(0xBEEF + 4 + rank, mine, P=P, fill=False, **shape)
        N, cap = case.N, case.capacity
        local_bytes = case.kv_bytes
        copies = max(2, int(np.ceil(300e6 / max(local_bytes, 1))))
        with torch.cuda.stream(stream):
            kp = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16) for _ in range(copies)]
            vp = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16) for _ in range(copies)]
            q = torch.randn((N, H, D), device=dev, dtype=torch.float16)
            kn = torch.randn((N, KVH, D), device=dev, dtype=torch.float16)
            vn = torch.randn((N, KVH, D), device=dev, dtype=torch.float16)
            out = torch.zeros((N, H, D), device=dev, dtype=torch.float16)
        plan = ex.createPlan(case.pt_flat, case.pt_off, case.seq_lens, case.q_pos, N, H, KVH, D, P, True, cap,
                             page_ids=case.page_ids, slots_in_page=case.slots)

        def enc():
            for c in range(copies):
                assert ex.encodePagedDecodeStepPlanned(plan, q, kn, vn, kp[c], vp[c], out, case.scale, MLC_F16, MLC_F16), ex.last_error()

        assert ex.beginForwardPassCB()
        enc()
        assert ex.flushForwardPassCB(), ex.last_error()
        assert ex.beginForwardPassCB()
        assert ex.beginCapture()
        enc()
        graph = ex.endCapture()
        for _ in range(max(args.warmup, 3)):
            graph.launch()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = ex.launchCount()
        reps = max(args.steps // copies, 1)
        e0.record(stream)
        for _ in range(reps):
            graph.launch()
        e1.record(stream)
        stream.synchronize()
        launches = ex.launchCount() - l0
        assert ex.flushForwardPassCB(), ex.last_error()
        sec = reduce(e0.elapsed_time(e1) * 1e-3, dist.ReduceOp.MAX if world > 1 else None) / (reps * copies)
        total_bytes = reduce(float(local_bytes), dist.ReduceOp.SUM if world > 1 else None)
        loads = np.array([all_lens[s].sum() for s in shards], np.float64)
        workload = "cfg4: 128 requests, H32/KVH8/D128, contexts U[512,8192], requests sharded by KV bytes; scatter + attention fused"
        extra = {"parallelism": f"request-sharded x{world}", "pool_copies_rotated": copies,
                 "kv_byte_imbalance_max_over_mean": float(loads.max() / loads.mean())}
        n_req = len(all_lens)

    peak, kind = measured_peak_gbs()
    if rank == 0:
        value = total_bytes / sec / 1e9
        print(json.dumps({
            "metric": "paged_decode_attn_kv_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong", "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": {"workload": workload, **extra}, "tokens_per_s": n_req / sec,
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak, "peak_source": kind, "note": "per GPU"},
            "gpu_launches": int(launches)}))
    if world > 1:
        dist.barrier()
    if args.workload == "cfg3" and xc is not None:
        xc.destroy()
    plan.destroy()
    ex.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
