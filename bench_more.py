#!/usr/bin/env python3
"""Secondary workloads of the paged-attention path (bench.py holds the headline one and runs these
too, under its `secondary` key).

    python bench_more.py --workload cfg3 [--steps K]          # long-context split-KV
    python bench_more.py --workload cfg4 [--steps K]          # wide GQA, requests sharded by KV bytes
    python bench_more.py --workload cfg5 [--steps K]          # chunked prefill on tcgen05
    python bench_more.py --workload model [--steps K]         # whole decode step of a 1.1B-shaped model
    python bench_more.py --workload matvec --rows R --cols C [--quant q4_0|q6_k] [--batch B]   # one quantised mat-vec
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        bench_more.py --workload cfg3|cfg4|cfg5

cfg3: 4 requests of 32768 tokens (512 pages each), H32/KVH4/D64. With N ranks every rank holds
a contiguous 1/N of every request's pages and computes the un-normalised partial (o, m, l); the
partials are exchanged by this library's peer-memory kernel (or all-gathered with NCCL, --exchange
nccl) and combined. With N > 1 one step is also checked on rank 0 against attention over the whole
sequence on that one GPU.
cfg4: 128 requests, H32/KVH8/D128, contexts U[512, 8192], requests assigned to ranks by greedy
longest-first packing on KV bytes; no collective.
cfg5: 8 requests, each a 512-token chunk on top of 1536 cached tokens, H32/KVH8/D128, causal; requests
are dealt round-robin to ranks, no collective. Metric: attention TFLOP/s (4*D flops per visible
(query, key) pair), against the measured dense bf16 tensor peak.
model: the whole walker step (compiler/runtime/batched_walker.cpp:183-458) of a model with TinyLlama-1.1B's
shape - 22 layers, hidden 2048, H32/KVH4/D64, FFN 5632, vocabulary 32000, Q4_0 weights, Q6_K lm_head - for
32 requests with contexts U[512, 2048], through the paged executor's run_decode: page extension, plan update,
token upload, every launch of the pass, logits [32, 32000] back on the host. Weights are seeded synthetic
bytes in the real formats (there is no checkpoint to load here), the contexts' K/V rows random. Metric:
generated tokens per second, wall clock around run_decode (the call returns when the logits are on the
host). With N ranks every rank serves its own 32 requests on its own copy of the weights.
matvec: one quantised batched mat-vec (mlc_encode_matmul_q4_0_batched / _q6k_batched) at a given shape, default
the 1.1B model's gate | up projection (11264 x 2048, Q4_0, 32 requests); the weights rotate over enough copies
to exceed L2, so every launch streams them from HBM. MLC_B200_MATVEC=tcgen05 selects the tensor-memory kernel.
Metric: GB/s of weight bytes against the measured copy bandwidth.
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


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class Env:
    """What every workload needs: the rank's device, stream, executor and the reductions over ranks."""

    def __init__(self, ex, stream, dev, rank, world):
        self.ex, self.stream, self.dev, self.rank, self.world = ex, stream, dev, rank, world

    def barrier(self):
        import torch
        import torch.distributed as dist
        self.stream.synchronize()
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(self, x, op):
        import torch
        import torch.distributed as dist
        if self.world == 1:
            return x
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM}[op])
        return float(t.item())


def _timed(env, fn, steps):
    """CUDA events on the launching stream around `steps` calls of fn(i); seconds per step, max over ranks."""
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(env.stream)
    for i in range(steps):
        fn(i)
    e1.record(env.stream)
    env.stream.synchronize()
    return env.reduce(e0.elapsed_time(e1) * 1e-3, "max") / steps


def run_cfg5(env, steps=200, warmup=10):
    import torch
    from mlcompiler_b200 import synth
    from mlcompiler_b200.capi import MLC_F16
    ex, stream, dev, rank, world = env.ex, env.stream, env.dev, env.rank, env.world
    P, H, KVH, D = 64, 32, 8, 128
    n_req, new, cached = 8, 512, 1536
    mine = list(range(rank, n_req, world))
    N = len(mine)
    if N == 0:      # more ranks than requests: this rank only takes part in the reductions
        env.barrier()
        env.reduce(0.0, "max")
        env.reduce(0.0, "sum")
        return None
    seq = np.full(N, new + cached, np.uint32)
    case = synth.make_case(0xBEEF + 5 + rank, seq, P=P, fill=False, H=H, KVH=KVH, D=D)
    q_start = np.full(N, cached, np.uint32)
    q_len = np.full(N, new, np.uint32)
    cap = case.capacity
    # visible (query, key) pairs per (request, head): sum_i (cached + i + 1)
    pairs = new * cached + new * (new + 1) // 2
    flops_local = 4.0 * D * pairs * H * N
    copies = max(2, int(np.ceil(300e6 / max(case.kv_bytes + 2 * N * new * H * D * 2, 1))))
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

    assert ex.beginForwardPassCB()
    for i in range(max(warmup, 3)):
        step(i)
    assert ex.flushForwardPassCB(), ex.last_error()
    assert ex.lastAttentionKernel() == 3, "the tcgen05 kernel did not run"
    env.barrier()
    l0 = ex.launchCount()
    assert ex.beginForwardPassCB()
    sec = _timed(env, step, steps)
    assert ex.flushForwardPassCB(), ex.last_error()
    launches = ex.launchCount() - l0
    flops = env.reduce(flops_local, "sum")
    peaks = measured_peaks()
    value = flops / sec / 1e12
    per_gpu = value / min(world, n_req)
    return {
        "metric": "paged_prefill_attn_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "dtype": "f16 in, f32 accumulate", "data": "synthetic",
        "config": {"workload": "cfg5: 8 requests x (512 new + 1536 cached tokens), H32/KVH8/D128, causal chunked prefill",
                   "parallelism": f"request-sharded x{world}", "pool_copies_rotated": copies},
        "tokens_per_s": n_req * new / sec,
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": per_gpu / peaks["bf16_tflops"], "peak_source": peaks["source"],
                     "peak_sustained": peaks["bf16_tflops_sustained"],
                     "note": "per GPU that holds a request; dense bf16 cuBLAS burst peak"},
        "gpu_launches": int(launches)}


def run_cfg3(env, steps=200, warmup=10, exchange="fused", check=True, seq_len=None):
    import torch
    from mlcompiler_b200 import sharding, synth
    from mlcompiler_b200.capi import MLC_F16, PeerExchange
    ex, stream, dev, rank, world = env.ex, env.stream, env.dev, env.rank, env.world
    P = 64
    shape = synth.SHAPE_A
    H, KVH, D = shape["H"], shape["KVH"], shape["D"]
    seq = synth.config_lengths(3) if seq_len is None else np.full(4, seq_len, np.uint32)
    case = synth.make_case(0xBEEF + 3, seq, P=P, fill=False, **shape)
    N = case.N
    flat, off, lens, _ = sharding.slice_tables_for_rank(case.pt_flat, case.pt_off, case.seq_lens, P, rank, world)
    # local pool: only this rank's pages, renumbered densely
    remap = {int(p): i for i, p in enumerate(flat)}
    flat_local = np.array([remap[int(p)] for p in flat], np.uint32)
    cap = len(flat_local)
    local_bytes = int(lens.astype(np.int64).sum()) * 2 * KVH * D * 2
    copies = max(2, int(np.ceil(300e6 / max(local_bytes, 1))))       # rotate over > 2x L2 worth of pools
    g = torch.Generator(device=dev)
    g.manual_seed(3000 + rank)
    with torch.cuda.stream(stream):
        kp = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16, generator=g) for _ in range(copies)]
        vp = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16, generator=g) for _ in range(copies)]
        gq = torch.Generator(device=dev)
        gq.manual_seed(3)      # the same queries on every rank
        q = torch.randn((N, H, D), device=dev, dtype=torch.float16, generator=gq)
        o_part = torch.zeros((N, H, D), device=dev, dtype=torch.float32)
        ml_part = torch.zeros((N, H, 2), device=dev, dtype=torch.float32)
        out = torch.zeros((N, H, D), device=dev, dtype=torch.float16)
    plan = ex.createPlan(flat_local, off, lens, np.zeros(N, np.uint32), N, H, KVH, D, P, False, cap)
    use_peer = world > 1 and exchange in ("peer", "fused")
    fused = use_peer and exchange == "fused"
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
        c = i % copies
        if world == 1:
            ok = ex.encodePagedFlashAttentionPlanned(plan, q, kp[c], vp[c], out, case.scale, MLC_F16, MLC_F16)
            assert ok, ex.last_error()
        elif fused:     # partial attention + exchange + combine: one launch
            assert xc.encodeAttentionExchange(plan, q, kp[c], vp[c], out, case.scale, MLC_F16, MLC_F16), ex.last_error()
        elif use_peer:
            ok = ex.encodePagedAttentionPartialPlanned(plan, q, kp[c], vp[c], o_part, ml_part, case.scale, MLC_F16)
            assert ok, ex.last_error()
            assert xc.encodeLseCombine(o_part, ml_part, N * H, out, MLC_F16), ex.last_error()
        else:
            ok = ex.encodePagedAttentionPartialPlanned(plan, q, kp[c], vp[c], o_part, ml_part, case.scale, MLC_F16)
            assert ok, ex.last_error()
            with torch.cuda.stream(stream):
                o_all, ml_all = sharding.gather_partials(o_part, ml_part)
            assert ex.encodeLseCombine(o_all, ml_all, world, N * H, D, out, MLC_F16), ex.last_error()

    for i in range(max(warmup, 3)):
        step(i)
    assert ex.flushForwardPassCB(), ex.last_error()
    env.barrier()

    # ---- one step of the split checked against the unsplit attention on one GPU (rank 0) ----
    checked = None
    if world > 1 and check:
        import torch.distributed as dist
        step(0)
        assert ex.flushForwardPassCB(), ex.last_error()
        split_out = out.clone()
        # rank 0 collects every rank's slice of pool copy 0 and lays the whole sequence out locally
        sizes = [None] * world
        dist.all_gather_object(sizes, cap)
        if rank == 0:
            full_k = [kp[0]] + [torch.empty((sizes[r], P, KVH, D), device=dev, dtype=torch.float16) for r in range(1, world)]
            full_v = [vp[0]] + [torch.empty((sizes[r], P, KVH, D), device=dev, dtype=torch.float16) for r in range(1, world)]
            for r in range(1, world):
                dist.recv(full_k[r], src=r)
                dist.recv(full_v[r], src=r)
            base = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
            all_flat, all_off = [], [0]
            per_rank = [sharding.slice_tables_for_rank(case.pt_flat, case.pt_off, case.seq_lens, P, r, world) for r in range(world)]
            for req in range(N):
                for r in range(world):
                    f_r, o_r, _, _ = per_rank[r]
                    # the rank's pages are renumbered densely in the order of its flat table
                    all_flat.extend(range(int(base[r] + o_r[req]), int(base[r] + o_r[req + 1])))
                all_off.append(len(all_flat))
            kw, vw = torch.cat(full_k), torch.cat(full_v)
            whole = torch.zeros_like(out)
            ok = ex.runPagedFlashAttention(q, kw, vw, whole, np.array(all_flat, np.uint32), np.array(all_off, np.uint32),
                                           case.seq_lens, np.zeros(N, np.uint32), N, H, KVH, D, P, False, case.scale,
                                           MLC_F16, MLC_F16, int(base[-1]))
            assert ok, ex.last_error()
            err = float((whole.float() - split_out.float()).abs().max().item())
            checked = {"max_abs_vs_one_gpu": err, "ok": err <= 2e-3}
            del kw, vw, full_k, full_v
        else:
            dist.send(kp[0], dst=0)
            dist.send(vp[0], dst=0)
        env.barrier()

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
        env.barrier()
    l0 = ex.launchCount()
    assert ex.beginForwardPassCB()
    sec = _timed(env, step, steps)
    assert ex.flushForwardPassCB(), ex.last_error()
    launches = ex.launchCount() - l0
    total_bytes = case.kv_bytes
    how = ("one GPU" if world == 1 else
           "one launch per rank: rows pushed to the peers' memory as each (request, head) finishes, flags, combine" if fused else
           "partial attention, then this library's exchange + combine kernel over peer memory" if use_peer else
           "NCCL all-gather of (o,m,l), LSE combine")
    peaks = measured_peaks()
    value = total_bytes / sec / 1e9
    res = {
        "metric": "paged_decode_attn_kv_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": sec * 1e3, "us_per_step": sec * 1e6, "higher_is_better": True,
        "scaling": "strong", "dtype": "f16 in, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"cfg3: 4 requests x {int(seq[0])} tokens, H32/KVH4/D64, KV sequence split over ranks, " + how,
                   "parallelism": f"sequence-sharded x{world}", "pool_copies_rotated": copies,
                   "cuda_graph": graphs is not None,
                   "gather_bytes_per_rank": int((o_part.numel() + ml_part.numel()) * 4) if world > 1 else 0},
        "tokens_per_s": N / sec,
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": value / world / peaks["hbm_gbs"], "peak_source": peaks["source"], "note": "per GPU"},
        "gpu_launches": int(launches)}
    if checked is not None:
        res["split_vs_one_gpu"] = checked
    if graphs:
        for gph in graphs:
            gph.destroy()
    if world > 1:
        env.barrier()
    if xc is not None:
        xc.destroy()
    plan.destroy()
    return res


def run_cfg4(env, steps=200, warmup=10):
    import torch
    from mlcompiler_b200 import synth
    from mlcompiler_b200.capi import MLC_F16
    ex, stream, dev, rank, world = env.ex, env.stream, env.dev, env.rank, env.world
    P = 64
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
    for _ in range(max(warmup, 3)):
        graph.launch()
    env.barrier()
    l0 = ex.launchCount()
    reps = max(steps // copies, 1)
    sec = _timed(env, lambda i: graph.launch(), reps) / copies
    launches = ex.launchCount() - l0
    assert ex.flushForwardPassCB(), ex.last_error()
    total_bytes = env.reduce(float(local_bytes), "sum")
    loads = np.array([all_lens[s].sum() for s in shards], np.float64)
    peaks = measured_peaks()
    value = total_bytes / sec / 1e9
    graph.destroy()
    plan.destroy()
    return {
        "metric": "paged_decode_attn_kv_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": reps * copies,
        "warmup": max(warmup, 3), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "dtype": "f16 in, f32 accumulate", "data": "synthetic",
        "config": {"workload": "cfg4: 128 requests, H32/KVH8/D128, contexts U[512,8192], requests sharded by KV bytes; "
                               "scatter + attention fused, one launch per layer",
                   "parallelism": f"request-sharded x{world}", "pool_copies_rotated": copies,
                   "kv_byte_imbalance_max_over_mean": float(loads.max() / loads.mean())},
        "tokens_per_s": len(all_lens) / sec,
        "roofline": {"bound": "hbm", "achieved": value / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": value / world / peaks["hbm_gbs"], "peak_source": peaks["source"], "note": "per GPU"},
        "gpu_launches": int(launches)}


class _RawHalf:
    """A device buffer of this library as something torch.as_tensor can wrap."""

    def __init__(self, ptr, n_halves):
        self.__cuda_array_interface__ = {"shape": (n_halves,), "typestr": "<f2", "data": (int(ptr), False), "version": 3}


def run_model(env, steps=40, warmup=5, batch=32, reference_order=False, from_gguf=False, prompt_tokens=1024):
    import time
    import torch
    from mlcompiler_b200 import synth
    from mlcompiler_b200.host import PagePool, PagedAttentionExecutor, PagedKVStorage
    ex, stream, dev, rank, world = env.ex, env.stream, env.dev, env.rank, env.world
    P, L, H, KVH, D, inner, vocab = 64, 22, 32, 4, 64, 5632, 32000
    model = synth.SyntheticModel(0x11B, L, H, KVH, D, inner, vocab, lm_head_quant="q6_k")
    lens = np.resize(synth.config_lengths(2), batch).astype(np.int64)   # past 32 requests the lengths repeat
    total_steps = steps + max(warmup, 3)
    sched_prompt, sched_new = 128, 64
    capacity = (int(sum((int(l) + total_steps + P - 1) // P for l in lens)) + 4 + 2 * ((prompt_tokens + P - 1) // P + 1) +
                batch * ((sched_prompt + sched_new) // P + 2))
    pool = PagePool(capacity)
    storage = PagedKVStorage(ex, capacity, L, P, KVH, D, 2)
    assert storage.initialize()
    pex = PagedAttentionExecutor(ex, H, KVH, D, L, 0)
    pex.attach_page_pool(pool, P)
    pex.attach_paged_storage(storage)
    pex.set_call_order(reference_order)
    with torch.cuda.stream(stream):
        model.to_device(dev)
        n_halves = capacity * P * KVH * D
        for l in range(L):
            for ptr in (storage.k_buffer(l), storage.v_buffer(l)):
                torch.as_tensor(_RawHalf(ptr, n_halves), device=dev).normal_()
    stream.synchronize()
    load = None
    if from_gguf:
        # the same weights through a file: written as a GGUF checkpoint (q / k / v and gate / up apart), read back by the
        # library's loader and streamed into device memory
        import tempfile
        from mlcompiler_b200.host import GgufFile
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "model.gguf")
            model.write_gguf(path)
            size = os.path.getsize(path)
            t0 = time.perf_counter()
            f = GgufFile(path)
            assert pex.attach_gguf(f), pex.attach_error
            load = {"file_bytes": size, "seconds": time.perf_counter() - t0, "what": "mlc_gguf_open + mlc_executor_attach_gguf, "
                    "file in the page cache"}
            load["gbps"] = size / load["seconds"] / 1e9
            f.close()
    else:
        assert pex.attach_model(model)
    for r in range(batch):
        assert pex.assume_context(r, int(lens[r]) - 1)
    pos = [int(l) - 1 for l in lens]
    rng = np.random.default_rng(rank)

    def step():
        slots = [(r, int(rng.integers(0, vocab)), pos[r]) for r in range(batch)]
        out = pex.run_decode(slots)
        assert len(out) == batch and all(o[1] for o in out), ex.last_error()
        for r in range(batch):
            pos[r] += 1
        return out

    for _ in range(max(warmup, 3)):
        out = step()
    assert all(np.isfinite(o[2]).all() for o in out)
    env.barrier()
    l0 = ex.launchCount()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    launches = ex.launchCount() - l0
    sec = env.reduce(float(np.mean(times)), "max")
    # a prompt through run_prefill (32 tokens per pass in the fused order, one per pass in the reference's)
    prefill = None
    if prompt_tokens:
        n_prompt = prompt_tokens if not reference_order else min(prompt_tokens, 64)
        ptimes = []
        for rep_i in range(2):
            prompt = [int(t) for t in rng.integers(0, vocab, n_prompt)]
            t0 = time.perf_counter()
            lg = pex.run_prefill(batch + rep_i, prompt)
            ptimes.append(time.perf_counter() - t0)
            assert lg.size == vocab and np.isfinite(lg).all(), ex.last_error()
        psec = env.reduce(float(min(ptimes)), "max")
        prefill = {"prompt_tokens": n_prompt, "ms": psec * 1e3, "tokens_per_s": world * n_prompt / psec,
                   "what": "run_prefill of one request from an empty context, wall clock, last token's logits on the host"}
    kv_bytes = float(sum(pos)) * 2 * KVH * D * 2 * L
    # the same executor under the scheduler: `batch` requests of 128 prompt tokens, 64 new tokens each, greedy
    # sampling (on the device), one request admitted per tick as in the reference's scheduler
    served = None
    if prompt_tokens and not reference_order:
        from mlcompiler_b200.host import Scheduler
        for r in range(batch + 2):
            pex.release_request(r)
        sched = Scheduler(pex, max_batch_size=batch)
        for _ in range(batch):
            sched.add_request([int(t) for t in rng.integers(0, vocab, sched_prompt)], max_new_tokens=sched_new, eos_token_id=-1)
        t0 = time.perf_counter()
        ticks = 0
        while not sched.empty():
            sched.tick()
            ticks += 1
        dt = env.reduce(time.perf_counter() - t0, "max")
        made = sum(len(r["generated_tokens"]) for r in sched.drain_completed())
        served = {"requests": batch, "prompt_tokens": sched_prompt, "new_tokens": sched_new, "ticks": ticks, "ms": dt * 1e3,
                  "generated_tokens_per_s": world * made / dt,
                  "what": "Scheduler.tick until idle: admission (one prompt per tick, 32 tokens per pass), batched decode "
                          "passes with greedy sampling on the device"}
    pex.destroy()
    storage.destroy()
    return {
        "metric": "decode_tokens_per_s", "value": world * batch / sec, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "dtype": "Q4_0 / Q6_K weights, f16 KV, f32 activations", "data": "synthetic",
        "config": {"workload": "model: 1.1B-shaped decoder (22 layers, hidden 2048, H32/KVH4/D64, FFN 5632, vocabulary "
                               f"32000), {batch} requests, contexts U[512,2048], whole walker step through run_decode",
                   "call_order": "reference" if reference_order else "fused",
                   "parallelism": f"replicas x{world}, {batch} requests each", "timed": "wall clock around run_decode, "
                   "logits on the host when it returns"},
        "ms_per_step_median_min_max": [float(np.median(times)) * 1e3, float(np.min(times)) * 1e3, float(np.max(times)) * 1e3],
        "bytes_per_step": {"weights": model.weight_bytes() - model.host["token_embd.weight"].nbytes, "kv": kv_bytes},
        "gpu_launches": int(launches), "launches_per_step": launches / steps, "prefill": prefill, "served": served, "model_load": load}


def run_matvec(env, steps=200, warmup=10, rows=11264, cols=2048, quant="q4_0", batch=32):
    import torch
    from mlcompiler_b200 import synth
    ex, stream, dev = env.ex, env.stream, env.dev
    rng = np.random.default_rng(7)
    raw = synth.random_q4_0(rng, rows, cols) if quant == "q4_0" else synth.random_q6_k(rng, rows, cols)
    copies = max(2, int(np.ceil(300e6 / raw.nbytes)))
    with torch.cuda.stream(stream):
        ws = [torch.from_numpy(raw).to(dev) for _ in range(copies)]
        x = torch.randn((batch, cols), device=dev)
        out = torch.zeros((batch, rows), device=dev)
    stream.synchronize()

    def enc():
        for w in ws:
            ok = (ex.encodeMatMulQ4_0Batched(w, x, batch, rows, cols, raw.shape[1], out) if quant == "q4_0" else
                  ex.encodeMatMulQ6KBatched(w, x, batch, rows, cols, raw.shape[1], out))
            assert ok, ex.last_error()

    assert ex.beginForwardPassCB()
    enc()
    assert ex.flushForwardPassCB(), ex.last_error()
    assert ex.beginForwardPassCB()
    assert ex.beginCapture()
    enc()
    graph = ex.endCapture()
    for _ in range(max(warmup, 3)):
        graph.launch()
    env.barrier()
    reps = max(steps // copies, 1)
    sec = _timed(env, lambda i: graph.launch(), reps) / copies
    assert ex.flushForwardPassCB(), ex.last_error()
    graph.destroy()
    peaks = measured_peaks()
    value = raw.nbytes / sec / 1e9
    flop = 2.0 * rows * cols * batch * 2          # hi and lo activation planes
    return {"metric": "quant_matvec_weight_gbps", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": reps * copies,
            "warmup": max(warmup, 3), "us_per_launch": sec * 1e6, "higher_is_better": True, "dtype": f"{quant} weights, f32 activations",
            "data": "synthetic", "config": {"workload": f"matvec {rows} x {cols} {quant}, batch {batch}", "weight_copies_rotated": copies,
                                            "kernel": os.environ.get("MLC_B200_MATVEC", "mma.sync (default)")},
            "tensor_tflops": flop / sec / 1e12,
            "roofline": {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": value / peaks["hbm_gbs"],
                         "peak_source": peaks["source"], "bytes_per_launch": int(raw.nbytes)}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=["cfg3", "cfg4", "cfg5", "model", "matvec"], required=True)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--exchange", choices=["fused", "peer", "nccl"], default="fused",
                    help="cfg3 on several GPUs: exchange fused into the attention kernel (default), the separate "
                         "peer-memory exchange kernel, or NCCL all-gather + combine")
    ap.add_argument("--from-gguf", action="store_true", help="model: load the weights through a GGUF file and report the load")
    ap.add_argument("--reference-order", action="store_true",
                    help="model: the reference walker's 13 launches per layer instead of the fused 8")
    ap.add_argument("--rows", type=int, default=11264, help="matvec: weight rows")
    ap.add_argument("--cols", type=int, default=2048, help="matvec: weight columns")
    ap.add_argument("--quant", choices=["q4_0", "q6_k"], default="q4_0", help="matvec: weight format")
    ap.add_argument("--batch", type=int, default=32, help="matvec, model: requests (model: at most 64)")
    ap.add_argument("--seq-len", type=int, default=None, help="cfg3: tokens per request instead of 32768")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from mlcompiler_b200 import Executor

    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    stream = torch.cuda.Stream(device=dev)
    ex = Executor(local, stream=stream.cuda_stream)
    env = Env(ex, stream, dev, rank, world)
    if args.workload == "cfg5":
        res = run_cfg5(env, args.steps, args.warmup)
    elif args.workload == "cfg3":
        res = run_cfg3(env, args.steps, args.warmup, args.exchange, seq_len=args.seq_len)
    elif args.workload == "matvec":
        res = run_matvec(env, args.steps, args.warmup, args.rows, args.cols, args.quant, args.batch)
    elif args.workload == "model":
        res = run_model(env, min(args.steps, 100), args.warmup, batch=args.batch, reference_order=args.reference_order,
                        from_gguf=args.from_gguf)
    else:
        res = run_cfg4(env, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(res))
    ex.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
