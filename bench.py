#!/usr/bin/env python3
"""Benchmark of the paged decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): continuous-batching decode over 22 layers of the TinyLlama head
shape (32 q heads / 4 KV heads, d = 64, fp16 KV, 64-token pages), 32 requests with
context lengths seeded uniform in [64, 2048], non-contiguous random page tables
over per-layer pools sized to the total pages + 10 %. One step = for every layer:
write one new K/V row per request into the pool, then run attention.

`value` is KV GB/s with everything resident in HBM: the step is replayed from a
CUDA graph (per layer one attention kernel with the KV row write and the merge fused
in; consecutive kernels overlap by programmatic dependent launch) and timed with CUDA
events on the launching stream. `e2e` is the same metric through the C ABI with host
buffers, the call sequence a walker with host activations makes: every step one
host-buffer pass call (Q and the new K/V rows of all layers copied in from pinned host
memory, one fused launch per layer, the attention output copied back to pinned host
memory, copies and kernels pipelined over groups of layers inside the call) and one
in-place plan update that hands over the NEXT step's page tables / lengths / positions
/ (page, slot) pairs as host arrays (they grow by one token per step, as in serving, and
do not depend on this step's results) while this step runs; the flush returns when the
output is complete in host memory. With N > 1 (torchrun, one rank per GPU) every rank
runs its own 32-request batch: request sharding, no collective on the data path (weak
scaling).

`--impl reference` times MLcompiler's own executor-CPU attention (compiled from
its unmodified sources into oracle/_ref, else the C port of it) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS = 22
METRIC = "paged_decode_attn_kv_gbps"
UNIT = "GB/s"
WORKLOAD = ("cfg2: 22-layer continuous-batching decode, 32 requests, H32/KVH4/D64, fp16 KV, 64-token pages, "
            "contexts U[64,2048], random page tables, pool = pages + 10%; per layer: scatter 1 new K/V row "
            "per request, then attention")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the decode kernel on this workload
# (37.79 MB read + <= 1.5 KB written), from the ncu captures summarised in
# profiles/decode_attention_cfg2.md; the algorithmic KV bytes of that launch are 37.00 MB.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 37_793_792


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.stop_flag = [], set(), False
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.thread = None

    def _poll_once(self):
        nv = self.nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        try:
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                 0x4: "sw_power_cap", 0x80: "hw_power_brake"}
        for bit, name in names.items():
            if r & bit:
                self.reasons.add(name)

    def _run(self):
        while not self.stop_flag:
            try:
                self._poll_once()
            except Exception:
                break
            time.sleep(0.02)

    def start(self):
        if self.nv:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread:
            self.thread.join()
        if self.nv and not self.samples:
            try:
                self._poll_once()
            except Exception:
                pass
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# --------------------------------------------------------------------------------------
# CPU arm
# --------------------------------------------------------------------------------------
class CpuArm:
    """MLcompiler's executor-CPU attention over ONE layer's requests of a workload
    (oracle/_ref when it is present, else the C port), one request per host thread."""

    def __init__(self, case, threads: int):
        import ctypes as C
        import oracle
        self.case, self.threads, self.C = case, threads, C
        self.lib = oracle.ref()
        self.q = case.q.astype(np.float32)
        self.order = sorted(range(case.N), key=lambda r: -int(case.seq_lens[r]))  # longest first
        self.bytes_per_pass = case.kv_bytes
        if self.lib is not None:
            self.kind = "reference"
            fp = C.POINTER(C.c_float)
            self.handles, self.new_rows, self.outs = [], [], []
            for r in range(case.N):
                S = int(case.seq_lens[r])
                k = np.ascontiguousarray(case.tokens_of(r, case.k_pool).astype(np.float32))
                v = np.ascontiguousarray(case.tokens_of(r, case.v_pool).astype(np.float32))
                h = self.lib.ref_attn_create(case.H, case.KVH, case.D, S)
                if S > 1:
                    self.lib.ref_attn_load_history(h, k.ctypes.data_as(fp), v.ctypes.data_as(fp), S - 1)
                self.handles.append(h)
                self.new_rows.append((np.ascontiguousarray(k[S - 1]), np.ascontiguousarray(v[S - 1]),
                                      np.ascontiguousarray(self.q[r])))
                self.outs.append(np.zeros((case.H, case.D), np.float32))
        else:
            self.kind = "port"
            oracle.build_port()
            self.oracle = oracle

    def _one(self, r):
        case = self.case
        if self.lib is not None:
            fp = self.C.POINTER(self.C.c_float)
            kn, vn, qr = self.new_rows[r]
            self.lib.ref_attn_decode_direct(self.handles[r], int(case.seq_lens[r]) - 1, qr.ctypes.data_as(fp),
                                            kn.ctypes.data_as(fp), vn.ctypes.data_as(fp),
                                            self.outs[r].ctypes.data_as(fp))
        else:
            self.oracle.paged_attention(self.q[r:r + 1], case.k_pool, case.v_pool,
                                        case.pt_flat[case.pt_off[r]:case.pt_off[r + 1]],
                                        [0, case.pt_off[r + 1] - case.pt_off[r]], case.seq_lens[r:r + 1],
                                        case.q_pos[r:r + 1], case.H, case.KVH, case.D, case.P, scale=case.scale)

    def run_pass(self, pool) -> float:
        t0 = time.perf_counter()
        list(pool.map(self._one, self.order))
        return time.perf_counter() - t0

    def close(self):
        if self.lib is not None:
            for h in self.handles:
                self.lib.ref_attn_destroy(h)
            self.handles = []

    def sample_text(self, passes):
        return (f"one layer of the workload ({self.case.N} requests, {self.bytes_per_pass / 1e6:.1f} MB KV) x "
                f"{passes} passes, one request per host thread, {self.threads} threads")


def cpu_baseline_sample(case, budget_s: float):
    threads = os.cpu_count() or 1
    arm = CpuArm(case, threads)
    passes, total = 0, 0.0
    with ThreadPoolExecutor(max_workers=threads) as pool:
        arm.run_pass(pool)  # warm-up
        while total < budget_s or passes == 0:
            total += arm.run_pass(pool)
            passes += 1
    arm.close()
    return {"value": arm.bytes_per_pass * passes / total / 1e9, "unit": UNIT, "cores": threads, "kind": arm.kind,
            "sample": arm.sample_text(passes)}


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return 0
    from mlcompiler_b200 import synth
    case = synth.config_case(2)
    threads = os.cpu_count() or 1
    arm = CpuArm(case, threads)
    # every step = one layer's 32 requests once: a bounded sample of the 22-layer step
    with ThreadPoolExecutor(max_workers=threads) as pool:
        for _ in range(max(args.warmup, 0)):
            arm.run_pass(pool)
        times = [arm.run_pass(pool) for _ in range(max(args.steps, 1))]
    arm.close()
    dt = float(np.mean(times))
    value = case.kv_bytes / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over fp16 KV", "data": "synthetic",
        "config": {"workload": WORKLOAD, "step": "one layer of the 22 (bounded sample), all 32 requests"},
        "tokens_per_s": case.N / (dt * LAYERS),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": arm.kind,
                         "sample": f"one layer of the workload ({case.N} requests, {case.kv_bytes / 1e6:.1f} MB KV) "
                                   f"per step, one request per host thread, {threads} threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from mlcompiler_b200 import Executor, synth
    from mlcompiler_b200.capi import MLC_F16

    rank, world, local = dist_env()
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    # every rank decodes its own 32-request batch (request sharding)
    headroom = 17                                      # tokens the end-to-end loop may append
    lens0 = synth.config_lengths(2, seed=0xBEEF + 2 + 1000 * rank)
    case = synth.make_case(0xBEEF + 2 + 1000 * rank, lens0 + headroom, P=64, fill=False, **synth.SHAPE_A)
    N, H, KVH, D, P = case.N, case.H, case.KVH, case.D, case.P
    cap = case.capacity

    stream = torch.cuda.Stream(device=dev)
    ex = Executor(local, stream=stream.cuda_stream)
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    with torch.cuda.stream(stream):
        k_pools = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16, generator=g) for _ in range(LAYERS)]
        v_pools = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16, generator=g) for _ in range(LAYERS)]
        q_all = torch.randn((LAYERS, N, H, D), device=dev, dtype=torch.float16, generator=g)
        kn_all = torch.randn((LAYERS, N, KVH, D), device=dev, dtype=torch.float16, generator=g)
        vn_all = torch.randn((LAYERS, N, KVH, D), device=dev, dtype=torch.float16, generator=g)
        o_all = torch.zeros((LAYERS, N, H, D), device=dev, dtype=torch.float16)
    stream.synchronize()

    def tables(step):
        """Tables of decode step `step`: requests grow by one token per step (the
        growth wraps every 16 steps so that the contexts stay those of the workload)."""
        lens = (lens0 + (step % 16) + 1).astype(np.uint32)  # length after this step's token is written
        q_pos = lens - 1
        ids = np.array([case.pt_flat[case.pt_off[r] + (int(lens[r]) - 1) // P] for r in range(N)], np.uint32)
        slots = ((lens - 1) % P).astype(np.uint32)
        # a request's table lists only the pages it has reached, like RequestKVState
        pages = (lens.astype(np.int64) + P - 1) // P
        off = np.zeros(N + 1, np.uint32)
        off[1:] = np.cumsum(pages)
        flat = np.concatenate([case.pt_flat[case.pt_off[r]:case.pt_off[r] + pages[r]] for r in range(N)])
        return lens, q_pos, ids, slots, flat.astype(np.uint32), off

    kv_bytes_layer = lambda lens: int(lens.astype(np.int64).sum()) * 2 * KVH * D * 2

    # ---- device-resident arm: planned calls replayed from a CUDA graph ------------------
    lens, q_pos, ids, slots, flat, off = tables(0)
    plan = ex.createPlan(flat, off, lens, q_pos, N, H, KVH, D, P, True, cap, page_ids=ids, slots_in_page=slots)

    def encode_step(fused=True):
        for L in range(LAYERS):
            if fused:   # KV row write + attention of a layer in one launch
                ok = ex.encodePagedDecodeStepPlanned(plan, q_all[L], kn_all[L], vn_all[L], k_pools[L], v_pools[L],
                                                     o_all[L], case.scale, MLC_F16, MLC_F16)
            else:       # attention alone
                ok = ex.encodePagedFlashAttentionPlanned(plan, q_all[L], k_pools[L], v_pools[L], o_all[L], case.scale,
                                                         MLC_F16, MLC_F16)
            assert ok, ex.last_error()

    assert ex.beginForwardPassCB()
    encode_step()
    assert ex.flushForwardPassCB(), ex.last_error()
    assert ex.lastAttentionKernel() == 2, "the TMA / tensor-core kernel did not run"
    assert ex.beginForwardPassCB()
    assert ex.beginCapture(), ex.last_error()
    encode_step()
    graph = ex.endCapture()
    assert ex.beginCapture(), ex.last_error()
    encode_step(fused=False)
    graph_attn = ex.endCapture()

    def barrier():
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_replays(gr, k):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(k):
                gr.launch()
            e1.record(stream)
        stream.synchronize()
        return e0.elapsed_time(e1) * 1e-3

    for _ in range(max(args.warmup, 3)):
        graph.launch()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = ex.launchCount()
    t_step = timed_replays(graph, args.steps)
    gpu_launches = ex.launchCount() - launches0
    barrier()
    # the dominant kernel alone, same timed conditions (22 attention launches per replay)
    for _ in range(3):
        graph_attn.launch()
    stream.synchronize()
    t_attn = timed_replays(graph_attn, args.steps)
    clocks = sampler.stop()
    assert ex.flushForwardPassCB(), ex.last_error()

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    bytes_step_rank = kv_bytes_layer(lens) * LAYERS
    bytes_step_all = reduce_sum(float(bytes_step_rank))
    sec_per_step = reduce_max(t_step) / args.steps
    value = bytes_step_all / sec_per_step / 1e9
    tokens_per_s = N * world / sec_per_step
    # Duration of the dominant kernel. When the timed region is one kernel per layer (the planner kept every
    # request inside a CTA, so the KV row write, attention and merge are a single launch), the region's
    # CUDA-event time divided by its launches IS that kernel's average duration. Otherwise (attention + merge
    # kernel per layer) the attention-only graph, timed the same way right after, gives the pair's duration.
    kernels_per_step = gpu_launches / max(args.steps, 1)
    if abs(kernels_per_step - LAYERS) < 0.5:
        attn_launch_s = t_step / (args.steps * LAYERS)
        launch_timing = "timed region / launches (one fused kernel per layer)"
    else:
        attn_launch_s = t_attn / (args.steps * LAYERS)
        launch_timing = "attention-only graph (attention + merge kernel per layer)"
    achieved = kv_bytes_layer(lens) / attn_launch_s / 1e9
    peak, peak_kind = measured_peak_gbs()

    # ---- end-to-end arm: host buffers, host tables, reference-shaped calls ---------------
    # Per layer one packed row [Q | new K | new V] in pinned host memory and on the device, O back to
    # pinned host memory, all inside the timed region.
    nq, nkv = N * H * D, N * KVH * D
    in_host = torch.randn((LAYERS, nq + 2 * nkv), dtype=torch.float16).pin_memory()
    in_dev = torch.empty((LAYERS, nq + 2 * nkv), device=dev, dtype=torch.float16)
    o_host = torch.zeros((LAYERS, N, H, D), dtype=torch.float16).pin_memory()
    h2d = in_host.numel() * 2
    d2h = o_host.numel() * 2

    # The call sequence INTEGRATION.md recommends to a walker whose activations are host vectors: per step
    # one in-place plan update with the step's host tables and one host-buffer pass call. Inside that call
    # the layers go in a few groups so that the copies overlap the kernels (group g's rows are copied on a
    # copy stream while group g-1 computes, its O rows go back while group g+1 computes). The tables of
    # step s+1 do not depend on the results of step s (every request grows by one row), so they are handed
    # to the library - validated, planned, uploaded, into the other of two plans - while step s still runs.
    e2e_plans = [ex.createPlan(flat, off, lens, q_pos, N, H, KVH, D, P, True, cap, page_ids=ids, slots_in_page=slots)
                 for _ in range(2)]
    pool_ptrs = [ex.pointerArray(k_pools), ex.pointerArray(v_pools)]

    # the 16 table sets the growing requests cycle through, built once: what is timed is handing them
    # to the library (validation, planning, upload), not this script's numpy code
    table_sets = [tables(i) for i in range(16)]

    def plan_for(step):
        lens_s, q_pos_s, ids_s, slots_s, flat_s, off_s = table_sets[step % 16]
        assert e2e_plans[step % 2].update(flat_s, off_s, lens_s, q_pos_s, ids_s, slots_s), ex.last_error()

    def e2e_step(step):
        assert ex.beginForwardPassCB()
        ok = ex.encodePagedDecodePassHost(e2e_plans[step % 2], in_host, in_dev, *pool_ptrs, o_all, o_host, case.scale,
                                          MLC_F16, MLC_F16)                      # all 22 layers, copies included
        assert ok, ex.last_error()
        plan_for(step + 1)          # the next step's tables, while this step runs
        assert ex.flushForwardPassCB(), ex.last_error()      # returns when o_host is complete
        return kv_bytes_layer(table_sets[step % 16][0]) * LAYERS

    first = max(args.warmup, 3)
    plan_for(0)
    for w in range(first):
        e2e_step(w)
    barrier()
    t0 = time.perf_counter()
    e2e_bytes = 0
    for s in range(args.steps):
        e2e_bytes += e2e_step(first + s)
    stream.synchronize()
    t_e2e = time.perf_counter() - t0
    barrier()
    t_e2e_max = reduce_max(t_e2e)
    e2e_value = reduce_sum(float(e2e_bytes)) / t_e2e_max / 1e9

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_baseline_sample(synth.config_case(2), args.cpu_seconds)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "requests_per_gpu": N, "layers": LAYERS, "parallelism": f"request-sharded x{world}",
                       "kv_bytes_per_step": bytes_step_all,
                       "l2": "the step streams 22 layer pools (~0.8 GB per GPU) > 126 MB L2, so no flush between steps"},
            "tokens_per_s": tokens_per_s,
            "pct_of_nominal_8TBs": 100.0 * value / world / 8000.0,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peak_kind,
                         "kernel": "paged_decode_tma_kernel<64,false,unit>" if abs(kernels_per_step - LAYERS) < 0.5
                         else "paged_decode_tma_kernel<64,false,split> + paged_decode_merge_kernel", "bytes_per_launch": kv_bytes_layer(lens),
                         "us_per_launch": attn_launch_s * 1e6, "launch_timing": launch_timing,
                         "attention_only_us_per_layer": t_attn / (args.steps * LAYERS) * 1e6},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": t_e2e_max / args.steps * 1e3},
            "gpu_launches": int(gpu_launches),
            "clocks": clocks,
        }
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line))
    graph.destroy()
    graph_attn.destroy()
    plan.destroy()
    for pl in e2e_plans:
        pl.destroy()
    ex.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="wall-time budget of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
