#!/usr/bin/env python3
"""Benchmark of the paged decode-attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-secondary]

Workload (N = 1): continuous-batching decode over 22 layers of the TinyLlama head
shape (32 q heads / 4 KV heads, d = 64, fp16 KV, 64-token pages), 32 requests with
context lengths seeded uniform in [64, 2048], non-contiguous random page tables
over per-layer pools sized to the total pages + 10 %. One step = for every layer:
write one new K/V row per request into the pool, then run attention. The 22 layers
are independent layer pools with all inputs resident when the step starts.

`value` is KV GB/s with everything resident in HBM: one call of the whole-pass entry point
(mlc_encode_paged_decode_pass_planned: every layer's row write + attention in ONE launch whose
work items are dealt to the SMs across layers), replayed from a CUDA graph and timed with CUDA
events on the launching stream. The same step issued layer by layer - one launch per layer, each
ordered behind the one before, which is what a transformer that feeds layer l into layer l + 1
must do - and in the reference walker's own call order (scatter K, scatter V, attention with host
tables per layer) is timed the same way and reported under `call_forms`.
`e2e` is the same metric through the C ABI with host buffers: every step one host-buffer pass call
(Q and the new K/V rows of all layers live in pinned host memory, the attention output lands in
pinned host memory) and one in-place plan update that hands over the NEXT step's page tables /
lengths / positions / (page, slot) pairs as host arrays (they grow by one token per step, as in
serving, and do not depend on this step's results) while this step runs; the flush returns when
the output is complete in host memory. With N > 1 (torchrun, one rank per GPU) every rank runs a
32-request batch of the same context lengths over its own pools: request sharding, no collective on
the data path (weak scaling). `secondary` carries the other workloads: cfg3 (long contexts; with
N > 1 split by KV sequence over the ranks through the peer-memory exchange kernel and checked
against one GPU), cfg4 (wide GQA), cfg5 (chunked prefill on tcgen05) and model_step (the whole walker step
of a 1.1B-shaped decoder with synthetic Q4_0 / Q6_K weights through the paged executor: tokens per second).

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
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel on this workload, from an
# `ncu --set full` capture (a profiler run, never the source of a timing). `commit` is the revision of the
# kernel source the capture ran on; `kv_bytes` the algorithmic bytes of the captured launch, so that the
# figure can be scaled to the launch the bench times (traffic grows in proportion to the KV bytes read).
NCU_TRAFFIC = {
    "kernel": "paged_decode_pass_kernel<64,false>",
    "dram_bytes": 834_393_088,        # 828,432,384 read + 5,960,704 written
    "kv_bytes": 813_959_168,
    "commit": "0e86983",
}


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
        self.samples, self.times, self.reasons, self.stop_flag = [], [], set(), False
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
        self.times.append(time.time())
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
            time.sleep(0.002)

    def median_between(self, t0, t1):
        """Median SM clock of the samples taken between two host time stamps (None without a sample)."""
        n = min(len(self.samples), len(self.times))
        v = [self.samples[i] for i in range(n) if t0 <= self.times[i] <= t1]
        return float(np.median(v)) if v else None

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
def time_blocks(stream, launch, n_blocks, per_block):
    """CUDA events on the launching stream around each of n_blocks runs of per_block launches;
    returns the seconds of every block and the host time stamps around it."""
    import torch
    out = []
    for _ in range(n_blocks):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record(stream)
        for _ in range(per_block):
            launch()
        e1.record(stream)
        stream.synchronize()
        out.append((e0.elapsed_time(e1) * 1e-3, t0, time.time()))
    return out


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    import bench_more
    from mlcompiler_b200 import Executor, synth
    from mlcompiler_b200.capi import MLC_F16

    rank, world, local = dist_env()
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    # Every rank decodes a 32-request batch of its own (request sharding) with the SAME context lengths and
    # page tables on every rank, so that the scaling figure measures the machine and not the draw; the pool
    # contents differ per rank.
    headroom = 17                                      # tokens the end-to-end loop may append
    lens0 = synth.config_lengths(2)
    case = synth.make_case(0xBEEF + 2, lens0 + headroom, P=64, fill=False, **synth.SHAPE_A)
    N, H, KVH, D, P = case.N, case.H, case.KVH, case.D, case.P
    cap = case.capacity

    stream = torch.cuda.Stream(device=dev)
    ex = Executor(local, stream=stream.cuda_stream)
    env = bench_more.Env(ex, stream, dev, rank, world)
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    with torch.cuda.stream(stream):
        k_pools = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16, generator=g) for _ in range(LAYERS)]
        v_pools = [torch.randn((cap, P, KVH, D), device=dev, dtype=torch.float16, generator=g) for _ in range(LAYERS)]
        q_all = torch.randn((LAYERS, N, H, D), device=dev, dtype=torch.float16, generator=g)
        kn_all = torch.randn((LAYERS, N, KVH, D), device=dev, dtype=torch.float16, generator=g)
        vn_all = torch.randn((LAYERS, N, KVH, D), device=dev, dtype=torch.float16, generator=g)
        o_all = torch.zeros((LAYERS, N, H, D), device=dev, dtype=torch.float16)
        o_chk = torch.zeros((LAYERS, N, H, D), device=dev, dtype=torch.float16)
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

    # ---- device-resident arm: planned calls replayed from CUDA graphs ---------------------
    lens, q_pos, ids, slots, flat, off = tables(0)
    plan = ex.createPlan(flat, off, lens, q_pos, N, H, KVH, D, P, True, cap, page_ids=ids, slots_in_page=slots)
    ptr = ex.pointerArray
    pass_ptrs = [ptr(list(q_all)), ptr(list(kn_all)), ptr(list(vn_all)), ptr(k_pools), ptr(v_pools), ptr(list(o_all))]

    def encode_pass():          # the whole step in one call: one launch when the plan allows it
        assert ex.encodePagedDecodePassPlanned(plan, *pass_ptrs, case.scale, MLC_F16, MLC_F16), ex.last_error()

    def encode_layers():        # layer by layer, each launch ordered behind the one before
        for L in range(LAYERS):
            assert ex.encodePagedDecodeStepPlanned(plan, q_all[L], kn_all[L], vn_all[L], k_pools[L], v_pools[L],
                                                   o_chk[L], case.scale, MLC_F16, MLC_F16), ex.last_error()

    def encode_reference_order():   # what an unchanged reference walker calls per layer (batched_walker.cpp:299-331)
        for L in range(LAYERS):
            assert ex.encodeScatterKVPagedBatched(k_pools[L], ids, slots, P, KVH, D, N, kn_all[L], cap), ex.last_error()
            assert ex.encodeScatterKVPagedBatched(v_pools[L], ids, slots, P, KVH, D, N, vn_all[L], cap), ex.last_error()
            assert ex.encodePagedFlashAttention(q_all[L], k_pools[L], v_pools[L], o_chk[L], flat, off, lens, q_pos, N, H,
                                                KVH, D, P, True, case.scale, MLC_F16, MLC_F16, cap), ex.last_error()

    graphs, launches_per_step = {}, {}
    for name, fn in (("whole_pass", encode_pass), ("layer_by_layer", encode_layers)):
        assert ex.beginForwardPassCB()
        l0 = ex.launchCount()
        fn()
        launches_per_step[name] = ex.launchCount() - l0
        assert ex.flushForwardPassCB(), ex.last_error()
        assert ex.lastAttentionKernel() == 2, "the TMA / tensor-core kernel did not run"
        assert ex.beginForwardPassCB()
        assert ex.beginCapture(), ex.last_error()
        fn()
        graphs[name] = ex.endCapture()
        assert ex.flushForwardPassCB(), ex.last_error()
    torch.cuda.synchronize()
    agree = float((o_all.float() - o_chk.float()).abs().max().item())
    assert agree <= 2e-3, f"whole-pass and layer-by-layer outputs differ by {agree}"

    bytes_step_rank = kv_bytes_layer(lens) * LAYERS
    bytes_step_all = env.reduce(float(bytes_step_rank), "sum")
    peak, peak_kind = measured_peak_gbs()

    # ---- the timed region of the contract: W warm-up steps, then exactly K steps between barriers --------
    warm = max(args.warmup, 3)
    headline = graphs["whole_pass"]
    assert ex.beginForwardPassCB()
    for _ in range(warm):
        headline.launch()
    env.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    n_blocks = min(10, args.steps)
    sizes = [args.steps // n_blocks + (1 if i < args.steps % n_blocks else 0) for i in range(n_blocks)]
    l0 = ex.launchCount()
    blocks = []
    for sz in sizes:
        blocks += time_blocks(stream, headline.launch, 1, sz)
    gpu_launches = ex.launchCount() - l0
    env.barrier()
    t_step = sum(b[0] for b in blocks)
    sec_per_step = env.reduce(t_step, "max") / args.steps
    value = bytes_step_all / sec_per_step / 1e9
    tokens_per_s = N * world / sec_per_step

    # ---- distribution: >= 200 replays of every call form in blocks, median / min / max, clock per block -----
    def distribution(launch, per_block, n=10):
        for _ in range(3):
            launch()
        stream.synchronize()
        bl = time_blocks(stream, launch, n, per_block)
        us = np.array([b[0] / per_block * 1e6 for b in bl])
        mhz = [sampler.median_between(b[1], b[2]) for b in bl]
        return {"replays": n * per_block, "blocks": n, "us_per_step_median": float(np.median(us)),
                "us_per_step_min": float(us.min()), "us_per_step_max": float(us.max()),
                "sm_mhz_per_block": mhz}

    def form(dist_stats, launches, note):
        us = dist_stats["us_per_step_median"]
        gbs = bytes_step_rank / us / 1e3
        return {"kv_gbps": gbs, "frac_of_peak": gbs / peak, "launches_per_step": launches, **dist_stats, "what": note}

    per_block = max(20, (200 + 9) // 10)

    def reference_order_step():
        assert ex.beginForwardPassCB()
        encode_reference_order()

    def measure_forms():
        out = {}
        out["whole_pass"] = form(distribution(graphs["whole_pass"].launch, per_block), launches_per_step["whole_pass"],
                                 "mlc_encode_paged_decode_pass_planned: all layers in one call (layers independent by contract)")
        out["layer_by_layer"] = form(distribution(graphs["layer_by_layer"].launch, per_block), launches_per_step["layer_by_layer"],
                                     "mlc_encode_paged_decode_step_planned per layer (row write fused into attention), every "
                                     "launch ordered behind the previous one; us / launches is a throughput interval under "
                                     "programmatic dependent launch, not a kernel duration")
        assert ex.flushForwardPassCB(), ex.last_error()
        assert ex.beginForwardPassCB()
        l0 = ex.launchCount()
        encode_reference_order()
        ref_launches = ex.launchCount() - l0
        assert ex.flushForwardPassCB(), ex.last_error()
        out["reference_call_order"] = form(distribution(reference_order_step, per_block), ref_launches,
                                           "what an unchanged reference walker calls: per layer encodeScatterKVPagedBatched (K), "
                                           "(V), encodePagedFlashAttention with host tables (batched_walker.cpp:299-331); direct "
                                           "calls, no CUDA graph, host time of the calls included")
        return out

    # (--no-forms: a short run for a profiler's launch list - the timed region and the e2e leg only)
    forms = None if args.no_forms else measure_forms()
    assert ex.flushForwardPassCB(), ex.last_error()
    clocks = sampler.stop()

    # the dominant kernel of the timed region and its duration
    one_launch = launches_per_step["whole_pass"] == 1
    if one_launch:
        kernel = "paged_decode_pass_kernel<64,false>"
        bytes_per_launch = bytes_step_rank
        us_per_launch = t_step / args.steps * 1e6
        launch_timing = ("CUDA events around back-to-back graph replays / replays; one kernel per step, so this is the "
                         "launch-to-launch interval of that kernel (its duration plus what the next launch cannot overlap)")
    else:
        kernel = "paged_decode_tma_kernel<64,false,unit>"
        bytes_per_launch = kv_bytes_layer(lens)
        us_per_launch = t_step / args.steps / LAYERS * 1e6
        launch_timing = "timed region / launches: a throughput interval under programmatic dependent launch, not a kernel duration"
    achieved = bytes_per_launch / us_per_launch / 1e3
    traffic = None
    if NCU_TRAFFIC["kernel"] == kernel:
        traffic = int(NCU_TRAFFIC["dram_bytes"] * (bytes_per_launch / NCU_TRAFFIC["kv_bytes"]))

    # ---- end-to-end arm: host buffers, host tables -----------------------------------------
    # Per layer one packed row [Q | new K | new V] in pinned host memory, O in pinned host memory, all inside
    # the timed region: per step one in-place plan update with the step's host tables and one host-buffer
    # pass call. The tables of step s+1 do not depend on the results of step s (every request grows by one
    # row), so they are handed to the library - validated, planned, uploaded, into the other of two plans -
    # while step s still runs.
    nq, nkv = N * H * D, N * KVH * D
    in_host = torch.randn((LAYERS, nq + 2 * nkv), dtype=torch.float16).pin_memory()
    in_dev = torch.empty((LAYERS, nq + 2 * nkv), device=dev, dtype=torch.float16)
    o_host = torch.zeros((LAYERS, N, H, D), dtype=torch.float16).pin_memory()
    h2d = in_host.numel() * 2
    d2h = o_host.numel() * 2
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
                                          MLC_F16, MLC_F16)                      # all 22 layers, transfers included
        assert ok, ex.last_error()
        plan_for(step + 1)          # the next step's tables, while this step runs
        assert ex.flushForwardPassCB(), ex.last_error()      # returns when o_host is complete
        return kv_bytes_layer(table_sets[step % 16][0]) * LAYERS

    first = max(args.warmup, 3)
    plan_for(0)
    l0 = ex.launchCount()
    for w in range(first):
        e2e_step(w)
    e2e_launches_per_step = (ex.launchCount() - l0) / first
    env.barrier()
    t0 = time.perf_counter()
    e2e_bytes = 0
    e2e_times = []
    for s in range(args.steps):
        ts = time.perf_counter()
        e2e_bytes += e2e_step(first + s)
        e2e_times.append(time.perf_counter() - ts)
    stream.synchronize()
    t_e2e = time.perf_counter() - t0
    env.barrier()
    t_e2e_max = env.reduce(t_e2e, "max")
    e2e_value = env.reduce(float(e2e_bytes), "sum") / t_e2e_max / 1e9
    # the last end-to-end result checked against the device-resident per-layer path on the same rows
    last = first + args.steps - 1
    with torch.cuda.stream(stream):
        in_dev.copy_(in_host, non_blocking=True)
    stream.synchronize()
    chk_plan = ex.createPlan(*[table_sets[last % 16][i] for i in (4, 5, 0, 1)], N, H, KVH, D, P, True, cap,
                             page_ids=table_sets[last % 16][2], slots_in_page=table_sets[last % 16][3])
    assert ex.beginForwardPassCB()
    for L in range(LAYERS):
        assert ex.encodePagedDecodeStepPlanned(chk_plan, in_dev[L, :nq], in_dev[L, nq:nq + nkv], in_dev[L, nq + nkv:],
                                               k_pools[L], v_pools[L], o_chk[L], case.scale, MLC_F16, MLC_F16), ex.last_error()
    assert ex.flushForwardPassCB(), ex.last_error()
    e2e_err = float((o_chk.cpu().float() - o_host.float()).abs().max().item())
    chk_plan.destroy()

    secondary = None
    if not args.no_secondary:
        secondary = {}
        long_cfg3 = lambda e, steps, warmup: bench_more.run_cfg3(e, steps=steps, warmup=warmup, check=False, seq_len=262144)
        model_step = lambda e, steps, warmup: bench_more.run_model(e, steps=30, warmup=warmup)
        for name, fn in (("cfg3", bench_more.run_cfg3), ("cfg3_262144_tokens", long_cfg3), ("cfg4", bench_more.run_cfg4),
                         ("cfg5", bench_more.run_cfg5), ("model_step", model_step)):
            try:
                r = fn(env, steps=200, warmup=5)
            except Exception as e:            # a secondary workload must not take the headline line down
                r = {"error": f"{type(e).__name__}: {e}"}
            if r is not None:
                secondary[name] = {k: r[k] for k in r if k in ("metric", "value", "unit", "ms_per_step", "us_per_step", "scaling",
                                                                "config", "roofline", "gpu_launches", "split_vs_one_gpu",
                                                                "tokens_per_s", "error", "ms_per_step_median_min_max",
                                                                "bytes_per_step", "launches_per_step", "prefill", "served")}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_baseline_sample(synth.config_case(2), args.cpu_seconds)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "requests_per_gpu": N, "layers": LAYERS, "parallelism": f"request-sharded x{world}",
                       "kv_bytes_per_step": bytes_step_all,
                       "call": "mlc_encode_paged_decode_pass_planned (whole pass, CUDA-graph replay)",
                       "l2": "the step streams 22 layer pools (~0.8 GB per GPU) > 126 MB L2, so no flush between steps",
                       "same_lengths_on_every_rank": True},
            "tokens_per_s": tokens_per_s,
            "pct_of_nominal_8TBs": 100.0 * value / world / 8000.0,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_capture": NCU_TRAFFIC, "peak_source": peak_kind,
                         "kernel": kernel, "bytes_per_launch": bytes_per_launch, "us_per_launch": us_per_launch,
                         "launch_timing": launch_timing},
            "timing": {"timed_region_blocks": [b[0] / sz * 1e6 for b, sz in zip(blocks, sizes)],
                       "timed_region_block_sizes": sizes, "unit": "us per step"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": t_e2e_max / args.steps * 1e3,
                    "ms_per_step_median": float(np.median(e2e_times)) * 1e3,
                    "launches_per_step": e2e_launches_per_step,
                    "max_abs_vs_device_path": e2e_err,
                    "how": ("one launch per step reads the rows from pinned host memory and writes O into it"
                            if e2e_launches_per_step < 1.5 else "copies in, launches and copies out pipelined over groups of layers")},
            "gpu_launches": int(gpu_launches),
            "clocks": clocks,
        }
        if forms is not None:
            line["call_forms"] = forms
        if secondary is not None:
            line["secondary"] = secondary
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line))
    for gph in graphs.values():
        gph.destroy()
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
    ap.add_argument("--no-secondary", action="store_true", help="skip the cfg3 / cfg4 / cfg5 workloads")
    ap.add_argument("--no-forms", action="store_true", help="skip the per-call-form distributions (short run for a profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
