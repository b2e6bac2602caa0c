#!/usr/bin/env python3
"""Generates tests/golden/reference_attention.npz from MLcompiler's own CPU attention.

Run where the MLcompiler checkout is present (MLC_REFERENCE_ROOT, default: a directory `reference` beside this repository): it builds
oracle/_ref/libref_attention.so from the reference's unmodified sources
(oracle/build_ref.py) and records, for a set of seeded cases, the inputs and the
output of the reference's executor-CPU attention path
(ExecutionExecutor::run -> CpuExecutionBackend -> RunAttentionCPU,
compiler/runtime/attention_cpu.cpp:272-478). The file is small and committed, so the
oracle can be checked against the reference on machines that have no checkout.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402

# (name, H, KVH, D, S, seed, distribution)
CASES = [
    ("tinyllama_s96", 32, 4, 64, 96, 11, "uniform"),     # tests/test_paged_flash.cpp:259-266 shape
    ("tinyllama_s200", 32, 4, 64, 200, 12, "normal"),    # benchmark head shape, 4 pages
    ("gqa8x2_s20", 8, 2, 64, 20, 13, "uniform"),         # FourRequestsGQA shape
    ("mha_s33", 4, 4, 32, 33, 14, "normal"),
    ("wide_s70", 32, 8, 128, 70, 15, "normal"),          # shape B
    ("single_token", 32, 4, 64, 1, 16, "normal"),
]


def make_inputs(H, KVH, D, S, seed, dist):
    rng = np.random.default_rng(seed)
    draw = (lambda shape: rng.uniform(-0.5, 0.5, shape)) if dist == "uniform" else rng.standard_normal
    q = draw((H, D)).astype(np.float16)
    k = draw((S, KVH, D)).astype(np.float16)
    v = draw((S, KVH, D)).astype(np.float16)
    return q, k, v


def main():
    if oracle.ref() is None:
        raise SystemExit("the reference checkout is not available: cannot generate golden vectors")
    out = {}
    for name, H, KVH, D, S, seed, dist in CASES:
        q, k, v = make_inputs(H, KVH, D, S, seed, dist)
        o = oracle.reference_decode(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), H, KVH, D)
        out[f"{name}/q"], out[f"{name}/k"], out[f"{name}/v"], out[f"{name}/o"] = q, k, v, o.astype(np.float32)
        out[f"{name}/shape"] = np.array([H, KVH, D, S], np.int64)
    # the reference's scalar fp16 encoder on a spread of inputs (float_convert.hpp:57-76)
    lib = oracle.ref()
    rng = np.random.default_rng(99)
    xs = np.concatenate([rng.standard_normal(512).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 100.0, 7e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 5.96e-8, 6.1e-5, np.inf, -np.inf], np.float32)])
    out["fp16/x"] = xs
    out["fp16/bits"] = np.array([lib.ref_float_to_fp16(float(x)) for x in xs], np.uint16)
    hs = np.arange(0, 65536, 7, dtype=np.uint16)
    out["fp16/h"] = hs
    out["fp16/f"] = np.array([lib.ref_fp16_to_float(int(h)) for h in hs], np.float32)
    # the reference's rotary coefficients and rotation (quantization.cpp:773-823)
    import ctypes as C
    fp = C.POINTER(C.c_float)
    lib.ref_compute_rotary.restype = C.c_size_t
    lib.ref_compute_rotary.argtypes = [C.c_size_t, C.c_size_t, C.c_float, C.c_float, fp, fp]
    lib.ref_apply_rotary.restype = None
    lib.ref_apply_rotary.argtypes = [fp, fp, fp, C.c_size_t, C.c_size_t, C.c_size_t]
    positions = np.array([0, 1, 2, 17, 511, 2047, 32767], np.int64)
    for rd, base, scale in ((64, 10000.0, 1.0), (128, 500000.0, 1.0), (32, 0.0, 0.0), (64, 10000.0, 0.25)):
        cos = np.zeros((len(positions), rd // 2), np.float32)
        sin = np.zeros_like(cos)
        for i, pos in enumerate(positions):
            n = lib.ref_compute_rotary(int(pos), rd, base, scale, cos[i].ctypes.data_as(fp), sin[i].ctypes.data_as(fp))
            assert n == rd // 2
        key = f"rope/{rd}_{base:g}_{scale:g}"
        out[key + "/cos"], out[key + "/sin"] = cos, sin
    out["rope/positions"] = positions
    # one rotated head per position: head_dim 64, rotary_dim 64 and a partial rotary_dim 32
    x = rng.standard_normal((len(positions), 64)).astype(np.float32)
    out["rope/x"] = x
    for rd in (64, 32):
        y = x.copy()
        cs = out["rope/64_10000_1/cos"] if rd == 64 else out["rope/32_0_0/cos"]
        sn = out["rope/64_10000_1/sin"] if rd == 64 else out["rope/32_0_0/sin"]
        for i in range(len(positions)):
            lib.ref_apply_rotary(y[i].ctypes.data_as(fp), np.ascontiguousarray(cs[i]).ctypes.data_as(fp),
                                 np.ascontiguousarray(sn[i]).ctypes.data_as(fp), rd // 2, 64, rd)
        out[f"rope/y{rd}"] = y
    path = Path(__file__).with_name("reference_attention.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
