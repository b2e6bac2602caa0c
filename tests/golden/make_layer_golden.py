#!/usr/bin/env python3
"""Generates tests/golden/reference_layer_ops.npz: the ops around attention in the reference walker's step
(RMSNorm, SiLU(gate) * up, add, Q4_0 and Q6_K rows), computed by MLcompiler's own CPU code.

Run in the container that has the reference checkout: oracle/build_ref.py compiles the reference's unmodified
sources, and the harness calls quantization.cpp's row functions directly and runs one-node Norm / FeedForward /
Add graphs through CpuExecutionBackend (oracle/ref_driver.cpp). The file is small and committed, so that
oracle/layer_oracle.c can be pinned on machines without the checkout.

    python tests/golden/make_layer_golden.py
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from mlcompiler_b200 import synth  # noqa: E402

_fp = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)


def main():
    lib = oracle.ref()
    if lib is None:
        raise SystemExit("the reference checkout is not available: cannot generate golden vectors")
    rng = np.random.default_rng(2024)
    out = {}
    # element-wise nodes at a few lengths (2048 = TinyLlama hidden size, 5632 = its FFN width)
    for n in (6, 64, 2048, 5632):
        a = (rng.standard_normal(n) * 1.5).astype(np.float32)
        b = rng.standard_normal(n).astype(np.float32)
        w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        for kind, name, second in ((0, "rms_norm", w), (1, "silu_mul", b), (2, "add", b)):
            y = np.zeros(n, np.float32)
            rc = lib.ref_elementwise_node(kind, a.ctypes.data_as(_fp), second.ctypes.data_as(_fp), n, y.ctypes.data_as(_fp))
            assert rc == 0, (name, n, rc)
            out[f"{name}/{n}/a"], out[f"{name}/{n}/b"], out[f"{name}/{n}/y"] = a, second, y
    # quantised rows: de-quantised values and dot products with an activation vector
    for kind, gen, cols_list in (("q4_0", synth.random_q4_0, (32, 64, 2048)), ("q6_k", synth.random_q6_k, (256, 2048))):
        for cols in cols_list:
            rows = 5
            w = gen(rng, rows, cols)
            assert w.shape[1] == getattr(lib, f"ref_row_size_{kind}")(cols)
            x = rng.standard_normal(cols).astype(np.float32)
            deq = np.zeros((rows, cols), np.float32)
            dots = np.zeros(rows, np.float32)
            for r in range(rows):
                row = np.ascontiguousarray(w[r])
                getattr(lib, f"ref_dequant_{kind}")(row.ctypes.data_as(_u8p), cols, deq[r].ctypes.data_as(_fp))
                dots[r] = getattr(lib, f"ref_dot_{kind}")(row.ctypes.data_as(_u8p), cols, x.ctypes.data_as(_fp))
            out[f"{kind}/{cols}/w"], out[f"{kind}/{cols}/x"] = w, x
            out[f"{kind}/{cols}/dequant"], out[f"{kind}/{cols}/dot"] = deq, dots
    path = Path(__file__).with_name("reference_layer_ops.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
