"""oracle/layer_oracle.c (the walker step's ops around attention) pinned on the reference's own CPU code:
bit for bit against the committed golden vectors (tests/golden/reference_layer_ops.npz, made by
tests/golden/make_layer_golden.py from MLcompiler's quantization.cpp row functions and CpuExecutionBackend
nodes), and live against the reference-linked library where it is present."""
import ctypes as C

import numpy as np
import pytest

from pathlib import Path

GOLDEN = Path(__file__).resolve().parent / "golden" / "reference_layer_ops.npz"
_fp = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


def _bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


@pytest.mark.parametrize("n", [6, 64, 2048, 5632])
def test_elementwise_ops_match_golden_bit_for_bit(oracle_mod, gold, n):
    a, w, y = gold[f"rms_norm/{n}/a"], gold[f"rms_norm/{n}/b"], gold[f"rms_norm/{n}/y"]
    got = oracle_mod.rms_norm_batched(a[None], w, 1e-5)[0]
    assert np.array_equal(_bits(got), _bits(y))
    a, b, y = gold[f"add/{n}/a"], gold[f"add/{n}/b"], gold[f"add/{n}/y"]
    assert np.array_equal(_bits(oracle_mod.add(a, b)), _bits(y))
    a, b, y = gold[f"silu_mul/{n}/a"], gold[f"silu_mul/{n}/b"], gold[f"silu_mul/{n}/y"]
    gate, up, out = oracle_mod.gate_up_split_silu_mul(np.concatenate([a, b])[None], n)
    assert np.array_equal(gate[0], a) and np.array_equal(up[0], b)
    assert np.array_equal(_bits(out[0]), _bits(y))


@pytest.mark.parametrize("kind,cols", [("q4_0", 32), ("q4_0", 64), ("q4_0", 2048), ("q6_k", 256), ("q6_k", 2048)])
def test_quantised_rows_match_golden_bit_for_bit(oracle_mod, gold, kind, cols):
    w, x = gold[f"{kind}/{cols}/w"], gold[f"{kind}/{cols}/x"]
    rows = w.shape[0]
    assert oracle_mod.row_size(kind, cols) == w.shape[1]
    assert np.array_equal(_bits(oracle_mod.dequant_rows(kind, w, rows, cols)), _bits(gold[f"{kind}/{cols}/dequant"]))
    got = oracle_mod.matmul_quant_batched(kind, w, x[None], rows, cols)[0]
    assert np.array_equal(_bits(got), _bits(gold[f"{kind}/{cols}/dot"]))


def test_batched_forms_are_the_row_forms_per_request(oracle_mod):
    from mlcompiler_b200 import synth
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 64)).astype(np.float32)
    w = synth.random_q4_0(rng, 7, 64)
    full = oracle_mod.matmul_quant_batched("q4_0", w, x, 7, 64)
    for n in range(3):
        assert np.array_equal(full[n], oracle_mod.matmul_quant_batched("q4_0", w, x[n:n + 1], 7, 64)[0])
    # and a de-quantise-then-multiply in float64 agrees within fp32 rounding of a 64-term sum
    ref = x.astype(np.float64) @ oracle_mod.dequant_rows("q4_0", w, 7, 64).astype(np.float64).T
    assert np.allclose(full, ref, rtol=1e-5, atol=1e-6)
    g = rng.standard_normal((2, 10)).astype(np.float32)
    gate, up, out = oracle_mod.gate_up_split_silu_mul(g, 4)       # rows 10 > 2 * 4: trailing columns ignored
    assert np.array_equal(gate, g[:, :4]) and np.array_equal(up, g[:, 4:8])
    norm = oracle_mod.rms_norm_batched(g, np.ones(10, np.float32))
    assert np.allclose((norm.astype(np.float64) ** 2).mean(axis=1), 1.0, atol=1e-4)


def test_live_differential_against_the_reference(oracle_mod):
    lib = oracle_mod.ref()
    if lib is None:
        pytest.skip("reference-linked library not available here")
    from mlcompiler_b200 import synth
    rng = np.random.default_rng(77)
    for n in (33, 1000):
        a = rng.standard_normal(n).astype(np.float32)
        b = (1 + 0.2 * rng.standard_normal(n)).astype(np.float32)
        y = np.zeros(n, np.float32)
        assert lib.ref_elementwise_node(0, a.ctypes.data_as(_fp), b.ctypes.data_as(_fp), n, y.ctypes.data_as(_fp)) == 0
        assert np.array_equal(_bits(y), _bits(oracle_mod.rms_norm_batched(a[None], b)[0]))
        assert lib.ref_elementwise_node(1, a.ctypes.data_as(_fp), b.ctypes.data_as(_fp), n, y.ctypes.data_as(_fp)) == 0
        assert np.array_equal(_bits(y), _bits(oracle_mod.gate_up_split_silu_mul(np.concatenate([a, b])[None], n)[2][0]))
    for kind, gen, cols in (("q4_0", synth.random_q4_0, 4096), ("q6_k", synth.random_q6_k, 1024)):
        w = gen(rng, 3, cols)
        x = rng.standard_normal(cols).astype(np.float32)
        got = oracle_mod.matmul_quant_batched(kind, w, x[None], 3, cols)[0]
        for r in range(3):
            row = np.ascontiguousarray(w[r])
            want = getattr(lib, f"ref_dot_{kind}")(row.ctypes.data_as(_u8p), cols, x.ctypes.data_as(_fp))
            assert np.float32(want).view(np.uint32) == got[r].view(np.uint32)
