"""QKV split + rotary + cast: the CPU restatement against the reference's own rotary code (golden
vectors made by tests/golden/make_golden.py from computeRotaryCoefficients / applyRotaryEmbedding,
compiler/runtime/quantization.cpp:773-823), and the host entry point of the library against both."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import oracle

GOLDEN = Path(__file__).parent / "golden" / "reference_attention.npz"
CONFIGS = ((64, 10000.0, 1.0), (128, 500000.0, 1.0), (32, 0.0, 0.0), (64, 10000.0, 0.25))


@pytest.fixture(scope="module")
def z():
    return np.load(GOLDEN)


@pytest.mark.parametrize("rd,base,scale", CONFIGS)
def test_rotary_coefficients_match_reference_bit_for_bit(z, rd, base, scale):
    key = f"rope/{rd}_{base:g}_{scale:g}"
    for i, pos in enumerate(z["rope/positions"]):
        c, s = oracle.compute_rotary(int(pos), rd, base, scale)
        assert np.array_equal(c.view(np.uint32), z[key + "/cos"][i].view(np.uint32))
        assert np.array_equal(s.view(np.uint32), z[key + "/sin"][i].view(np.uint32))


@pytest.mark.parametrize("rd,key", [(64, "rope/64_10000_1"), (32, "rope/32_0_0")])
def test_rotation_matches_reference_bit_for_bit(z, rd, key):
    x = z["rope/x"]                       # [positions, 64]: one head of 64 per position
    n = x.shape[0]
    qkv = np.concatenate([x, x, x], axis=1)  # H = KVH = 1, D = 64
    q, k, v, k16, v16 = oracle.qkv_split_rope_cast(qkv, z[key + "/cos"], z[key + "/sin"], 1, 1, 64, rd)
    want = z[f"rope/y{rd}"]
    assert np.array_equal(q.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(k.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(v, x)           # V is only split, never rotated
    assert np.array_equal(k16, want.astype(np.float16).view(np.uint16))   # numpy casts RNE, like MSL half()
    assert np.array_equal(v16, x.astype(np.float16).view(np.uint16))
    assert n == len(z["rope/positions"])


def test_split_uses_row_stride_and_offsets():
    # mm:7942-7961: q at offset 0, k at q_rows, v at q_rows + k_rows of a row of qkv_rows floats
    H, KVH, D = 4, 2, 8
    rng = np.random.default_rng(3)
    qkv = rng.standard_normal((3, H * D + 2 * KVH * D + 6)).astype(np.float32)   # 6 floats of padding per row
    q, k, v, _, _ = oracle.qkv_split_rope_cast(qkv, np.zeros((3, 0), np.float32), np.zeros((3, 0), np.float32),
                                               H, KVH, D, 0)
    assert np.array_equal(q, qkv[:, :32]) and np.array_equal(k, qkv[:, 32:48]) and np.array_equal(v, qkv[:, 48:64])


def test_library_host_rotary_matches_reference(z):
    from mlcompiler_b200 import capi
    lib = capi.load_library()
    fp = C.POINTER(C.c_float)
    lib.mlc_compute_rotary_coefficients.restype = C.c_int
    lib.mlc_compute_rotary_coefficients.argtypes = [C.c_size_t, C.c_size_t, C.c_float, C.c_float, fp, fp]
    for rd, base, scale in CONFIGS:
        key = f"rope/{rd}_{base:g}_{scale:g}"
        for i, pos in enumerate(z["rope/positions"]):
            c, s = np.zeros(rd // 2, np.float32), np.zeros(rd // 2, np.float32)
            assert lib.mlc_compute_rotary_coefficients(int(pos), rd, base, scale, c.ctypes.data_as(fp),
                                                       s.ctypes.data_as(fp)) == 0
            assert np.array_equal(c.view(np.uint32), z[key + "/cos"][i].view(np.uint32))
            assert np.array_equal(s.view(np.uint32), z[key + "/sin"][i].view(np.uint32))
