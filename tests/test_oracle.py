"""Pins of the CPU oracle (no GPU): known-answer vectors of the reference, the committed
golden vectors produced by the reference's own CPU attention, and - where the reference
checkout or its prebuilt library is present - a live differential run against it."""
from pathlib import Path

import numpy as np
import pytest

from mlcompiler_b200 import synth

GOLDEN = Path(__file__).parent / "golden" / "reference_attention.npz"


def contiguous_as_paged(k_tokens, v_tokens, P, rng):
    """Lays [S, KVH, D] rows out through a random page table."""
    S, KVH, D = k_tokens.shape
    pages = (S + P - 1) // P
    cap = pages + 3
    table = rng.permutation(cap)[:pages].astype(np.uint32)
    kp = rng.standard_normal((cap, P, KVH, D)).astype(np.float16)   # unused slots hold noise
    vp = rng.standard_normal((cap, P, KVH, D)).astype(np.float16)
    for s in range(S):
        kp[table[s // P], s % P] = k_tokens[s]
        vp[table[s // P], s % P] = v_tokens[s]
    return kp, vp, table


def golden_cases():
    z = np.load(GOLDEN)
    names = sorted({k.split("/")[0] for k in z.files if k.endswith("/shape")})
    return z, names


def test_tiny_known_answer(oracle_mod):
    """compiler/main.cpp:4026-4031."""
    eye = np.eye(4, dtype=np.float16).reshape(1, 4, 1, 4)
    q = np.array([[[1, 0, 0, 0]]], np.float32)
    for fn in (oracle_mod.paged_attention, lambda *a, **k: oracle_mod.paged_attention_tiled(*a, tile=2, **k)):
        out = fn(q, eye, eye, [0], [0, 1], [4], [3], 1, 1, 4, 4)
        np.testing.assert_allclose(out.ravel(), [0.354661, 0.215113, 0.215113, 0.215113], atol=1e-6)


def test_attention_updates_kv_cache_vector(oracle_mod):
    """tests/test_runtime.cpp:1691-1716: q=[1,0], k=[0.25,0], v=[0.5,1] at position 0 -> [0.5, 1.0]."""
    k = np.array([0.25, 0.0], np.float16).reshape(1, 1, 1, 2)
    v = np.array([0.5, 1.0], np.float16).reshape(1, 1, 1, 2)
    out = oracle_mod.paged_attention(np.array([[[1.0, 0.0]]], np.float32), k, v, [0], [0, 1], [1], [0], 1, 1, 2, 1)
    np.testing.assert_allclose(out.ravel(), [0.5, 1.0], atol=1e-6)


def test_stress_online_tiled_equals_two_pass(oracle_mod):
    """compiler/main.cpp:4033-4065, 4291-4294: scores grow with position, every tile rescales;
    the tiled recurrence must stay within 1e-5 of the two-pass softmax."""
    S, H, KVH, D, P = 128, 32, 4, 64, 64
    rng = np.random.default_rng(42)
    k = np.zeros((S, KVH, D), np.float16)
    k[:] = (0.1 * np.arange(S) / D).astype(np.float16)[:, None, None]
    v = (0.1 * rng.standard_normal((S, KVH, D))).astype(np.float16)
    kp, vp, table = contiguous_as_paged(k, v, P, rng)
    q = np.ones((1, H, D), np.float32)
    args = (q, kp, vp, table, [0, len(table)], [S], [S - 1], H, KVH, D, P)
    two_pass = oracle_mod.paged_attention(*args)
    for tile in (32, 24, 7):
        tiled = oracle_mod.paged_attention_tiled(*args, tile=tile)
        assert np.abs(tiled - two_pass).max() <= 1e-5


def test_empty_and_fully_masked_rows_are_zero(oracle_mod):
    """metal_runtime.mm:2254-2257 and the inv_l guard at 2333."""
    case = synth.make_case(5, [0, 40], 4, 2, 16, P=8)
    out = oracle_mod.paged_attention(case.q, case.k_pool, case.v_pool, case.pt_flat, case.pt_off, case.seq_lens,
                                     case.q_pos, 4, 2, 16, 8)
    assert (out[0] == 0).all() and np.abs(out[1]).max() > 0


def test_split_partials_combine_to_whole(oracle_mod):
    case = synth.make_case(6, [300, 77], 8, 2, 32, P=16)
    a = dict(H=8, KVH=2, D=32, P=16)
    whole = oracle_mod.paged_attention(case.q, case.k_pool, case.v_pool, case.pt_flat, case.pt_off, case.seq_lens,
                                       case.q_pos, **a)
    cuts = [0, 64, 100, 1 << 20]
    parts = [oracle_mod.paged_attention_tiled(case.q, case.k_pool, case.v_pool, case.pt_flat, case.pt_off,
                                              case.seq_lens, case.q_pos, t0=cuts[i], t1=cuts[i + 1], partial=True, **a)
             for i in range(3)]
    comb = oracle_mod.lse_combine(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]))
    assert np.abs(comb - whole).max() <= 2e-6


def test_prefill_is_a_loop_of_causal_steps(oracle_mod):
    """compiler/runtime/operator_backend.cpp:906-968."""
    case = synth.make_case(7, [50], 4, 2, 16, P=8)
    rng = np.random.default_rng(1)
    q = rng.standard_normal((10, 4, 16)).astype(np.float32)
    out = oracle_mod.paged_prefill(q, case.k_pool, case.v_pool, case.pt_flat, case.pt_off, [50], [40], [10], 4, 2, 16, 8)
    for i in (0, 4, 9):
        one = oracle_mod.paged_attention(q[i:i + 1], case.k_pool, case.v_pool, case.pt_flat, case.pt_off, [50],
                                         [40 + i], 4, 2, 16, 8, causal=True)
        assert np.array_equal(out[i], one[0])


def test_oracle_matches_golden_reference_outputs(oracle_mod):
    """The committed outputs of the reference's own RunAttentionCPU (tests/golden/make_golden.py)."""
    z, names = golden_cases()
    assert len(names) >= 6
    rng = np.random.default_rng(0)
    for name in names:
        H, KVH, D, S = (int(x) for x in z[f"{name}/shape"])
        q, k, v, want = z[f"{name}/q"], z[f"{name}/k"], z[f"{name}/v"], z[f"{name}/o"]
        for P in (64, 16):
            kp, vp, table = contiguous_as_paged(k, v, P, rng)
            got = oracle_mod.paged_attention(q[None].astype(np.float32), kp, vp, table, [0, len(table)], [S], [S - 1],
                                             H, KVH, D, P)[0]
            # same fp32 math, different summation order (the reference normalises the weights first)
            assert np.abs(got - want).max() <= 2e-6, name


def test_fp16_converters_match_golden(oracle_mod):
    """float_convert.hpp:14-76 through the reference's own functions (golden) and the subnormal
    known answers of tests/test_runtime.cpp:63-70."""
    z, _ = golden_cases()
    port = oracle_mod.port()
    got = np.array([port.orc_float_to_fp16_ref_scalar(float(x)) for x in z["fp16/x"]], np.uint16)
    assert np.array_equal(got, z["fp16/bits"])
    back = np.array([port.orc_fp16_to_float(int(h)) for h in z["fp16/h"]], np.float32)
    assert np.array_equal(back.view(np.uint32), z["fp16/f"].view(np.uint32))
    assert port.orc_fp16_to_float(0x0001) == pytest.approx(2.0 ** -24, abs=1e-10)
    assert port.orc_fp16_to_float(0x0002) == pytest.approx(2.0 ** -23, abs=1e-10)
    # the round-to-nearest-even encoder agrees with IEEE (numpy) everywhere, and with the
    # reference's scalar encoder except on ties
    xs = z["fp16/x"][np.isfinite(z["fp16/x"])]
    rne = np.array([port.orc_float_to_fp16_rne(float(x)) for x in xs], np.uint16)
    with np.errstate(over="ignore"):
        assert np.array_equal(rne, xs.astype(np.float16).view(np.uint16))


def test_scatter_gather_patterns(oracle_mod):
    """tests/test_paged_kv.cpp:219-267, 404-474 on the oracle itself."""
    cap, P, KVH, D = 16, 8, 4, 16
    p, s, h, d = np.meshgrid(np.arange(cap), np.arange(P), np.arange(KVH), np.arange(D), indexing="ij")
    pool = (p * 100000.0 + s * 1000.0 + h * 10.0 + d).astype(np.float32)
    got = oracle_mod.gather_kv_pages(pool, [7, 2, 11], P, KVH, D, 20)
    for hh, t, dd in ((0, 0, 0), (3, 19, 15), (2, 8, 5)):
        assert got[hh, t, dd] == [7, 2, 11][t // P] * 100000.0 + (t % P) * 1000.0 + hh * 10.0 + dd
    kv, t, d = np.meshgrid(np.arange(KVH), np.arange(11), np.arange(D), indexing="ij")
    src = (kv * 1000.0 + t * 10.0 + d).astype(np.float32)
    storage = np.zeros(8 * P * KVH * D, np.float32)
    oracle_mod.scatter_kv_paged(src, storage, [5, 1], P, KVH, D, 11, 3)
    back = oracle_mod.gather_kv_pages(storage, [5, 1], P, KVH, D, 16)
    expect = np.zeros((KVH, 16, D), np.float32)
    expect[:, 3:14] = src
    assert np.array_equal(back, expect)


def test_live_differential_against_reference(oracle_mod):
    """With the reference library present (built from the MLcompiler checkout, or prebuilt and shipped):
    random cases through ExecutionExecutor::run (and RunAttentionCPU called directly) vs the oracle."""
    lib = oracle_mod.ref()
    if lib is None:
        pytest.skip("reference library not available on this machine")
    rng = np.random.default_rng(2024)
    for H, KVH, D, S in ((32, 4, 64, 300), (8, 8, 32, 17), (32, 8, 128, 65), (6, 2, 20, 9)):
        q = rng.standard_normal((H, D)).astype(np.float16)
        k = rng.standard_normal((S, KVH, D)).astype(np.float16)
        v = rng.standard_normal((S, KVH, D)).astype(np.float16)
        want = oracle_mod.reference_decode(q, k, v, H, KVH, D)
        direct = oracle_mod.reference_decode(q, k, v, H, KVH, D, direct=True)
        assert np.array_equal(want, direct)
        kp, vp, table = contiguous_as_paged(k, v, 16, rng)
        got = oracle_mod.paged_attention(q[None].astype(np.float32), kp, vp, table, [0, len(table)], [S], [S - 1],
                                         H, KVH, D, 16)[0]
        assert np.abs(got - want).max() <= 2e-6
