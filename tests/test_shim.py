"""The MLcompiler-side binding, compiled: include/mlc_b200_shim.cpp defines the paged-attention members
of mlc::runtime::MetalExecutor (compiler/runtime/metal_runtime.hpp:510-547, 619-703) on the C ABI, and
tests/shim/shim_driver.cpp is a caller written against the reference's header only.

CPU part: both compile with -Wall -Wextra -Werror against the unmodified reference header and link with
libmlc_b200.so (skipped when the MLcompiler checkout is absent); without a CUDA device the driver reports
the executor as unavailable instead of computing anything. GPU part: the driver makes the walker's calls
for one decode step (scatter K, scatter V, attention, flush; compiler/runtime/batched_walker.cpp:299-331)
through the C++ class, and the results are compared with the oracle.
"""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from mlcompiler_b200 import synth
from tests.util import assert_attention_close

sys.path.insert(0, str(Path(__file__).resolve().parent / "shim"))
import build_shim  # noqa: E402


def _binary():
    import mlcompiler_b200
    mlcompiler_b200.load_library(build_if_missing=True)
    b = build_shim.build()
    if b is None:
        pytest.skip("MLcompiler checkout absent and no shim driver built earlier")
    return b


def _write_case(case, path):
    with open(path, "wb") as f:
        for a in (case.q.astype(np.float32), case.k_new, case.v_new, case.k_pool, case.v_pool, case.pt_flat,
                  case.pt_off, case.seq_lens, case.q_pos, case.page_ids, case.slots):
            f.write(np.ascontiguousarray(a).tobytes())


def _run(binary, case, tmp_path):
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    _write_case(case, inp)
    args = [str(binary), str(inp), str(out)] + [str(int(v)) for v in
                                                (case.N, case.H, case.KVH, case.D, case.P, case.capacity, case.pt_flat.size)]
    return subprocess.run(args, capture_output=True, text=True, timeout=300), out


def test_shim_compiles_against_the_reference_header_and_needs_a_device(tmp_path):
    if build_shim.reference_root() is None:
        pytest.skip("MLcompiler checkout absent")
    binary = _binary()
    assert binary.exists()
    import torch
    if torch.cuda.is_available():
        return
    # no CUDA device: the executor says so; nothing is computed on the host instead
    res, out = _run(binary, synth.make_case(1, [5], 4, 2, 64), tmp_path)
    assert res.returncode == 1 and "isAvailable" in res.stderr, res.stderr
    assert not out.exists()


CASES = [
    ("cfg1", lambda: synth.config_case(1)),
    ("ragged", lambda: synth.make_case(21, [1, 63, 64, 65, 700, 2048, 129], **synth.SHAPE_A)),
    ("wide", lambda: synth.make_case(22, [300, 1, 1000], **synth.SHAPE_B)),
]


@pytest.mark.gpu
@pytest.mark.parametrize("name,build", CASES, ids=[c[0] for c in CASES])
def test_walker_call_order_through_the_cpp_class(oracle_mod, tmp_path, name, build):
    binary = _binary()
    case = build()
    res, out = _run(binary, case, tmp_path)
    assert res.returncode == 0, res.stderr + res.stdout
    raw = np.fromfile(out, dtype=np.uint8)
    q_elems = case.N * case.H * case.D
    pool_elems = case.k_pool.size
    o = raw[:q_elems * 4].view(np.float32).reshape(case.N, case.H, case.D)
    o2 = raw[q_elems * 4:2 * q_elems * 4].view(np.float32).reshape(case.N, case.H, case.D)
    off = 2 * q_elems * 4
    kp = raw[off:off + pool_elems * 2].view(np.uint16)
    vp = raw[off + pool_elems * 2:off + pool_elems * 4].view(np.uint16)
    gathered = raw[off + pool_elems * 4:].view(np.uint16)

    want_k = case.k_pool.view(np.uint16).copy().reshape(-1)
    want_v = case.v_pool.view(np.uint16).copy().reshape(-1)
    oracle_mod.scatter_kv_paged_batched_f16(case.k_new, want_k, case.page_ids, case.slots, case.P, case.KVH, case.D)
    oracle_mod.scatter_kv_paged_batched_f16(case.v_new, want_v, case.page_ids, case.slots, case.P, case.KVH, case.D)
    assert np.array_equal(kp, want_k) and np.array_equal(vp, want_v), "KV scatter through the shim is not bit-exact"
    want = oracle_mod.paged_attention(case.q.astype(np.float32), want_k, want_v, case.pt_flat, case.pt_off,
                                      case.seq_lens, case.q_pos, case.H, case.KVH, case.D, case.P, scale=case.scale)
    assert_attention_close(o, want)
    assert_attention_close(o2, want)
    # gatherKVPages of request 0: [KVH, S0, D] from the pool after the scatter
    S0 = int(case.seq_lens[0])
    rows = want_k.reshape(case.capacity, case.P, case.KVH, case.D)[case.pt_flat[case.pt_off[0]:case.pt_off[1]]]
    rows = rows.reshape(-1, case.KVH, case.D)[:S0].transpose(1, 0, 2)
    assert np.array_equal(gathered.reshape(case.KVH, S0, case.D), rows)


@pytest.mark.gpu
def test_layer_ops_through_the_cpp_class(oracle_mod, tmp_path):
    """RMSNorm -> Q4_0 mat-vec -> add, and the gate | up split with SiLU * up, called as the walker calls them:
    weights as host vectors, cached on the device under the tensor's name."""
    binary = _binary()
    batch, rows, cols = 5, 384, 512
    rng = np.random.default_rng(31)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    nw = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    w = synth.random_q4_0(rng, rows, cols)
    resid = rng.standard_normal((batch, rows)).astype(np.float32)
    gate_up = (rng.standard_normal((batch, rows)) * 2).astype(np.float32)
    inp, out = tmp_path / "ops_in.bin", tmp_path / "ops_out.bin"
    with open(inp, "wb") as f:
        for a in (x, nw, w, resid, gate_up):
            f.write(np.ascontiguousarray(a).tobytes())
    res = subprocess.run([str(binary), "ops", str(inp), str(out), str(batch), str(rows), str(cols)],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr + res.stdout
    raw = np.fromfile(out, dtype=np.float32)
    n, z, a, sm = np.split(raw, np.cumsum([batch * cols, batch * rows, batch * rows]))
    n_want = oracle_mod.rms_norm_batched(x, nw, 1e-5)
    np.testing.assert_allclose(n.reshape(batch, cols), n_want, rtol=1e-5, atol=1e-6)
    z_want = oracle_mod.matmul_quant_batched("q4_0", w, n_want, rows, cols)
    absdot = np.abs(n_want).astype(np.float64) @ np.abs(oracle_mod.dequant_rows("q4_0", w, rows, cols)).astype(np.float64).T
    assert (np.abs(z.reshape(batch, rows) - z_want) <= 4e-5 * absdot + 1e-6).all()
    assert np.array_equal(a.view(np.uint32), oracle_mod.add(z.reshape(batch, rows), resid).reshape(-1).view(np.uint32))
    _, _, sm_want = oracle_mod.gate_up_split_silu_mul(gate_up, rows // 2)
    np.testing.assert_allclose(sm.reshape(batch, rows // 2), sm_want, rtol=1e-5, atol=1e-6)
