"""The walker step's ops around attention on the GPU against the CPU oracle (oracle/layer_oracle.c, itself
pinned bit for bit on the reference's CPU code by tests/test_layer_oracle.py).

What is compared, and how closely:
  add                       bit for bit.
  gate / up copies          bit for bit.
  RMSNorm                   the GPU sums the squares in another order: rtol 1e-5, atol 1e-6 (fp32).
  SiLU(gate) * up           CUDA's expf against libm's (both within 2 ulp): rtol 1e-5, atol 1e-6.
  Q4_0 / Q6_K mat-vec       the kernel keeps the block integers exact, carries every activation as two fp16
                            numbers (22 bits) and sums in fp32, so only the order of the fp32 sum differs
                            from the CPU loop:   |err| <= 2e-5 * sum_c |W[r,c] x[n,c]|
                            (the CPU's own chain of up to 5632 fp32 additions is the larger part of that),
                            for activations that are fp16 numbers and for general fp32 ones alike.
"""
import zlib

import numpy as np
import pytest

from mlcompiler_b200 import synth

pytestmark = pytest.mark.gpu


def _dev(a):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.cuda()


def _run(executor, fn):
    import torch
    assert executor.beginForwardPassCB()
    ok = fn()
    assert ok, executor.last_error()
    assert executor.flushForwardPassCB(), executor.last_error()
    torch.cuda.synchronize()


@pytest.mark.parametrize("batch,length", [(32, 2048), (1, 2050), (5, 64), (3, 4099), (64, 5632)])
def test_rms_norm_batched(executor, oracle_mod, batch, length):
    import torch
    rng = np.random.default_rng(batch * 7919 + length)
    x = (rng.standard_normal((batch, length)) * rng.uniform(0.1, 8.0, (batch, 1))).astype(np.float32)
    w = rng.uniform(0.5, 1.5, length).astype(np.float32)
    want = oracle_mod.rms_norm_batched(x, w, 1e-5)
    dx, dw = _dev(x), _dev(w)
    out = torch.full((batch, length), float("nan"), device="cuda")
    out16 = torch.full((batch, length), float("nan"), device="cuda", dtype=torch.float16)
    _run(executor, lambda: executor.encodeRmsNormBatched(dx, dw, 1e-5, batch, length, out, out16))
    got = out.cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    assert torch.equal(out16, out.half()), "the fp16 copy is not the rounded fp32 row"
    out2 = torch.full((batch, length), float("nan"), device="cuda")
    _run(executor, lambda: executor.encodeRmsNormBatched(dx, dw, 1e-5, batch, length, out2))
    assert torch.equal(out, out2)


@pytest.mark.parametrize("n", [32 * 2048, 1027, 3, 4])
def test_add_batched_bit_exact(executor, oracle_mod, n):
    import torch
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float32)
    b = (rng.standard_normal(n) * 100).astype(np.float32)
    out = torch.full((n,), float("nan"), device="cuda")
    da, db = _dev(a), _dev(b)
    _run(executor, lambda: executor.encodeAddBatched(da, db, out, n))
    assert np.array_equal(out.cpu().numpy().view(np.uint32), oracle_mod.add(a, b).view(np.uint32))


@pytest.mark.parametrize("batch,inner,rows", [(32, 5632, 11264), (3, 100, 260), (1, 7, 14)])
def test_gate_up_split_silu_mul(executor, oracle_mod, batch, inner, rows):
    import torch
    rng = np.random.default_rng(batch + inner)
    gu = (rng.standard_normal((batch, rows)) * 3).astype(np.float32)
    gu[0, :4] = [0.0, -0.0, 60.0, -60.0][:min(4, rows)]
    g_want, u_want, want = oracle_mod.gate_up_split_silu_mul(gu, inner)
    dgu = _dev(gu)
    gate, up, out = (torch.full((batch, inner), float("nan"), device="cuda") for _ in range(3))
    _run(executor, lambda: executor.encodeGateUpSplitSiluMul(dgu, gate, up, out, batch, inner, rows))
    assert np.array_equal(gate.cpu().numpy().view(np.uint32), g_want.view(np.uint32))
    assert np.array_equal(up.cpu().numpy().view(np.uint32), u_want.view(np.uint32))
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    # without the copies, and as the two-buffer op
    out2 = torch.full((batch, inner), float("nan"), device="cuda")
    _run(executor, lambda: executor.encodeGateUpSplitSiluMul(dgu, None, None, out2, batch, inner, rows))
    assert torch.equal(out, out2)
    out3 = torch.full((batch, inner), float("nan"), device="cuda")
    _run(executor, lambda: executor.encodeSiluMulBatched(gate, up, out3, batch * inner))
    assert torch.equal(out, out3)


def _weights(kind, rng, rows, cols, pad_to=16):
    raw = synth.random_q4_0(rng, rows, cols) if kind == "q4_0" else synth.random_q6_k(rng, rows, cols)
    row_bytes = raw.shape[1]
    stride = (row_bytes + pad_to - 1) // pad_to * pad_to
    w = np.zeros((rows, stride), np.uint8)
    w[:, :row_bytes] = raw
    if stride > row_bytes:
        w[:, row_bytes:] = 0xA5          # bytes between rows must not matter
    return w, stride


def _oracle_matvec(oracle_mod, kind, w, x, rows, cols):
    want = oracle_mod.matmul_quant_batched(kind, w, x, rows, cols)
    dense = oracle_mod.dequant_rows(kind, w, rows, cols)
    absdot = np.abs(x).astype(np.float64) @ np.abs(dense).astype(np.float64).T
    return want, absdot


def _encode(executor, kind, dw, dx, batch, rows, cols, stride, out):
    if kind == "q4_0":
        return executor.encodeMatMulQ4_0Batched(dw, dx, batch, rows, cols, stride, out)
    return executor.encodeMatMulQ6KBatched(dw, dx, batch, rows, cols, stride, out)


MATVEC = [
    # kind, batch, rows, cols
    ("q4_0", 32, 2560, 2048),       # fused QKV of the 1.1B model
    ("q4_0", 32, 2048, 5632),       # ffn_down: 11 column slices
    ("q4_0", 1, 256, 2048),
    ("q4_0", 7, 100, 64),           # rows short of a tile, 36-byte rows padded to 48
    ("q4_0", 64, 300, 1024),
    ("q4_0", 33, 129, 416),         # ragged everywhere: 13 blocks, one row into a second tile
    ("q4_0", 16, 11264, 2048),      # gate | up
    ("q6_k", 32, 4000, 2048),       # a slice of the lm_head
    ("q6_k", 3, 130, 256),
    ("q6_k", 64, 512, 512),
    ("q6_k", 9, 200, 1280),         # 5 super-blocks: slices of 2 + 2 + 1
]


@pytest.mark.parametrize("kind,batch,rows,cols", MATVEC, ids=[f"{c[0]}-{c[1]}x{c[2]}x{c[3]}" for c in MATVEC])
def test_quant_matvec(executor, oracle_mod, kind, batch, rows, cols):
    import torch
    rng = np.random.default_rng(zlib.crc32(f"{kind}-{batch}-{rows}-{cols}".encode()))
    w, stride = _weights(kind, rng, rows, cols)
    dw = _dev(w)
    for form in ("fp16_numbers", "fp32"):
        x = rng.standard_normal((batch, cols)).astype(np.float32) * 2.0
        if form == "fp16_numbers":
            x = x.astype(np.float16).astype(np.float32)
        want, absdot = _oracle_matvec(oracle_mod, kind, w, x, rows, cols)
        dx = _dev(x)
        out = torch.full((batch, rows), float("nan"), device="cuda")
        _run(executor, lambda: _encode(executor, kind, dw, dx, batch, rows, cols, stride, out))
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        err = np.abs(got.astype(np.float64) - want)
        rel = 2e-5
        worst = (err - rel * absdot).max()
        assert worst <= 1e-7, f"{form}: error {err.max():.3e} exceeds {rel:.1e} * sum |w x| by {worst:.3e}"
        assert np.sqrt((err ** 2).mean()) <= 2e-6 * np.sqrt((absdot ** 2).mean())
        out2 = torch.full((batch, rows), float("nan"), device="cuda")
        _run(executor, lambda: _encode(executor, kind, dw, dx, batch, rows, cols, stride, out2))
        assert torch.equal(out, out2), "two runs of the mat-vec differ"


@pytest.mark.parametrize("batch,inner,hidden", [(32, 5632, 2048), (5, 256, 200)])
def test_matvec_with_silu_mul_input_and_residual(executor, oracle_mod, batch, inner, hidden):
    """ffn_down fused with its neighbours: input = SiLU(gate) * up from the gate | up rows, output = residual +
    W input - against the oracle's three separate ops."""
    import torch
    rng = np.random.default_rng(inner)
    w, stride = _weights("q4_0", rng, hidden, inner)
    gu = (rng.standard_normal((batch, 2 * inner + 8)) * 2).astype(np.float32)
    resid = rng.standard_normal((batch, hidden)).astype(np.float32)
    _, _, mix = oracle_mod.gate_up_split_silu_mul(gu, inner)
    down, absdot = _oracle_matvec(oracle_mod, "q4_0", w, mix, hidden, inner)
    want = oracle_mod.add(resid, down)
    dw, dgu, dres = _dev(w), _dev(gu), _dev(resid)
    out = torch.full((batch, hidden), float("nan"), device="cuda")
    _run(executor, lambda: executor.encodeMatMulQuantFused(0, dw, dgu, gu.shape[1], True, dres, batch, hidden, inner,
                                                           stride, out))
    err = np.abs(out.cpu().numpy().astype(np.float64) - want)
    bound = 4e-5 * absdot + 1e-6 * (1 + np.abs(want))
    assert (err <= bound).all(), f"max error {err.max():.3e}"
    # the residual alone (the output projection's form), plain input
    x = rng.standard_normal((batch, inner)).astype(np.float32)
    down, absdot = _oracle_matvec(oracle_mod, "q4_0", w, x, hidden, inner)
    want = oracle_mod.add(resid, down)
    dx = _dev(x)
    _run(executor, lambda: executor.encodeMatMulQuantFused(0, dw, dx, inner, False, dres, batch, hidden, inner, stride, out))
    err = np.abs(out.cpu().numpy().astype(np.float64) - want)
    assert (err <= 2e-5 * absdot + 1e-6 * (1 + np.abs(want))).all()


@pytest.mark.parametrize("kind,batch,rows,cols", [("q4_0", 32, 2560, 2048), ("q6_k", 5, 300, 512), ("q4_0", 9, 70, 416)])
def test_packed_activations_give_the_same_bits(executor, kind, batch, rows, cols):
    """RMSNorm writing the mat-vec's operand format + a mat-vec that takes it (input_kind 2) must equal, bit for
    bit, RMSNorm to fp32 + the plain mat-vec: the packed words are what the plain kernel makes of the fp32 values."""
    import torch
    rng = np.random.default_rng(cols + rows)
    w, stride = _weights(kind, rng, rows, cols)
    x = (rng.standard_normal((batch, cols)) * 3).astype(np.float32)
    g = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    dw, dx, dg = _dev(w), _dev(x), _dev(g)
    norm = torch.full((batch, cols), float("nan"), device="cuda")
    norm2 = torch.full((batch, cols), float("nan"), device="cuda")
    packed = torch.zeros((batch, cols), device="cuda", dtype=torch.int32)
    want = torch.full((batch, rows), float("nan"), device="cuda")
    got = torch.full((batch, rows), float("nan"), device="cuda")
    quant = 0 if kind == "q4_0" else 1

    def both():
        return (executor.encodeRmsNormBatched(dx, dg, 1e-5, batch, cols, norm) and
                _encode(executor, kind, dw, norm, batch, rows, cols, stride, want) and
                executor.encodeRmsNormBatchedPacked(dx, dg, 1e-5, batch, cols, norm2, packed) and
                executor.encodeMatMulQuantFused(quant, dw, packed, cols, 2, None, batch, rows, cols, stride, got))
    _run(executor, both)
    assert torch.equal(norm, norm2)
    assert torch.equal(want, got)
    # without the fp32 copy
    got2 = torch.full((batch, rows), float("nan"), device="cuda")
    packed.zero_()
    _run(executor, lambda: executor.encodeRmsNormBatchedPacked(dx, dg, 1e-5, batch, cols, None, packed) and
         executor.encodeMatMulQuantFused(quant, dw, packed, cols, 2, None, batch, rows, cols, stride, got2))
    assert torch.equal(want, got2)


def _unpack_words(words):
    """Operand words [batch, n] (int32; per pair of columns {hi0, hi1}, {lo0, lo1}) -> hi + lo as float64 [batch, n]."""
    h = words.view(np.uint16).view(np.float16).reshape(words.shape[0], -1, 2, 2).astype(np.float64)   # [b, pair, hi|lo, 2]
    return (h[:, :, 0, :] + h[:, :, 1, :]).reshape(words.shape[0], -1)


@pytest.mark.parametrize("kind,batch,inner,hidden", [("q4_0", 32, 5632, 2048), ("q4_0", 5, 100, 64), ("q6_k", 7, 72, 256),
                                                     ("q4_0", 16, 4100, 256)])
def test_gate_up_projection_with_silu_epilogue(executor, oracle_mod, kind, batch, inner, hidden):
    """gate | up mat-vec whose row tiles pair gate rows with their up rows and whose epilogue writes
    SiLU(gate) * up as operand words: against the oracle's mat-vec + gate_up_split_silu_mul, and - fed to the
    down projection as input_kind 2 - against the oracle's down projection + add."""
    import torch
    rng = np.random.default_rng(inner + hidden)
    w, stride = _weights(kind, rng, 2 * inner, hidden)
    x = (rng.standard_normal((batch, hidden)) * 0.5).astype(np.float32)
    gu, absdot = _oracle_matvec(oracle_mod, kind, w, x, 2 * inner, hidden)
    gu32 = gu.astype(np.float32)
    _, _, mix = oracle_mod.gate_up_split_silu_mul(gu32, inner)
    quant = 0 if kind == "q4_0" else 1
    dw, dx = _dev(w), _dev(x)
    words = torch.zeros((batch, inner), device="cuda", dtype=torch.int32)
    _run(executor, lambda: executor.encodeMatMulGateUpSiluPacked(quant, dw, dx, hidden, 0, batch, inner, hidden, stride, words))
    got = _unpack_words(words.cpu().numpy())
    # d(silu(g) u) <= |u| 1.1 dg + |silu(g)| du, the sums' own bound as in test_quant_matvec, + 22-bit words + expf
    g, u = gu[:, :inner].astype(np.float64), gu[:, inner:2 * inner].astype(np.float64)
    dg, du = 2e-5 * absdot[:, :inner] + 1e-7, 2e-5 * absdot[:, inner:2 * inner] + 1e-7
    silu = g / (1 + np.exp(-g))
    bound = np.abs(u) * 1.1 * dg + np.abs(silu) * du + 2e-5 * np.abs(mix) + 1e-6
    err = np.abs(got - mix)
    assert (err <= bound).all(), f"max error {err.max():.3e}, worst excess {(err - bound).max():.3e}"
    # fed to the down projection as operand words (input_kind 2), with the residual: the oracle's three separate ops
    if inner % 32 == 0:
        wd, stride_d = _weights("q4_0", rng, hidden, inner)
        resid = rng.standard_normal((batch, hidden)).astype(np.float32)
        down, absdot_d = _oracle_matvec(oracle_mod, "q4_0", wd, mix, hidden, inner)
        want = oracle_mod.add(resid, down)
        dwd, dres = _dev(wd), _dev(resid)
        out = torch.full((batch, hidden), float("nan"), device="cuda")
        _run(executor, lambda: executor.encodeMatMulQuantFused(0, dwd, words, inner, 2, dres, batch, hidden, inner, stride_d, out))
        err = np.abs(out.cpu().numpy().astype(np.float64) - want)
        assert (err <= 4e-5 * absdot_d + 1e-6 * (1 + np.abs(want))).all(), f"max error {err.max():.3e}"
    # twice the same bits
    words2 = torch.zeros_like(words)
    _run(executor, lambda: executor.encodeMatMulGateUpSiluPacked(quant, dw, dx, hidden, 0, batch, inner, hidden, stride, words2))
    assert torch.equal(words, words2)


@pytest.mark.parametrize("batch,vocab,group_rows", [(32, 32000, 8000), (3, 1000, 0), (5, 321, 128), (1, 7, 64), (64, 4099, 1088)])
def test_argmax_rows(executor, batch, vocab, group_rows):
    """Greedy sampling on the device: the first maximum of every request's logits, from a plain [batch, vocab] array
    or from the walker's layout (groups of vocabulary rows, each a [batch, rows of the group] array)."""
    import torch
    rng = np.random.default_rng(vocab)
    logits = rng.standard_normal((batch, vocab)).astype(np.float32)
    logits[0, 5 % vocab] = logits[0, vocab - 1] = 9.0           # a tie: the lower index wins
    if batch > 1:
        logits[1, :] = -3.5                                     # all equal: index 0
    if batch > 2:
        logits[2, vocab - 1] = 50.0                             # the last column
    want = logits.argmax(axis=1).astype(np.uint32)
    if group_rows and group_rows < vocab:
        laid = np.concatenate([logits[:, r0:r0 + group_rows].reshape(-1) for r0 in range(0, vocab, group_rows)])
    else:
        laid = logits.reshape(-1)
    d = _dev(laid)
    out = torch.full((batch,), 0x7FFFFFFF, device="cuda", dtype=torch.int32)
    _run(executor, lambda: executor.encodeArgmaxRows(d, batch, vocab, group_rows, out))
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want)


def test_layer_ops_argument_rules(executor):
    import torch
    x = torch.zeros((2, 64), device="cuda")
    w = torch.zeros((64,), device="cuda")
    out = torch.zeros((2, 64), device="cuda")
    wq = torch.zeros((128, 48), device="cuda", dtype=torch.uint8)
    # no open pass: every encode* refuses, like the reference's (metal_runtime.mm:7935)
    assert not executor.encodeRmsNormBatched(x, w, 1e-5, 2, 64, out)
    assert "open pass" in executor.last_error()
    assert not executor.encodeAddBatched(x, x, out, 128)
    assert not executor.encodeMatMulQ4_0Batched(wq, x, 2, 128, 64, 48, out)
    assert executor.beginForwardPassCB()
    assert not executor.encodeMatMulQ4_0Batched(wq, x, 2, 128, 48, 48, out)       # 1.5 blocks per row
    assert not executor.encodeMatMulQ4_0Batched(wq, x, 2, 128, 64, 32, out)       # stride shorter than a row
    assert not executor.encodeMatMulQ4_0Batched(wq, x, 65, 128, 64, 48, out)      # batch above the limit
    assert not executor.encodeMatMulQ6KBatched(wq, x, 2, 128, 64, 48, out)        # not a whole super-block
    assert not executor.encodeGateUpSplitSiluMul(x, None, None, out, 2, 40, 64)   # row shorter than gate + up
    assert not executor.encodeMatMulGateUpSiluPacked(0, wq, x, 64, 0, 2, 62, 64, 48, out)   # inner not a multiple of 4
    assert not executor.encodeMatMulGateUpSiluPacked(0, wq, x, 64, 1, 2, 64, 64, 48, out)   # SiLU input makes no sense here
    assert executor.encodeAddBatched(x, x, out, 0)                                # nothing to do is not an error
    assert executor.flushForwardPassCB(), executor.last_error()


def test_layer_op_suites_on_the_tensor_memory_kernel():
    """The mat-vec has two kernels: mma.sync (the default) and tcgen05 with the accumulator in tensor memory
    (MLC_B200_MATVEC=tcgen05, batches of up to 32). The op tests above and the whole-model replay run again with
    the second one selected."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MLC_B200_MATVEC="tcgen05")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
                        "tests/test_gpu_layer_ops.py", "tests/test_gpu_model_walker.py", "-k", "not tensor_memory_kernel"],
                       cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1000:]
