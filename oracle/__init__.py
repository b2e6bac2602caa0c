"""CPU oracle for the paged-attention path. TEST INFRASTRUCTURE ONLY.

Two layers:
  * `port`  - paged_oracle.c, a plain-C restatement of the reference's algorithm
              (each function cites the reference lines it follows);
  * `ref`   - oracle/_ref/libref_attention.so, MLcompiler's own executor-CPU
              attention compiled from its unmodified sources by build_ref.py
              (present only where the reference checkout was available at build
              time, or where the prebuilt file travelled with the tree).

Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py may
import this package. The product library never does.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_LIB = HERE / "libpaged_oracle.so"
REF_LIB = HERE / "_ref" / "libref_attention.so"

_u32p = C.POINTER(C.c_uint32)
_u16p = C.POINTER(C.c_uint16)
_fp = C.POINTER(C.c_float)
_vp, _sz, _u32, _i, _f = C.c_void_p, C.c_size_t, C.c_uint32, C.c_int, C.c_float


PORT_SOURCES = ["paged_oracle.c", "layer_oracle.c"]


def build_port(force: bool = False) -> Path:
    srcs = [HERE / n for n in PORT_SOURCES]
    # -ffp-contract=off: the restatements must round like the reference's scalar C++ (no fused multiply-add)
    if force or not PORT_LIB.exists() or PORT_LIB.stat().st_mtime < max(s.stat().st_mtime for s in srcs):
        subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-std=c11", "-ffp-contract=off", "-o", str(PORT_LIB),
                        *map(str, srcs), "-lm"], check=True)
    return PORT_LIB


def build_ref():
    import importlib
    return importlib.import_module(__name__ + ".build_ref").build(verbose=False)


_port = None
_ref = None


def port():
    global _port
    if _port is None:
        lib = C.CDLL(str(build_port()))
        lib.orc_fp16_to_float.restype = _f
        lib.orc_fp16_to_float.argtypes = [C.c_uint16]
        for n in ("orc_float_to_fp16_ref_scalar", "orc_float_to_fp16_rne"):
            getattr(lib, n).restype = C.c_uint16
            getattr(lib, n).argtypes = [_f]
        lib.orc_paged_attention.restype = None
        lib.orc_paged_attention.argtypes = [_fp, _u16p, _u16p, _u32p, _u32p, _u32p, _u32p, _u32, _u32, _u32,
                                            _u32, _u32, _i, _f, _fp]
        lib.orc_paged_attention_tiled.restype = None
        lib.orc_paged_attention_tiled.argtypes = [_fp, _u16p, _u16p, _u32p, _u32p, _u32p, _u32p, _u32, _u32,
                                                  _u32, _u32, _u32, _i, _f, _u32, _u32, _u32, _fp, _fp]
        lib.orc_lse_combine.restype = None
        lib.orc_lse_combine.argtypes = [_fp, _fp, _u32, _sz, _u32, _fp]
        lib.orc_paged_prefill.restype = None
        lib.orc_paged_prefill.argtypes = [_fp, _u16p, _u16p, _u32p, _u32p, _u32p, _u32p, _u32p, _u32, _u32,
                                          _u32, _u32, _u32, _f, _fp]
        lib.orc_scatter_kv_paged_batched_f16.restype = None
        lib.orc_scatter_kv_paged_batched_f16.argtypes = [_u16p, _u16p, _u32p, _u32p, _u32, _u32, _u32, _u32]
        lib.orc_scatter_kv_paged.restype = None
        lib.orc_scatter_kv_paged.argtypes = [_vp, _vp, _u32p, _u32, _u32, _u32, _u32, _u32, _u32]
        lib.orc_gather_kv_pages.restype = None
        lib.orc_gather_kv_pages.argtypes = [_vp, _u32p, _vp, _u32, _u32, _u32, _u32, _u32]
        lib.orc_pool_create.restype = _vp
        lib.orc_pool_create.argtypes = [_u32]
        lib.orc_pool_destroy.argtypes = [_vp]
        lib.orc_pool_allocate.argtypes = [_vp, _u32p]
        lib.orc_pool_release.argtypes = [_vp, _u32]
        lib.orc_pool_in_use.restype = _sz
        lib.orc_pool_in_use.argtypes = [_vp]
        lib.orc_pool_free.restype = _sz
        lib.orc_pool_free.argtypes = [_vp]
        lib.orc_kvstate_extend.argtypes = [_vp, _u32, _u32p, C.POINTER(_sz), _u32p, _u32p, _u32p]
        # layer_oracle.c
        _u8p = C.POINTER(C.c_uint8)
        lib.orc_rms_norm_batched.restype = None
        lib.orc_rms_norm_batched.argtypes = [_fp, _fp, _f, _u32, _u32, _fp]
        lib.orc_add.restype = None
        lib.orc_add.argtypes = [_fp, _fp, _fp, _sz]
        lib.orc_silu_mul.restype = None
        lib.orc_silu_mul.argtypes = [_fp, _fp, _fp, _sz]
        lib.orc_gate_up_split_silu_mul.restype = None
        lib.orc_gate_up_split_silu_mul.argtypes = [_fp, _u32, _u32, _u32, _fp, _fp, _fp]
        for q in ("q4_0", "q6_k"):
            getattr(lib, f"orc_row_size_{q}").restype = _sz
            getattr(lib, f"orc_row_size_{q}").argtypes = [_sz]
            getattr(lib, f"orc_dequant_row_{q}").restype = None
            getattr(lib, f"orc_dequant_row_{q}").argtypes = [_u8p, _sz, _fp]
            getattr(lib, f"orc_dot_row_{q}").restype = _f
            getattr(lib, f"orc_dot_row_{q}").argtypes = [_u8p, _sz, _fp]
            getattr(lib, f"orc_matmul_{q}_batched").restype = None
            getattr(lib, f"orc_matmul_{q}_batched").argtypes = [_u8p, _fp, _u32, _u32, _u32, _sz, _fp]
        _port = lib
    return _port


def ref():
    """The reference-linked library, or None when it is not available here."""
    global _ref
    if _ref is None:
        path = REF_LIB
        if not path.exists():
            try:
                built = build_ref()
            except Exception:
                built = None
            if not built or not Path(built).exists():
                return None
        lib = C.CDLL(str(path))
        lib.ref_attn_create.restype = _vp
        lib.ref_attn_create.argtypes = [_sz, _sz, _sz, _sz]
        lib.ref_attn_destroy.argtypes = [_vp]
        lib.ref_attn_cache_dtype.argtypes = [_vp]
        lib.ref_attn_load_history.argtypes = [_vp, _fp, _fp, _sz]
        lib.ref_attn_decode.argtypes = [_vp, _sz, _fp, _fp, _fp, _fp]
        lib.ref_attn_decode_direct.argtypes = [_vp, _sz, _fp, _fp, _fp, _fp]
        lib.ref_attn_read_cache_row.argtypes = [_vp, _i, _sz, _sz, _u16p]
        lib.ref_fp16_to_float.restype = _f
        lib.ref_fp16_to_float.argtypes = [C.c_uint16]
        lib.ref_float_to_fp16.restype = C.c_uint16
        lib.ref_float_to_fp16.argtypes = [_f]
        lib.ref_pool_create.restype = _vp
        lib.ref_pool_create.argtypes = [_u32]
        lib.ref_pool_destroy.argtypes = [_vp]
        lib.ref_pool_allocate.argtypes = [_vp, _u32p]
        lib.ref_pool_release.argtypes = [_vp, _u32]
        lib.ref_pool_in_use.restype = _sz
        lib.ref_pool_in_use.argtypes = [_vp]
        lib.ref_pool_free.restype = _sz
        lib.ref_pool_free.argtypes = [_vp]
        lib.ref_kvstate_create.restype = _vp
        lib.ref_kvstate_create.argtypes = [_u32]
        lib.ref_kvstate_destroy.argtypes = [_vp]
        lib.ref_kvstate_extend.argtypes = [_vp, _vp, _u32p, _u32p]
        lib.ref_kvstate_reserve.argtypes = [_vp, _vp, _sz]
        lib.ref_kvstate_pages.restype = _sz
        lib.ref_kvstate_pages.argtypes = [_vp, _u32p, _sz]
        lib.ref_kvstate_total.restype = _sz
        lib.ref_kvstate_total.argtypes = [_vp]
        lib.ref_kvstate_release.argtypes = [_vp, _vp]
        _u8p = C.POINTER(C.c_uint8)
        lib.ref_elementwise_node.argtypes = [_i, _fp, _fp, _sz, _fp]
        lib.ref_gguf_describe.restype = _sz
        lib.ref_gguf_describe.argtypes = [C.c_char_p, _i, C.c_char_p, _sz]
        lib.ref_gguf_tensor.restype = C.c_longlong
        lib.ref_gguf_tensor.argtypes = [C.c_char_p, C.c_char_p, _i, C.c_void_p, _sz]
        lib.ref_tokenizer_create.restype = _vp
        lib.ref_tokenizer_create.argtypes = [C.c_char_p]
        lib.ref_tokenizer_destroy.argtypes = [_vp]
        lib.ref_tokenizer_info.argtypes = [_vp, C.POINTER(C.c_ulonglong)]
        lib.ref_tokenizer_encode.restype = _sz
        lib.ref_tokenizer_encode.argtypes = [_vp, C.c_char_p, _sz, _i, _i, C.POINTER(C.c_ulonglong), _sz]
        lib.ref_tokenizer_decode.restype = _sz
        lib.ref_tokenizer_decode.argtypes = [_vp, C.POINTER(C.c_ulonglong), _sz, C.c_char_p, _sz]
        lib.ref_tokenizer_token_string.restype = _sz
        lib.ref_tokenizer_token_string.argtypes = [_vp, C.c_ulonglong, C.c_char_p, _sz]
        lib.ref_tokenizer_flags.argtypes = [_vp, C.c_ulonglong]
        for q in ("q4_0", "q6_k"):
            getattr(lib, f"ref_dequant_{q}").restype = None
            getattr(lib, f"ref_dequant_{q}").argtypes = [_u8p, _sz, _fp]
            getattr(lib, f"ref_dot_{q}").restype = _f
            getattr(lib, f"ref_dot_{q}").argtypes = [_u8p, _sz, _fp]
            getattr(lib, f"ref_row_size_{q}").restype = _sz
            getattr(lib, f"ref_row_size_{q}").argtypes = [_sz]
        _ref = lib
    return _ref


# ---- numpy-facing helpers ---------------------------------------------------------
def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def paged_attention(q, k_pages, v_pages, pt_flat, pt_off, seq_lens, q_pos, H, KVH, D, P, causal=True,
                    scale=None):
    """fp32 two-pass paged attention (orc_paged_attention). q: [N,H,D] float32 (or
    float16, widened exactly); k_pages / v_pages: fp16 pools as uint16 or float16."""
    q = _c(np.asarray(q, dtype=np.float32), np.float32)
    kp = _c(np.asarray(k_pages).view(np.uint16), np.uint16)
    vp = _c(np.asarray(v_pages).view(np.uint16), np.uint16)
    pt_flat, pt_off = _c(pt_flat, np.uint32), _c(pt_off, np.uint32)
    seq_lens, q_pos = _c(seq_lens, np.uint32), _c(q_pos, np.uint32)
    N = seq_lens.size
    out = np.zeros((N, H, D), np.float32)
    port().orc_paged_attention(_p(q, _fp), _p(kp, _u16p), _p(vp, _u16p), _p(pt_flat, _u32p), _p(pt_off, _u32p),
                               _p(seq_lens, _u32p), _p(q_pos, _u32p), N, H, KVH, D, P, 1 if causal else 0,
                               float(scale if scale is not None else 1.0 / np.sqrt(np.float32(D))), _p(out, _fp))
    return out


def paged_attention_tiled(q, k_pages, v_pages, pt_flat, pt_off, seq_lens, q_pos, H, KVH, D, P, causal=True,
                          scale=None, tile=32, t0=0, t1=0xFFFFFFFF, partial=False):
    """The MSL kernel's tiled recurrence (orc_paged_attention_tiled). With partial=True
    returns (o_unnormalised [N,H,D], ml [N,H,2]) restricted to tokens [t0, t1)."""
    q = _c(np.asarray(q, dtype=np.float32), np.float32)
    kp = _c(np.asarray(k_pages).view(np.uint16), np.uint16)
    vp = _c(np.asarray(v_pages).view(np.uint16), np.uint16)
    pt_flat, pt_off = _c(pt_flat, np.uint32), _c(pt_off, np.uint32)
    seq_lens, q_pos = _c(seq_lens, np.uint32), _c(q_pos, np.uint32)
    N = seq_lens.size
    out = np.zeros((N, H, D), np.float32)
    ml = np.zeros((N, H, 2), np.float32) if partial else None
    port().orc_paged_attention_tiled(_p(q, _fp), _p(kp, _u16p), _p(vp, _u16p), _p(pt_flat, _u32p),
                                     _p(pt_off, _u32p), _p(seq_lens, _u32p), _p(q_pos, _u32p), N, H, KVH, D, P,
                                     1 if causal else 0,
                                     float(scale if scale is not None else 1.0 / np.sqrt(np.float32(D))),
                                     tile, t0, min(t1, 0xFFFFFFFF), _p(out, _fp),
                                     _p(ml, _fp) if partial else None)
    return (out, ml) if partial else out


def lse_combine(o_parts, ml_parts):
    """o_parts [parts, rows..., D] un-normalised, ml_parts [parts, rows..., 2] -> [rows..., D]."""
    o_parts = _c(o_parts, np.float32)
    ml_parts = _c(ml_parts, np.float32)
    parts, D = o_parts.shape[0], o_parts.shape[-1]
    rows = int(np.prod(o_parts.shape[1:-1]))
    out = np.zeros(o_parts.shape[1:], np.float32)
    port().orc_lse_combine(_p(o_parts, _fp), _p(ml_parts, _fp), parts, rows, D, _p(out, _fp))
    return out


def paged_prefill(q, k_pages, v_pages, pt_flat, pt_off, seq_lens, q_start, q_len, H, KVH, D, P, scale=None):
    q = _c(np.asarray(q, dtype=np.float32), np.float32)
    kp = _c(np.asarray(k_pages).view(np.uint16), np.uint16)
    vp = _c(np.asarray(v_pages).view(np.uint16), np.uint16)
    pt_flat, pt_off = _c(pt_flat, np.uint32), _c(pt_off, np.uint32)
    seq_lens, q_start, q_len = _c(seq_lens, np.uint32), _c(q_start, np.uint32), _c(q_len, np.uint32)
    out = np.zeros_like(q)
    port().orc_paged_prefill(_p(q, _fp), _p(kp, _u16p), _p(vp, _u16p), _p(pt_flat, _u32p), _p(pt_off, _u32p),
                             _p(seq_lens, _u32p), _p(q_start, _u32p), _p(q_len, _u32p), seq_lens.size, H, KVH,
                             D, P, float(scale if scale is not None else 1.0 / np.sqrt(np.float32(D))),
                             _p(out, _fp))
    return out


def scatter_kv_paged_batched_f16(src, pool, page_ids, slots, P, KVH, D):
    """In place on `pool` (uint16 view of fp16)."""
    src = _c(np.asarray(src).view(np.uint16), np.uint16)
    assert pool.dtype == np.uint16 and pool.flags["C_CONTIGUOUS"]
    page_ids, slots = _c(page_ids, np.uint32), _c(slots, np.uint32)
    port().orc_scatter_kv_paged_batched_f16(_p(src, _u16p), _p(pool, _u16p), _p(page_ids, _u32p),
                                            _p(slots, _u32p), P, KVH, D, page_ids.size)
    return pool


def scatter_kv_paged(src, pool, page_table, P, KVH, D, tokens, start_slot):
    src = np.ascontiguousarray(src)
    assert pool.flags["C_CONTIGUOUS"] and pool.dtype.itemsize == src.dtype.itemsize
    page_table = _c(page_table, np.uint32)
    port().orc_scatter_kv_paged(_p(src, _vp), _p(pool, _vp), _p(page_table, _u32p), P, KVH, D, tokens,
                                start_slot, src.dtype.itemsize)
    return pool


def gather_kv_pages(pool, page_table, P, KVH, D, num_tokens):
    pool = np.ascontiguousarray(pool)
    page_table = _c(page_table, np.uint32)
    dst = np.zeros((KVH, num_tokens, D), pool.dtype)
    port().orc_gather_kv_pages(_p(pool, _vp), _p(page_table, _u32p), _p(dst, _vp), P, KVH, D, num_tokens,
                               pool.dtype.itemsize)
    return dst


def reference_decode(q, k_tokens, v_tokens, H, KVH, D, direct=False):
    """MLcompiler's executor-CPU attention for ONE request through the reference-
    linked library: k_tokens / v_tokens [S, KVH, D] in logical token order (values
    exactly representable in fp16); the last row is fed as the new token at
    position S-1, the others are loaded as history. Returns (out [H, D], S) or
    None when the reference library is unavailable."""
    lib = ref()
    if lib is None:
        return None
    k = _c(np.asarray(k_tokens, dtype=np.float32), np.float32)
    v = _c(np.asarray(v_tokens, dtype=np.float32), np.float32)
    q = _c(np.asarray(q, dtype=np.float32), np.float32)
    S = k.shape[0]
    h = lib.ref_attn_create(H, KVH, D, S)
    try:
        if S > 1:
            assert lib.ref_attn_load_history(h, _p(k, _fp), _p(v, _fp), S - 1) == 0
        out = np.zeros((H, D), np.float32)
        fn = lib.ref_attn_decode_direct if direct else lib.ref_attn_decode
        kn, vn = np.ascontiguousarray(k[S - 1]), np.ascontiguousarray(v[S - 1])
        assert fn(h, S - 1, _p(q, _fp), _p(kn, _fp), _p(vn, _fp), _p(out, _fp)) == 0
        return out
    finally:
        lib.ref_attn_destroy(h)


def compute_rotary(position, rotary_dim, freq_base=10000.0, freq_scale=1.0):
    """(cos, sin) float32 [rotary_dim // 2] of one position (quantization.cpp:795-823)."""
    pairs = rotary_dim // 2
    c, s = np.zeros(pairs, np.float32), np.zeros(pairs, np.float32)
    port().orc_compute_rotary(C.c_size_t(position), C.c_size_t(rotary_dim), C.c_float(freq_base),
                              C.c_float(freq_scale), _p(c, _fp), _p(s, _fp))
    return c, s


def qkv_split_rope_cast(qkv, cos_t, sin_t, H, KVH, D, rotary_dim):
    """encodeQkvSplitRopeCast (metal_runtime.mm:7915-8025) on the CPU.
    qkv float32 [batch, qkv_rows]; returns q, k, v (float32) and k16, v16 (uint16 fp16 bits)."""
    qkv = _c(qkv, np.float32)
    batch, qkv_rows = qkv.shape
    q_rows, k_rows = H * D, KVH * D
    cos_t, sin_t = _c(cos_t, np.float32), _c(sin_t, np.float32)
    q = np.zeros((batch, q_rows), np.float32)
    k = np.zeros((batch, k_rows), np.float32)
    v = np.zeros((batch, k_rows), np.float32)
    k16 = np.zeros((batch, k_rows), np.uint16)
    v16 = np.zeros((batch, k_rows), np.uint16)
    port().orc_qkv_split_rope_cast(_p(qkv, _fp), _p(q, _fp), _p(k, _fp), _p(v, _fp), _p(k16, _u16p),
                                   _p(v16, _u16p), _p(cos_t, _fp), _p(sin_t, _fp), batch, H, KVH, D,
                                   qkv_rows, q_rows, k_rows, k_rows, rotary_dim)
    return q, k, v, k16, v16


# ---- the walker step's other ops (layer_oracle.c) ---------------------------------------
_u8p = C.POINTER(C.c_uint8)


def rms_norm_batched(x, weight, eps=1e-5):
    """x [batch, length] fp32, weight [length] -> [batch, length] (orc_rms_norm_batched)."""
    x = _c(x, np.float32)
    w = _c(weight, np.float32)
    out = np.zeros_like(x)
    port().orc_rms_norm_batched(_p(x, _fp), _p(w, _fp), float(eps), x.shape[0], x.shape[1], _p(out, _fp))
    return out


def add(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    out = np.zeros_like(a)
    port().orc_add(_p(a, _fp), _p(b, _fp), _p(out, _fp), a.size)
    return out


def gate_up_split_silu_mul(gate_up, ffn_inner):
    """gate_up [batch, rows >= 2 * ffn_inner] -> (gate, up, SiLU(gate) * up), each [batch, ffn_inner]."""
    gu = _c(gate_up, np.float32)
    batch, rows = gu.shape
    gate, up, out = (np.zeros((batch, ffn_inner), np.float32) for _ in range(3))
    port().orc_gate_up_split_silu_mul(_p(gu, _fp), batch, ffn_inner, rows, _p(gate, _fp), _p(up, _fp), _p(out, _fp))
    return gate, up, out


def row_size(kind: str, cols: int) -> int:
    return int(getattr(port(), f"orc_row_size_{kind}")(cols))


def dequant_rows(kind: str, weights, rows: int, cols: int):
    """Quantised rows (uint8 [rows, row_stride]) -> fp32 [rows, cols]."""
    w = _c(weights, np.uint8).reshape(rows, -1)
    out = np.zeros((rows, cols), np.float32)
    fn = getattr(port(), f"orc_dequant_row_{kind}")
    for r in range(rows):
        fn(w[r].ctypes.data_as(_u8p), cols, out[r].ctypes.data_as(_fp))
    return out


def matmul_quant_batched(kind: str, weights, x, rows: int, cols: int):
    """out[n, r] = sum_c W[r, c] * x[n, c] with W quantised as `kind` ("q4_0" / "q6_k"), fp32 sums in the
    order of the reference's CPU row functions."""
    w = _c(weights, np.uint8).reshape(rows, -1)
    x = _c(x, np.float32)
    out = np.zeros((x.shape[0], rows), np.float32)
    getattr(port(), f"orc_matmul_{kind}_batched")(w.ctypes.data_as(_u8p), _p(x, _fp), x.shape[0], rows, cols,
                                                  w.shape[1], _p(out, _fp))
    return out


def reference_gguf_describe(path, concatenate=False):
    """What the reference's GGUFLoader (compiler/frontends/gguf_loader.cpp: load() 306-433, concatenateBlockWeights()
    877-943) makes of a file, as the dict the product's mlc_gguf_describe gives (without alignment and data_start,
    which the loader does not expose). Raises RuntimeError with the loader's message if it throws."""
    import json
    lib = ref()
    assert lib is not None, "the reference library is not available here"
    cap = 1 << 16
    while True:
        buf = C.create_string_buffer(cap)
        n = lib.ref_gguf_describe(str(path).encode(), 1 if concatenate else 0, buf, cap)
        if n == 0:
            raise RuntimeError(buf.value.decode(errors="replace"))
        if n <= cap:
            return json.loads(buf.value.decode("utf-8", errors="surrogateescape"))
        cap = n


def reference_gguf_tensor(path, name, concatenate=False):
    """GGUFLoader::loadTensorData (gguf_loader.cpp:844-875) as a uint8 array; None if the loader refuses."""
    lib = ref()
    assert lib is not None, "the reference library is not available here"
    n = lib.ref_gguf_tensor(str(path).encode(), name.encode(), 1 if concatenate else 0, None, 0)
    if n < 0:
        return None
    out = np.zeros(n, np.uint8)
    lib.ref_gguf_tensor(str(path).encode(), name.encode(), 1 if concatenate else 0, out.ctypes.data_as(C.c_void_p), n)
    return out


class ReferenceTokenizer:
    """The reference's runtime::Tokenizer (compiler/runtime/tokenizer.cpp, compiled without llama.cpp: its own BPE /
    unigram / greedy code) over a GGUF file. Text is bytes in and out."""

    def __init__(self, path):
        lib = ref()
        assert lib is not None, "the reference library is not available here"
        self._lib = lib
        self._h = lib.ref_tokenizer_create(str(path).encode())
        assert self._h, "the reference could not load the file"
        info = (C.c_ulonglong * 5)()
        lib.ref_tokenizer_info(self._h, info)
        self.valid, self.vocab_size, self.bos, self.eos, self.unk = bool(info[0]), *[int(v) for v in info[1:]]

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._lib.ref_tokenizer_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def encode(self, data: bytes, add_bos=True, add_eos=False):
        n = self._lib.ref_tokenizer_encode(self._h, data, len(data), int(add_bos), int(add_eos), None, 0)
        ids = (C.c_ulonglong * max(n, 1))()
        self._lib.ref_tokenizer_encode(self._h, data, len(data), int(add_bos), int(add_eos), ids, n)
        return [int(ids[i]) for i in range(n)]

    def decode(self, ids) -> bytes:
        arr = (C.c_ulonglong * max(len(ids), 1))(*[int(i) for i in ids])
        n = self._lib.ref_tokenizer_decode(self._h, arr, len(ids), None, 0)
        buf = C.create_string_buffer(max(n, 1))
        self._lib.ref_tokenizer_decode(self._h, arr, len(ids), buf, n)
        return buf.raw[:n]

    def token_string(self, token_id) -> bytes:
        n = self._lib.ref_tokenizer_token_string(self._h, token_id, None, 0)
        buf = C.create_string_buffer(max(n, 1))
        self._lib.ref_tokenizer_token_string(self._h, token_id, buf, n)
        return buf.raw[:n]

    def flags(self, token_id) -> int:
        return int(self._lib.ref_tokenizer_flags(self._h, token_id))
