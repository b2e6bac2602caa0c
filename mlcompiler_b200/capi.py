"""ctypes binding of include/mlc_b200.h plus a thin `Executor` whose methods carry
the names and argument order of the reference's MetalExecutor members
(compiler/runtime/metal_runtime.hpp:510-533, 619-703), so that tests written
against it read like the reference's own tests.

Device buffers are passed as integers (addresses), `torch.Tensor`s (their
data_ptr() is taken) or anything with a `data_ptr()`; host arrays as anything
numpy can view as uint32.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_PKG = Path(__file__).resolve().parent
_LIB = None

MLC_F32, MLC_F16 = 0, 1
STATUS = {0: "MLC_OK", 1: "MLC_ERR_INVALID_ARG", 2: "MLC_ERR_NO_OPEN_PASS", 3: "MLC_ERR_CUDA",
          4: "MLC_ERR_BOUNDS", 5: "MLC_ERR_UNSUPPORTED", 6: "MLC_ERR_NO_DEVICE", 7: "MLC_ERR_OOM",
          8: "MLC_ERR_DEVICE_FLAG"}


class MlcError(RuntimeError):
    def __init__(self, status: int, message: str = ""):
        self.status = status
        super().__init__(f"{STATUS.get(status, status)}: {message}")


def library_path() -> Path:
    return _PKG / "libmlc_b200.so"


_u32p = C.POINTER(C.c_uint32)
_vp, _sz, _i, _f = C.c_void_p, C.c_size_t, C.c_int, C.c_float

_PROTOTYPES = {
    "mlc_ctx_create": (_i, [_i, _vp, C.POINTER(_vp)]),
    "mlc_ctx_destroy": (None, [_vp]),
    "mlc_ctx_available": (_i, [_vp]),
    "mlc_last_error": (C.c_char_p, [_vp]),
    "mlc_device_error_word": (_i, [_vp, _u32p]),
    "mlc_ctx_stream": (_vp, [_vp]),
    "mlc_ctx_launch_count": (C.c_uint64, [_vp]),
    "mlc_ctx_alloc_count": (C.c_uint64, [_vp]),
    "mlc_ctx_set_wait_limit": (_i, [_vp, C.c_uint32]),
    "mlc_ctx_set_attention_kernel": (_i, [_vp, _i]),
    "mlc_alloc": (_vp, [_vp, _sz]),
    "mlc_free": (None, [_vp, _vp]),
    "mlc_upload": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "mlc_download": (_i, [_vp, _vp, _vp, _sz, _sz]),
    "mlc_cached_buffer": (_vp, [_vp, C.c_char_p, _sz]),
    "mlc_buffer_bytes": (_sz, [_vp, _vp]),
    "mlc_pass_begin": (_i, [_vp]),
    "mlc_pass_is_open": (_i, [_vp]),
    "mlc_pass_flush": (_i, [_vp]),
    "mlc_run_scatter_kv_paged_batched_f16": (_i, [_vp, _vp, _u32p, _u32p, _sz, _sz, _sz, _sz, _vp, _sz]),
    "mlc_encode_scatter_kv_paged_batched_f16": (_i, [_vp, _vp, _u32p, _u32p, _sz, _sz, _sz, _sz, _vp, _sz]),
    "mlc_encode_scatter_kv_pair_paged_batched_f16": (_i, [_vp, _vp, _vp, _u32p, _u32p, _sz, _sz, _sz, _sz, _vp, _vp, _sz]),
    "mlc_run_scatter_kv_paged": (_i, [_vp, _vp, _u32p, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _sz, _sz]),
    "mlc_run_gather_kv_pages": (_i, [_vp, _vp, _u32p, _sz, _sz, _sz, _sz, _sz, _vp, _sz, _sz]),
    "mlc_run_paged_flash_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _u32p, _sz, _u32p, _u32p, _u32p,
                                           _sz, _sz, _sz, _sz, _sz, _i, _f, _i, _i, _sz]),
    "mlc_encode_paged_flash_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _u32p, _sz, _u32p, _u32p, _u32p,
                                              _sz, _sz, _sz, _sz, _sz, _i, _f, _i, _i, _sz]),
    "mlc_run_paged_prefill_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _u32p, _sz, _u32p, _u32p, _u32p, _u32p,
                                             _sz, _sz, _sz, _sz, _sz, _f, _i, _i, _sz]),
    "mlc_encode_paged_prefill_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _u32p, _sz, _u32p, _u32p, _u32p, _u32p,
                                                _sz, _sz, _sz, _sz, _sz, _f, _i, _i, _sz]),
    "mlc_encode_qkv_split_rope_cast": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz,
                                            _sz, _sz, _sz, _sz]),
    "mlc_encode_qkv_split_rope_scatter_planned": (_i, [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _sz, _sz]),
    "mlc_encode_matmul_qkv_rope_scatter_planned": (_i, [_vp, _vp, _i, _vp, _vp, _sz, _i, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _sz]),
    "mlc_encode_rms_norm_batched": (_i, [_vp, _vp, _vp, _f, _sz, _sz, _vp, _vp]),
    "mlc_encode_rms_norm_batched_packed": (_i, [_vp, _vp, _vp, _f, _sz, _sz, _vp, _vp]),
    "mlc_encode_add_batched": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "mlc_encode_silu_mul_batched": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "mlc_encode_gate_up_split_silu_mul": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "mlc_encode_matmul_q4_0_batched": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp]),
    "mlc_encode_matmul_q6k_batched": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp]),
    "mlc_encode_matmul_quant_fused": (_i, [_vp, _i, _vp, _vp, _sz, _i, _vp, _sz, _sz, _sz, _sz, _vp]),
    "mlc_encode_argmax_rows": (_i, [_vp, _vp, _sz, _sz, _sz, _vp]),
    "mlc_encode_matmul_gate_up_silu_packed": (_i, [_vp, _i, _vp, _vp, _sz, _i, _sz, _sz, _sz, _sz, _vp]),
    "mlc_compute_rotary_coefficients": (_i, [_sz, _sz, _f, _f, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "mlc_exchange_create": (_i, [_vp, _i, _i, _sz, _sz, C.POINTER(_vp)]),
    "mlc_exchange_handle": (_i, [_vp, _vp, _vp]),
    "mlc_exchange_attach": (_i, [_vp, _vp, _vp]),
    "mlc_exchange_attach_pointers": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "mlc_exchange_local_buffer": (_vp, [_vp]),
    "mlc_exchange_read_trace": (_i, [_vp, C.POINTER(C.c_uint64)]),
    "mlc_exchange_slot_floats": (_sz, [_vp]),
    "mlc_exchange_layout": (_i, [_i, _sz, _sz, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(_sz)]),
    "mlc_encode_exchange_lse_combine": (_i, [_vp, _vp, _vp, _vp, _sz, _vp, _i]),
    "mlc_encode_paged_attention_exchange_planned": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_float, _i, _i]),
    "mlc_exchange_destroy": (None, [_vp, _vp]),
    "mlc_ctx_last_attention_kernel": (_i, [_vp]),
    "mlc_ctx_read_trace": (C.c_uint32, [_vp, C.POINTER(C.c_uint64), _sz, _i]),
    "mlc_attn_plan_create": (_i, [_vp, _u32p, _sz, _u32p, _u32p, _u32p, _u32p, _u32p, _sz, _sz, _sz, _sz, _sz,
                                  _i, _sz, C.POINTER(_vp)]),
    "mlc_attn_plan_destroy": (None, [_vp, _vp]),
    "mlc_attn_plan_update": (_i, [_vp, _vp, _u32p, _sz, _u32p, _u32p, _u32p, _u32p, _u32p, _sz]),
    "mlc_encode_paged_flash_attention_planned": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i]),
    "mlc_encode_scatter_kv_pair_planned": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "mlc_static_scratch_bytes": (_sz, []),
    "mlc_encode_paged_flash_attention_planned_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i]),
    "mlc_encode_paged_decode_step_planned": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i]),
    "mlc_encode_paged_decode_pass_planned": (_i, [_vp, _vp, _sz, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                                  C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _f, _i, _i]),
    "mlc_encode_paged_decode_pass_host": (_i, [_vp, _vp, _sz, _vp, _vp, C.POINTER(_vp), C.POINTER(_vp), _vp, _vp, _f,
                                               _i, _i, _sz]),
    "mlc_encode_paged_attention_partial_planned": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i]),
    "mlc_encode_lse_combine": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _vp, _i]),
    "mlc_graph_begin_capture": (_i, [_vp]),
    "mlc_graph_end_capture": (_i, [_vp, C.POINTER(_vp)]),
    "mlc_graph_launch": (_i, [_vp, _vp]),
    "mlc_graph_destroy": (None, [_vp, _vp]),
}


def load_library(build_if_missing: bool = False):
    """Loads libmlc_b200.so. There is no fallback: a missing library is an error."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        if not build_if_missing:
            raise ImportError(
                f"{path} is missing: build the CUDA extension first "
                "(python -m mlcompiler_b200.build, or __graft_entry__.build())")
        from . import build as _build
        _build.build()
    lib = C.CDLL(str(path))
    for name, (res, args) in _PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def _ptr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    raise TypeError(f"not a device buffer: {type(x)}")


def _u32(a):
    arr = np.ascontiguousarray(np.asarray(a, dtype=np.uint32))
    return arr, arr.ctypes.data_as(_u32p)


class Executor:
    """One context on one GPU; replaces MetalExecutor::Instance()."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self._lib = load_library()
        h = _vp()
        st = self._lib.mlc_ctx_create(device, _vp(stream) if stream else None, C.byref(h))
        if st != 0:
            raise MlcError(st, "mlc_ctx_create failed (is a CUDA device present?)")
        self._h = h
        self.device = device

    def close(self):
        if getattr(self, "_h", None):
            self._lib.mlc_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- status ---------------------------------------------------------------
    @property
    def handle(self):
        return self._h

    def last_error(self) -> str:
        return (self._lib.mlc_last_error(self._h) or b"").decode()

    def status(self, st: int) -> bool:
        """bool view of a status code, like the reference's bool returns."""
        self.last_status = st
        return st == 0

    def check(self, st: int):
        if st != 0:
            raise MlcError(st, self.last_error())

    def isAvailable(self) -> bool:
        return bool(self._lib.mlc_ctx_available(self._h))

    def deviceErrorWord(self) -> int:
        w = C.c_uint32(0)
        self.check(self._lib.mlc_device_error_word(self._h, C.byref(w)))
        return w.value

    def launchCount(self) -> int:
        return int(self._lib.mlc_ctx_launch_count(self._h))

    def allocCount(self) -> int:
        return int(self._lib.mlc_ctx_alloc_count(self._h))

    def setWaitLimit(self, polls: int) -> bool:
        """Polls (about a microsecond each) before a wait on another GPU's flag gives up; 0 = default."""
        return self.status(self._lib.mlc_ctx_set_wait_limit(self._h, int(polls)))

    def stream(self) -> int:
        return int(self._lib.mlc_ctx_stream(self._h) or 0)

    def setAttentionKernel(self, which: int):
        self.check(self._lib.mlc_ctx_set_attention_kernel(self._h, which))

    # -- buffers (metal_runtime.hpp:693-703) --------------------------------------
    def allocateScratchBuffer(self, nbytes: int) -> int:
        return int(self._lib.mlc_alloc(self._h, nbytes) or 0)

    def releaseScratchBuffer(self, buf: int):
        self._lib.mlc_free(self._h, _vp(buf))

    def uploadToBuffer(self, buf, src: np.ndarray, dst_offset: int = 0):
        src = np.ascontiguousarray(src)
        self.check(self._lib.mlc_upload(self._h, _vp(_ptr(buf)), src.ctypes.data_as(_vp), src.nbytes, dst_offset))

    def downloadFromBuffer(self, buf, dst: np.ndarray, src_offset: int = 0):
        assert dst.flags["C_CONTIGUOUS"]
        self.check(self._lib.mlc_download(self._h, _vp(_ptr(buf)), dst.ctypes.data_as(_vp), dst.nbytes, src_offset))

    def getOrAllocCachedBuffer(self, name: str, nbytes: int) -> int:
        return int(self._lib.mlc_cached_buffer(self._h, name.encode(), nbytes) or 0)

    def bufferBytes(self, buf) -> int:
        return int(self._lib.mlc_buffer_bytes(self._h, _vp(_ptr(buf))))

    # -- pass bracketing (metal_runtime.hpp:181-183) --------------------------------
    def beginForwardPassCB(self) -> bool:
        return self.status(self._lib.mlc_pass_begin(self._h))

    def hasForwardPassCB(self) -> bool:
        return bool(self._lib.mlc_pass_is_open(self._h))

    def flushForwardPassCB(self) -> bool:
        return self.status(self._lib.mlc_pass_flush(self._h))

    # -- KV writers / readers ----------------------------------------------------------
    def scatterKVPagedBatched(self, page_storage, page_ids, slots_in_page, page_size_tokens, n_kv_heads,
                              head_dim, batch, src, capacity_pages: int = 0) -> bool:
        ids, pids = _u32(page_ids)
        sl, pslots = _u32(slots_in_page)
        if ids.size != batch or sl.size != batch:  # metal_runtime.mm:7243
            return self.status(1)
        return self.status(self._lib.mlc_run_scatter_kv_paged_batched_f16(
            self._h, _vp(_ptr(page_storage)), pids, pslots, page_size_tokens, n_kv_heads, head_dim, batch,
            _vp(_ptr(src)), capacity_pages))

    def encodeScatterKVPagedBatched(self, page_storage, page_ids, slots_in_page, page_size_tokens,
                                    n_kv_heads, head_dim, batch, src, capacity_pages: int = 0) -> bool:
        ids, pids = _u32(page_ids)
        sl, pslots = _u32(slots_in_page)
        if ids.size != batch or sl.size != batch:
            return self.status(1)
        return self.status(self._lib.mlc_encode_scatter_kv_paged_batched_f16(
            self._h, _vp(_ptr(page_storage)), pids, pslots, page_size_tokens, n_kv_heads, head_dim, batch,
            _vp(_ptr(src)), capacity_pages))

    def encodeScatterKVPairPagedBatched(self, k_storage, v_storage, page_ids, slots_in_page,
                                        page_size_tokens, n_kv_heads, head_dim, batch, k_src, v_src,
                                        capacity_pages: int = 0) -> bool:
        ids, pids = _u32(page_ids)
        sl, pslots = _u32(slots_in_page)
        if ids.size != batch or sl.size != batch:
            return self.status(1)
        return self.status(self._lib.mlc_encode_scatter_kv_pair_paged_batched_f16(
            self._h, _vp(_ptr(k_storage)), _vp(_ptr(v_storage)), pids, pslots, page_size_tokens,
            n_kv_heads, head_dim, batch, _vp(_ptr(k_src)), _vp(_ptr(v_src)), capacity_pages))

    def scatterKVPaged(self, page_storage, page_table, page_size_tokens, n_kv_heads, head_dim, tokens,
                       start_slot, src, dtype_bytes, capacity_pages: int = 0) -> bool:
        pt, ppt = _u32(page_table)
        return self.status(self._lib.mlc_run_scatter_kv_paged(
            self._h, _vp(_ptr(page_storage)), ppt, pt.size, page_size_tokens, n_kv_heads, head_dim, tokens,
            start_slot, _vp(_ptr(src)), dtype_bytes, capacity_pages))

    def gatherKVPages(self, page_storage, page_table, page_size_tokens, n_kv_heads, head_dim, num_tokens,
                      dst, dtype_bytes, capacity_pages: int = 0) -> bool:
        pt, ppt = _u32(page_table)
        return self.status(self._lib.mlc_run_gather_kv_pages(
            self._h, _vp(_ptr(page_storage)), ppt, pt.size, page_size_tokens, n_kv_heads, head_dim,
            num_tokens, _vp(_ptr(dst)), dtype_bytes, capacity_pages))

    # -- attention ---------------------------------------------------------------------
    def _attention(self, fn, q, k_pages, v_pages, o, page_tables_flat, page_table_offsets, seq_lens,
                   q_positions, batch, num_heads, kv_heads, head_dim, page_size_tokens, apply_causal,
                   scale, q_dtype, o_dtype, capacity_pages) -> bool:
        flat, pflat = _u32(page_tables_flat)
        off, poff = _u32(page_table_offsets)
        sl, psl = _u32(seq_lens)
        qp, pqp = _u32(q_positions)
        # metal_runtime.mm:7746-7748: vector-size rules a raw-pointer ABI cannot see
        if off.size != batch + 1 or sl.size != batch or qp.size != batch:
            return self.status(1)
        return self.status(fn(self._h, _vp(_ptr(q)), _vp(_ptr(k_pages)), _vp(_ptr(v_pages)), _vp(_ptr(o)),
                              pflat, flat.size, poff, psl, pqp, batch, num_heads, kv_heads, head_dim,
                              page_size_tokens, 1 if apply_causal else 0, float(scale), q_dtype, o_dtype,
                              capacity_pages))

    def runPagedFlashAttention(self, q, k_pages, v_pages, o, page_tables_flat, page_table_offsets, seq_lens,
                               q_positions, batch, num_heads, kv_heads, head_dim, page_size_tokens,
                               apply_causal, scale: float = 0.0, q_dtype: int = MLC_F32,
                               o_dtype: int = MLC_F32, capacity_pages: int = 0) -> bool:
        return self._attention(self._lib.mlc_run_paged_flash_attention, q, k_pages, v_pages, o,
                               page_tables_flat, page_table_offsets, seq_lens, q_positions, batch, num_heads,
                               kv_heads, head_dim, page_size_tokens, apply_causal, scale, q_dtype, o_dtype,
                               capacity_pages)

    def encodePagedFlashAttention(self, q, k_pages, v_pages, o, page_tables_flat, page_table_offsets,
                                  seq_lens, q_positions, batch, num_heads, kv_heads, head_dim,
                                  page_size_tokens, apply_causal, scale: float = 0.0,
                                  q_dtype: int = MLC_F32, o_dtype: int = MLC_F32,
                                  capacity_pages: int = 0) -> bool:
        return self._attention(self._lib.mlc_encode_paged_flash_attention, q, k_pages, v_pages, o,
                               page_tables_flat, page_table_offsets, seq_lens, q_positions, batch, num_heads,
                               kv_heads, head_dim, page_size_tokens, apply_causal, scale, q_dtype, o_dtype,
                               capacity_pages)

    def _prefill(self, fn, q, k_pages, v_pages, o, page_tables_flat, page_table_offsets, seq_lens, q_start,
                 q_len, batch, num_heads, kv_heads, head_dim, page_size_tokens, scale, q_dtype, o_dtype,
                 capacity_pages) -> bool:
        flat, pflat = _u32(page_tables_flat)
        off, poff = _u32(page_table_offsets)
        sl, psl = _u32(seq_lens)
        qs, pqs = _u32(q_start)
        ql, pql = _u32(q_len)
        if off.size != batch + 1 or sl.size != batch or qs.size != batch or ql.size != batch:
            return self.status(1)
        return self.status(fn(self._h, _vp(_ptr(q)), _vp(_ptr(k_pages)), _vp(_ptr(v_pages)), _vp(_ptr(o)),
                              pflat, flat.size, poff, psl, pqs, pql, batch, num_heads, kv_heads, head_dim,
                              page_size_tokens, float(scale), q_dtype, o_dtype, capacity_pages))

    def runPagedPrefillAttention(self, q, k_pages, v_pages, o, page_tables_flat, page_table_offsets, seq_lens,
                                 q_start, q_len, batch, num_heads, kv_heads, head_dim, page_size_tokens,
                                 scale: float = 0.0, q_dtype: int = MLC_F16, o_dtype: int = MLC_F16,
                                 capacity_pages: int = 0) -> bool:
        """Chunked causal attention: query i of request r is at position q_start[r] + i.
        q / o are [sum(q_len), num_heads, head_dim]."""
        return self._prefill(self._lib.mlc_run_paged_prefill_attention, q, k_pages, v_pages, o, page_tables_flat,
                             page_table_offsets, seq_lens, q_start, q_len, batch, num_heads, kv_heads, head_dim,
                             page_size_tokens, scale, q_dtype, o_dtype, capacity_pages)

    def encodePagedPrefillAttention(self, q, k_pages, v_pages, o, page_tables_flat, page_table_offsets, seq_lens,
                                    q_start, q_len, batch, num_heads, kv_heads, head_dim, page_size_tokens,
                                    scale: float = 0.0, q_dtype: int = MLC_F16, o_dtype: int = MLC_F16,
                                    capacity_pages: int = 0) -> bool:
        return self._prefill(self._lib.mlc_encode_paged_prefill_attention, q, k_pages, v_pages, o,
                             page_tables_flat, page_table_offsets, seq_lens, q_start, q_len, batch, num_heads,
                             kv_heads, head_dim, page_size_tokens, scale, q_dtype, o_dtype, capacity_pages)

    def readTrace(self, previous: bool = False) -> np.ndarray:
        """[ctas, 4, 8] uint64 nanosecond stamps of the last traced decode launch
        (or, with previous=True, of the launch before it)."""
        buf = np.zeros(1 << 15, np.uint64)
        n = self._lib.mlc_ctx_read_trace(self._h, buf.ctypes.data_as(C.POINTER(C.c_uint64)), buf.size,
                                         1 if previous else 0)
        return buf[: n * 32].reshape(n, 4, 8)

    def lastAttentionKernel(self) -> int:
        return int(self._lib.mlc_ctx_last_attention_kernel(self._h))

    # -- device-resident plans -------------------------------------------------------
    def createPlan(self, page_tables_flat, page_table_offsets, seq_lens, q_positions, batch, num_heads,
                   kv_heads, head_dim, page_size_tokens, apply_causal=True, capacity_pages=0,
                   page_ids=None, slots_in_page=None) -> "Plan":
        flat, pflat = _u32(page_tables_flat)
        off, poff = _u32(page_table_offsets)
        sl, psl = _u32(seq_lens)
        qp, pqp = _u32(q_positions)
        if off.size != batch + 1 or sl.size != batch or qp.size != batch:
            raise MlcError(1, "table sizes do not match batch")
        pids = pslots = None
        if page_ids is not None:
            ids, pids = _u32(page_ids)
            sls, pslots = _u32(slots_in_page)
            if ids.size != batch or sls.size != batch:
                raise MlcError(1, "page_ids / slots_in_page sizes do not match batch")
        h = _vp()
        self.check(self._lib.mlc_attn_plan_create(self._h, pflat, flat.size, poff, psl, pqp, pids, pslots, batch,
                                                  num_heads, kv_heads, head_dim, page_size_tokens,
                                                  1 if apply_causal else 0, capacity_pages, C.byref(h)))
        return Plan(self, h)

    def encodePagedFlashAttentionPlanned(self, plan, q, k_pages, v_pages, o, scale=0.0, q_dtype=MLC_F32,
                                         o_dtype=MLC_F32) -> bool:
        return self.status(self._lib.mlc_encode_paged_flash_attention_planned(
            self._h, plan.handle, _vp(_ptr(q)), _vp(_ptr(k_pages)), _vp(_ptr(v_pages)), _vp(_ptr(o)),
            float(scale), q_dtype, o_dtype))

    def encodePagedDecodeStepPlanned(self, plan, q, k_new, v_new, k_pages, v_pages, o, scale=0.0,
                                     q_dtype=MLC_F32, o_dtype=MLC_F32) -> bool:
        return self.status(self._lib.mlc_encode_paged_decode_step_planned(
            self._h, plan.handle, _vp(_ptr(q)), _vp(_ptr(k_new)), _vp(_ptr(v_new)), _vp(_ptr(k_pages)),
            _vp(_ptr(v_pages)), _vp(_ptr(o)), float(scale), q_dtype, o_dtype))

    def encodePagedFlashAttentionPlannedStatic(self, plan, q, k_pages, v_pages, o, scale=0.0, q_dtype=MLC_F32,
                                               o_dtype=MLC_F32) -> bool:
        """Same as encodePagedFlashAttentionPlanned, but allocates nothing: the split-KV
        scratch is the library's fixed 8 MiB array (see include/mlc_b200.h for the limits)."""
        return self.status(self._lib.mlc_encode_paged_flash_attention_planned_static(
            self._h, plan.handle, _vp(_ptr(q)), _vp(_ptr(k_pages)), _vp(_ptr(v_pages)), _vp(_ptr(o)),
            float(scale), q_dtype, o_dtype))

    def staticScratchBytes(self) -> int:
        return int(self._lib.mlc_static_scratch_bytes())

    @staticmethod
    def pointerArray(buffers):
        """A C array of device pointers (void* const*) for the per-layer entry points; keep it alive
        as long as it is used and rebuild it only when a buffer moves."""
        arr = (_vp * len(buffers))(*[_vp(_ptr(b)) for b in buffers])
        return arr

    def encodePagedDecodePassPlanned(self, plan, q, k_new, v_new, k_pages, v_pages, o, scale=0.0,
                                     q_dtype=MLC_F32, o_dtype=MLC_F32) -> bool:
        """All layers of a decode pass in one call: q / k_new / v_new / k_pages / v_pages / o are
        pointer arrays (pointerArray) with one entry per layer."""
        return self.status(self._lib.mlc_encode_paged_decode_pass_planned(
            self._h, plan.handle, len(q), q, k_new, v_new, k_pages, v_pages, o, float(scale), q_dtype, o_dtype))

    def encodePagedDecodePassHost(self, plan, host_in, dev_in, k_pages, v_pages, dev_o, host_o, scale=0.0,
                                  q_dtype=MLC_F32, o_dtype=MLC_F32, n_groups=0) -> bool:
        """A decode pass whose activations live in host memory: host_in holds one packed row
        [Q | new K | new V] per layer (pinned memory lets the copies overlap the kernels), dev_in is a
        device staging buffer of the same size, k_pages / v_pages are pointer arrays with one pool per
        layer, O goes to dev_o and from there to host_o. Complete when flushForwardPassCB returns."""
        return self.status(self._lib.mlc_encode_paged_decode_pass_host(
            self._h, plan.handle, len(k_pages), _vp(_ptr(host_in)), _vp(_ptr(dev_in)), k_pages, v_pages,
            _vp(_ptr(dev_o)), _vp(_ptr(host_o)), float(scale), q_dtype, o_dtype, n_groups))

    # -- the ops of the walker step around attention (metal_runtime.hpp:474-506, 549-552) --------
    # Weights are device buffers here (the reference takes host vectors and caches them on the
    # device by name: getOrAllocCachedBuffer + uploadToBuffer do the same).
    def encodeRmsNormBatched(self, in_buf, weight_buf, epsilon, batch, length, out_buf, out_f16_buf=None) -> bool:
        """metal_runtime.hpp:474-479. weight_buf: device fp32 [length]."""
        return self.status(self._lib.mlc_encode_rms_norm_batched(
            self._h, _vp(_ptr(in_buf)), _vp(_ptr(weight_buf)), epsilon, batch, length, _vp(_ptr(out_buf)),
            _vp(_ptr(out_f16_buf)) if out_f16_buf is not None else None))

    def encodeMatMulQ4_0Batched(self, weights_buf, in_buf, batch, rows, cols, row_stride, out_buf) -> bool:
        """metal_runtime.hpp:481-489 (without weight_name / quant_version: the weights are already a device buffer)."""
        return self.status(self._lib.mlc_encode_matmul_q4_0_batched(
            self._h, _vp(_ptr(weights_buf)), _vp(_ptr(in_buf)), batch, rows, cols, row_stride, _vp(_ptr(out_buf))))

    def encodeMatMulQ6KBatched(self, weights_buf, in_buf, batch, rows, cols, row_stride, out_buf) -> bool:
        """metal_runtime.hpp:491-498."""
        return self.status(self._lib.mlc_encode_matmul_q6k_batched(
            self._h, _vp(_ptr(weights_buf)), _vp(_ptr(in_buf)), batch, rows, cols, row_stride, _vp(_ptr(out_buf))))

    def encodeRmsNormBatchedPacked(self, in_buf, weight_buf, epsilon, batch, length, out_buf, packed_buf) -> bool:
        """RMSNorm into the mat-vec kernel's operand format (input_kind 2 of encodeMatMulQuantFused); out_buf may be None."""
        return self.status(self._lib.mlc_encode_rms_norm_batched_packed(
            self._h, _vp(_ptr(in_buf)), _vp(_ptr(weight_buf)), epsilon, batch, length,
            _vp(_ptr(out_buf)) if out_buf is not None else None, _vp(_ptr(packed_buf))))

    def encodeMatMulQuantFused(self, quant, weights_buf, in_buf, in_stride, input_kind, residual_buf, batch, rows,
                               cols, row_stride, out_buf) -> bool:
        """The mat-vec with its input computed on load (input_kind 1: SiLU(gate) * up; True counts as 1) or already in
        operand format (2), and / or the residual add in its epilogue."""
        return self.status(self._lib.mlc_encode_matmul_quant_fused(
            self._h, quant, _vp(_ptr(weights_buf)), _vp(_ptr(in_buf)), in_stride, int(input_kind),
            _vp(_ptr(residual_buf)) if residual_buf is not None else None, batch, rows, cols, row_stride,
            _vp(_ptr(out_buf))))

    def encodeMatMulGateUpSiluPacked(self, quant, weights_buf, in_buf, in_stride, input_kind, batch, ffn_inner, cols,
                                     row_stride, packed_buf) -> bool:
        """gate | up projection with SiLU(gate) * up in its epilogue, written in operand format [batch, ffn_inner]."""
        return self.status(self._lib.mlc_encode_matmul_gate_up_silu_packed(
            self._h, quant, _vp(_ptr(weights_buf)), _vp(_ptr(in_buf)), in_stride, int(input_kind), batch, ffn_inner, cols,
            row_stride, _vp(_ptr(packed_buf))))

    def encodeArgmaxRows(self, logits_buf, batch, vocab, group_rows, out_ids) -> bool:
        """Index of the first maximum per request (uint32), logits plain [batch, vocab] or in the walker's groups."""
        return self.status(self._lib.mlc_encode_argmax_rows(self._h, _vp(_ptr(logits_buf)), batch, vocab, group_rows,
                                                            _vp(_ptr(out_ids))))

    def encodeAddBatched(self, a_buf, b_buf, out_buf, total_elements) -> bool:
        """metal_runtime.hpp:501-502."""
        return self.status(self._lib.mlc_encode_add_batched(self._h, _vp(_ptr(a_buf)), _vp(_ptr(b_buf)),
                                                            _vp(_ptr(out_buf)), total_elements))

    def encodeSiluMulBatched(self, gate_buf, up_buf, out_buf, total_elements) -> bool:
        """metal_runtime.hpp:505-506."""
        return self.status(self._lib.mlc_encode_silu_mul_batched(self._h, _vp(_ptr(gate_buf)), _vp(_ptr(up_buf)),
                                                                 _vp(_ptr(out_buf)), total_elements))

    def encodeGateUpSplitSiluMul(self, gate_up_buf, gate_buf, up_buf, out_buf, batch, ffn_inner, ffn_gate_up_rows) -> bool:
        """metal_runtime.hpp:549-552; gate_buf / up_buf may be None."""
        opt = lambda b: _vp(_ptr(b)) if b is not None else None
        return self.status(self._lib.mlc_encode_gate_up_split_silu_mul(
            self._h, _vp(_ptr(gate_up_buf)), opt(gate_buf), opt(up_buf), _vp(_ptr(out_buf)), batch, ffn_inner,
            ffn_gate_up_rows))

    def encodeQkvSplitRopeCast(self, qkv_buf, q_buf, k_buf, v_buf, k_f16_buf, v_f16_buf, cos_buf, sin_buf, batch,
                               num_heads, kv_heads, head_dim, qkv_rows, q_rows, k_rows, v_rows, rotary_dim) -> bool:
        """metal_runtime.hpp:540-547, one launch instead of seven dispatches."""
        return self.status(self._lib.mlc_encode_qkv_split_rope_cast(
            self._h, _vp(_ptr(qkv_buf)), _vp(_ptr(q_buf)), _vp(_ptr(k_buf)), _vp(_ptr(v_buf)), _vp(_ptr(k_f16_buf)),
            _vp(_ptr(v_f16_buf)), _vp(_ptr(cos_buf)), _vp(_ptr(sin_buf)), batch, num_heads, kv_heads, head_dim,
            qkv_rows, q_rows, k_rows, v_rows, rotary_dim))

    def encodeQkvSplitRopeScatterPlanned(self, plan, qkv_buf, q_out, q_dtype, k_storage, v_storage, cos_buf, sin_buf,
                                         qkv_rows, rotary_dim) -> bool:
        """Split + rotate + cast + scatter of the step's K/V rows into the pools, one launch."""
        return self.status(self._lib.mlc_encode_qkv_split_rope_scatter_planned(
            self._h, plan.handle, _vp(_ptr(qkv_buf)), _vp(_ptr(q_out)), q_dtype, _vp(_ptr(k_storage)),
            _vp(_ptr(v_storage)), _vp(_ptr(cos_buf)), _vp(_ptr(sin_buf)), qkv_rows, rotary_dim))

    def encodeMatMulQkvRopeScatterPlanned(self, plan, quant, weights_buf, in_buf, in_stride, input_kind, cols, row_stride,
                                          q_out, k_storage, v_storage, cos_buf, sin_buf, rotary_dim) -> bool:
        """The fused Q | K | V projection with split + rotate + cast + page write in its epilogue, one launch."""
        return self.status(self._lib.mlc_encode_matmul_qkv_rope_scatter_planned(
            self._h, plan.handle, quant, _vp(_ptr(weights_buf)), _vp(_ptr(in_buf)), in_stride, int(input_kind), cols,
            row_stride, _vp(_ptr(q_out)), _vp(_ptr(k_storage)), _vp(_ptr(v_storage)), _vp(_ptr(cos_buf)),
            _vp(_ptr(sin_buf)), rotary_dim))

    def computeRotaryCoefficients(self, position, rotary_dim, freq_base=10000.0, freq_scale=1.0):
        """quantization.cpp:795-823: (cos, sin) float32 [rotary_dim // 2]."""
        c, s = np.zeros(rotary_dim // 2, np.float32), np.zeros(rotary_dim // 2, np.float32)
        fp = C.POINTER(C.c_float)
        self.check(self._lib.mlc_compute_rotary_coefficients(position, rotary_dim, float(freq_base), float(freq_scale),
                                                             c.ctypes.data_as(fp), s.ctypes.data_as(fp)))
        return c, s

    def encodeScatterKVPairPlanned(self, plan, k_storage, v_storage, k_src, v_src) -> bool:
        return self.status(self._lib.mlc_encode_scatter_kv_pair_planned(
            self._h, plan.handle, _vp(_ptr(k_storage)), _vp(_ptr(v_storage)), _vp(_ptr(k_src)), _vp(_ptr(v_src))))

    def encodePagedAttentionPartialPlanned(self, plan, q, k_pages, v_pages, o_partial, ml_partial, scale=0.0,
                                           q_dtype=MLC_F32) -> bool:
        return self.status(self._lib.mlc_encode_paged_attention_partial_planned(
            self._h, plan.handle, _vp(_ptr(q)), _vp(_ptr(k_pages)), _vp(_ptr(v_pages)), _vp(_ptr(o_partial)),
            _vp(_ptr(ml_partial)), float(scale), q_dtype))

    def encodeLseCombine(self, o_parts, ml_parts, parts, rows, head_dim, out, o_dtype=MLC_F32) -> bool:
        return self.status(self._lib.mlc_encode_lse_combine(
            self._h, _vp(_ptr(o_parts)), _vp(_ptr(ml_parts)), parts, rows, head_dim, _vp(_ptr(out)), o_dtype))

    # -- CUDA graphs -------------------------------------------------------------------
    def beginCapture(self) -> bool:
        return self.status(self._lib.mlc_graph_begin_capture(self._h))

    def endCapture(self) -> "Graph":
        h = _vp()
        self.check(self._lib.mlc_graph_end_capture(self._h, C.byref(h)))
        return Graph(self, h)


class Plan:
    def __init__(self, ex: Executor, handle):
        self._ex, self.handle = ex, handle

    def update(self, page_tables_flat, page_table_offsets, seq_lens, q_positions, page_ids=None,
               slots_in_page=None) -> bool:
        """New tables (next decode step) into the same plan object; its buffers are reused."""
        flat, pflat = _u32(page_tables_flat)
        off, poff = _u32(page_table_offsets)
        sl, psl = _u32(seq_lens)
        qp, pqp = _u32(q_positions)
        ids = sl_in = None
        pids = pslots = None
        if page_ids is not None:
            ids, pids = _u32(page_ids)
            sl_in, pslots = _u32(slots_in_page)
        if off.size != sl.size + 1 or qp.size != sl.size:
            return self._ex.status(1)
        return self._ex.status(self._ex._lib.mlc_attn_plan_update(
            self._ex._h, self.handle, pflat, flat.size, poff, psl, pqp, pids, pslots, sl.size))

    def destroy(self):
        if self.handle and self._ex._h:
            self._ex._lib.mlc_attn_plan_destroy(self._ex._h, self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class PeerExchange:
    """Gather buffer of one rank for the peer-memory exchange + combine kernel."""
    HANDLE_BYTES = 64

    def __init__(self, ex: Executor, rank: int, world: int, max_rows: int, head_dim: int):
        self._ex = ex
        h = _vp()
        ex.check(ex._lib.mlc_exchange_create(ex._h, rank, world, max_rows, head_dim, C.byref(h)))
        self.handle, self.rank, self.world = h, rank, world

    def ipc_handle(self) -> bytes:
        buf = (C.c_ubyte * self.HANDLE_BYTES)()
        self._ex.check(self._ex._lib.mlc_exchange_handle(self._ex._h, self.handle, C.cast(buf, _vp)))
        return bytes(buf)

    def attach(self, handles: list[bytes]):
        assert len(handles) == self.world and all(len(h) == self.HANDLE_BYTES for h in handles)
        blob = b"".join(handles)
        buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
        self._ex.check(self._ex._lib.mlc_exchange_attach(self._ex._h, self.handle, C.cast(buf, _vp)))

    def read_trace(self) -> np.ndarray:
        """ns stamps of CTA 0 of the last exchange kernel (context created with MLC_B200_TRACE=1)."""
        buf = np.zeros(8, np.uint64)
        self._ex.check(self._ex._lib.mlc_exchange_read_trace(self._ex._h, buf.ctypes.data_as(C.POINTER(C.c_uint64))))
        return buf

    def local_buffer(self) -> int:
        return int(self._ex._lib.mlc_exchange_local_buffer(self.handle) or 0)

    def slot_floats(self) -> int:
        return int(self._ex._lib.mlc_exchange_slot_floats(self.handle))

    def attach_pointers(self, bases: list[int]):
        """Peers in this process: bases[r] = local_buffer() of rank r's exchange object."""
        assert len(bases) == self.world
        arr = (_vp * self.world)(*[_vp(b) for b in bases])
        self._ex.check(self._ex._lib.mlc_exchange_attach_pointers(self._ex._h, self.handle, arr))

    def attach_with_torch_distributed(self, group=None):
        """Exchanges the handles with torch.distributed.all_gather_object and attaches."""
        import torch.distributed as dist
        if self.world == 1:
            return
        handles = [None] * self.world
        dist.all_gather_object(handles, self.ipc_handle(), group=group)
        self.attach(handles)

    def encodeAttentionExchange(self, plan, q, k_pages, v_pages, out, scale=0.0, q_dtype=MLC_F32, o_dtype=MLC_F32) -> bool:
        """Partial attention over this rank's slice + exchange + combine in one launch; `out` is the full
        attention output on every rank."""
        return self._ex.status(self._ex._lib.mlc_encode_paged_attention_exchange_planned(
            self._ex._h, plan.handle, self.handle, _vp(_ptr(q)), _vp(_ptr(k_pages)), _vp(_ptr(v_pages)), _vp(_ptr(out)),
            float(scale), q_dtype, o_dtype))

    def encodeLseCombine(self, o_partial, ml_partial, rows, out, o_dtype=MLC_F32) -> bool:
        return self._ex.status(self._ex._lib.mlc_encode_exchange_lse_combine(
            self._ex._h, self.handle, _vp(_ptr(o_partial)), _vp(_ptr(ml_partial)), rows, _vp(_ptr(out)), o_dtype))

    def destroy(self):
        if self.handle and self._ex._h:
            self._ex._lib.mlc_exchange_destroy(self._ex._h, self.handle)
        self.handle = None


class Graph:
    def __init__(self, ex: Executor, handle):
        self._ex, self.handle = ex, handle

    def launch(self):
        self._ex.check(self._ex._lib.mlc_graph_launch(self._ex._h, self.handle))

    def destroy(self):
        if self.handle and self._ex._h:
            self._ex._lib.mlc_graph_destroy(self._ex._h, self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
