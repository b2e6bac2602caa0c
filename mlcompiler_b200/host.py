"""ctypes binding of the host-side objects of include/mlc_b200.h under the reference's
class and method names (compiler/runtime/paged_kv.hpp, batched_executor.hpp,
scheduler.hpp), so that the host-logic tests read like the reference's
tests/test_paged_kv.cpp and tests/test_scheduler.cpp. None of these needs a GPU except
PagedKVStorage.initialize and the paged executor's passes.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .capi import load_library

_vp, _sz, _u32, _u64, _i = C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint64, C.c_int
_u32p, _u64p, _fp, _szp = C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_float), C.POINTER(C.c_size_t)


class RequestSlotC(C.Structure):
    _fields_ = [("request_id", _u32), ("input_token", _u64), ("sequence_position", _u64)]


class DecodeRowC(C.Structure):
    _fields_ = [("request_id", _u32), ("success", _i), ("logits", _fp), ("n_logits", _sz)]


RUN_DECODE_CB = C.CFUNCTYPE(_sz, _vp, C.POINTER(RequestSlotC), _sz, C.POINTER(DecodeRowC))
RUN_PREFILL_CB = C.CFUNCTYPE(_sz, _vp, _u32, _u64p, _sz, C.POINTER(_fp))
RELEASE_CB = C.CFUNCTYPE(None, _vp, _u32)
TOKEN_CB = C.CFUNCTYPE(None, _vp, _u32, _u64)


class LayerWeightsC(C.Structure):
    _fields_ = [(n, _vp) for n in ("attn_norm", "attn_qkv", "attn_output", "ffn_norm", "ffn_gate_up", "ffn_down")]


class ModelDescC(C.Structure):
    _fields_ = [("hidden_size", _u32), ("ffn_inner", _u32), ("vocab_size", _u32), ("rotary_dim", _u32),
                ("rope_base", C.c_float), ("rope_scale", C.c_float), ("rms_epsilon", C.c_float),
                ("lm_head_quant", C.c_int32), ("token_embd", _vp), ("output_norm", _vp), ("lm_head", _vp),
                ("layers", C.POINTER(LayerWeightsC)), ("n_layers", _u32)]


class ExecutorCallbacksC(C.Structure):
    _fields_ = [("user", _vp), ("run_decode", RUN_DECODE_CB), ("run_prefill", RUN_PREFILL_CB),
                ("release_request", RELEASE_CB)]


_PROTOTYPES = {
    "mlc_page_pool_create": (_vp, [_u32]),
    "mlc_page_pool_destroy": (None, [_vp]),
    "mlc_page_pool_allocate": (_i, [_vp, _u32p]),
    "mlc_page_pool_allocate_n": (_i, [_vp, _sz, _u32p]),
    "mlc_page_pool_release": (_i, [_vp, _u32]),
    "mlc_page_pool_capacity": (_u32, [_vp]),
    "mlc_page_pool_in_use": (_sz, [_vp]),
    "mlc_page_pool_free": (_sz, [_vp]),
    "mlc_kv_state_create": (_vp, [_u32, _u32]),
    "mlc_kv_state_destroy": (None, [_vp]),
    "mlc_kv_state_reserve": (_i, [_vp, _vp, _sz]),
    "mlc_kv_state_extend_one_token": (_i, [_vp, _vp, _u32p, _u32p]),
    "mlc_kv_state_locate": (_i, [_vp, _sz, _u32p, _u32p]),
    "mlc_kv_state_release_all": (None, [_vp, _vp]),
    "mlc_kv_state_total_tokens": (_sz, [_vp]),
    "mlc_kv_state_tokens_in_last_page": (_u32, [_vp]),
    "mlc_kv_state_page_table": (_sz, [_vp, _u32p, _sz]),
    "mlc_kv_storage_create": (_vp, [_vp, _u32, _u32, _u32, _u32, _u32, _u32]),
    "mlc_kv_storage_destroy": (None, [_vp]),
    "mlc_kv_storage_initialize": (_i, [_vp]),
    "mlc_kv_storage_k_buffer": (_vp, [_vp, _sz]),
    "mlc_kv_storage_v_buffer": (_vp, [_vp, _sz]),
    "mlc_kv_storage_page_bytes": (_sz, [_vp]),
    "mlc_paged_executor_create": (_vp, [_vp, _u32, _u32, _u32, _u32, _u64]),
    "mlc_callback_executor_create": (_vp, [C.POINTER(ExecutorCallbacksC)]),
    "mlc_executor_destroy": (None, [_vp]),
    "mlc_executor_attach_page_pool": (_i, [_vp, _vp, _u32]),
    "mlc_executor_attach_paged_storage": (_i, [_vp, _vp]),
    "mlc_executor_set_call_order": (_i, [_vp, _i]),
    "mlc_executor_attach_model": (_i, [_vp, C.POINTER(ModelDescC)]),
    "mlc_executor_assume_context": (_i, [_vp, _u32, _sz]),
    "mlc_gguf_open": (_vp, [C.c_char_p, C.c_char_p, _sz]),
    "mlc_gguf_close": (None, [_vp]),
    "mlc_gguf_concatenate_block_weights": (_i, [_vp, C.c_char_p, _sz]),
    "mlc_gguf_describe": (_sz, [_vp, C.c_char_p, _sz]),
    "mlc_gguf_tensor_data": (C.c_int64, [_vp, C.c_char_p, _vp, _sz, C.c_char_p, _sz]),
    "mlc_executor_attach_gguf": (_i, [_vp, _vp, C.c_char_p, _sz]),
    "mlc_tokenizer_create": (_vp, [_vp]),
    "mlc_tokenizer_destroy": (None, [_vp]),
    "mlc_tokenizer_info": (_i, [_vp, _szp, _u64p, _u64p, _u64p]),
    "mlc_tokenizer_encode": (_sz, [_vp, C.c_char_p, _sz, _i, _i, _u64p, _sz]),
    "mlc_tokenizer_decode": (_sz, [_vp, _u64p, _sz, C.c_char_p, _sz]),
    "mlc_tokenizer_token_string": (_sz, [_vp, _u64, C.c_char_p, _sz]),
    "mlc_tokenizer_token_flags": (_i, [_vp, _u64]),
    "mlc_executor_run_decode": (_sz, [_vp, C.POINTER(RequestSlotC), _sz, C.POINTER(C.c_uint8), _fp, _sz]),
    "mlc_executor_run_decode_greedy": (_sz, [_vp, C.POINTER(RequestSlotC), _sz, _u64p]),
    "mlc_executor_run_prefill": (_sz, [_vp, _u32, _u64p, _sz, _fp, _sz]),
    "mlc_executor_release_request": (None, [_vp, _u32]),
    "mlc_executor_live_request_count": (_sz, [_vp]),
    "mlc_executor_known_position": (_sz, [_vp, _u32]),
    "mlc_executor_page_table": (_sz, [_vp, _u32, _u32p, _sz, _szp]),
    "mlc_hash_qkv_value": (C.c_float, [_u64, _u32, _u64, _u64, _u32, _u32, _u32]),
    "mlc_scheduler_create": (_vp, [_vp, _sz]),
    "mlc_scheduler_destroy": (None, [_vp]),
    "mlc_scheduler_add_request": (_u32, [_vp, _u64p, _sz, _sz, C.c_int64]),
    "mlc_scheduler_set_token_callback": (None, [_vp, TOKEN_CB, _vp]),
    "mlc_scheduler_tick": (_i, [_vp]),
    "mlc_scheduler_set_prefill_chunk_tokens": (None, [_vp, _sz]),
    "mlc_scheduler_prefill_calls": (_sz, [_vp]),
    "mlc_scheduler_run_until_idle": (_sz, [_vp]),
    "mlc_scheduler_empty": (_i, [_vp]),
    "mlc_scheduler_queued_count": (_sz, [_vp]),
    "mlc_scheduler_active_count": (_sz, [_vp]),
    "mlc_scheduler_completed_count": (_sz, [_vp]),
    "mlc_scheduler_stats": (None, [_vp, _szp, _szp, _szp]),
    "mlc_scheduler_drain_completed": (_sz, [_vp]),
    "mlc_scheduler_drained_request": (_i, [_vp, _sz, _u32p, C.POINTER(_i), _szp, _u64p, _sz]),
}

_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        l = load_library()
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _LIB = l
    return _LIB


class PagePool:
    def __init__(self, capacity: int):
        self._h = _vp(lib().mlc_page_pool_create(capacity))

    def __del__(self):
        if getattr(self, "_h", None) and _LIB is not None:
            _LIB.mlc_page_pool_destroy(self._h)
            self._h = None

    def allocate(self):
        """Page id, or None when the pool is exhausted (std::nullopt in the reference)."""
        v = _u32(0)
        return v.value if lib().mlc_page_pool_allocate(self._h, C.byref(v)) else None

    def allocate_n(self, n: int, out: list) -> bool:
        buf = (C.c_uint32 * max(n, 1))()
        if not lib().mlc_page_pool_allocate_n(self._h, n, buf):
            return False
        out.extend(buf[i] for i in range(n))
        return True

    def release(self, page_id: int) -> bool:
        return bool(lib().mlc_page_pool_release(self._h, page_id))

    def capacity(self) -> int:
        return lib().mlc_page_pool_capacity(self._h)

    def pages_in_use(self) -> int:
        return lib().mlc_page_pool_in_use(self._h)

    def pages_free(self) -> int:
        return lib().mlc_page_pool_free(self._h)


class RequestKVState:
    def __init__(self, page_size_tokens: int = 64, request_id: int = 0):
        self._h = _vp(lib().mlc_kv_state_create(request_id, page_size_tokens))

    def __del__(self):
        if getattr(self, "_h", None) and _LIB is not None:
            _LIB.mlc_kv_state_destroy(self._h)
            self._h = None

    def reserve(self, pool: PagePool, target_tokens: int) -> bool:
        return bool(lib().mlc_kv_state_reserve(self._h, pool._h, target_tokens))

    def extend_one_token(self, pool: PagePool):
        p, s = _u32(0), _u32(0)
        ok = lib().mlc_kv_state_extend_one_token(self._h, pool._h, C.byref(p), C.byref(s))
        return (p.value, s.value) if ok else None

    def locate(self, pos: int):
        p, s = _u32(0), _u32(0)
        ok = lib().mlc_kv_state_locate(self._h, pos, C.byref(p), C.byref(s))
        return (p.value, s.value) if ok else None

    def release_all(self, pool: PagePool):
        lib().mlc_kv_state_release_all(self._h, pool._h)

    def total_tokens(self) -> int:
        return lib().mlc_kv_state_total_tokens(self._h)

    @property
    def tokens_in_last_page(self) -> int:
        return lib().mlc_kv_state_tokens_in_last_page(self._h)

    @property
    def page_table(self) -> list:
        n = lib().mlc_kv_state_page_table(self._h, None, 0)
        buf = (C.c_uint32 * max(n, 1))()
        lib().mlc_kv_state_page_table(self._h, buf, n)
        return [buf[i] for i in range(n)]


class PagedKVStorage:
    def __init__(self, executor, capacity_pages, n_layers, page_size_tokens, n_kv_heads, head_dim, dtype_bytes=2):
        self._ex = executor
        self._h = _vp(lib().mlc_kv_storage_create(executor.handle, capacity_pages, n_layers, page_size_tokens,
                                                   n_kv_heads, head_dim, dtype_bytes))
        self.capacity_pages, self.n_layers = capacity_pages, n_layers

    def destroy(self):
        if getattr(self, "_h", None) and _LIB is not None and self._ex._h:
            _LIB.mlc_kv_storage_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def initialize(self) -> bool:
        return bool(lib().mlc_kv_storage_initialize(self._h))

    def k_buffer(self, layer: int) -> int:
        return int(lib().mlc_kv_storage_k_buffer(self._h, layer) or 0)

    def v_buffer(self, layer: int) -> int:
        return int(lib().mlc_kv_storage_v_buffer(self._h, layer) or 0)

    def page_bytes(self) -> int:
        return lib().mlc_kv_storage_page_bytes(self._h)


class GgufFile:
    """frontend::GGUFLoader (compiler/frontends/gguf_loader.hpp:60-139): open + load in the constructor (raises
    RuntimeError with the loader's message), metadata and tensor directory through describe(), tensor bytes through
    tensor_data(), concatenate_block_weights() as in the reference."""

    def __init__(self, path):
        err = C.create_string_buffer(512)
        self._h = lib().mlc_gguf_open(str(path).encode(), err, len(err))
        if not self._h:
            raise RuntimeError(err.value.decode(errors="replace"))

    def close(self):
        if getattr(self, "_h", None):
            lib().mlc_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def describe(self) -> dict:
        import json
        n = lib().mlc_gguf_describe(self._h, None, 0)
        buf = C.create_string_buffer(n)
        lib().mlc_gguf_describe(self._h, buf, n)
        return json.loads(buf.value.decode("utf-8", errors="surrogateescape"))

    def concatenate_block_weights(self) -> int:
        err = C.create_string_buffer(512)
        n = lib().mlc_gguf_concatenate_block_weights(self._h, err, len(err))
        if n < 0:
            raise RuntimeError(err.value.decode(errors="replace"))
        return n

    def tensor_data(self, name: str) -> np.ndarray:
        err = C.create_string_buffer(512)
        n = lib().mlc_gguf_tensor_data(self._h, name.encode(), None, 0, err, len(err))
        if n < 0:
            raise RuntimeError(err.value.decode(errors="replace"))
        out = np.zeros(n, np.uint8)
        lib().mlc_gguf_tensor_data(self._h, name.encode(), out.ctypes.data_as(_vp), n, err, len(err))
        return out


class Tokenizer:
    """runtime::Tokenizer (compiler/runtime/tokenizer.hpp:22-77) over the vocabulary of a GgufFile. Text goes in and
    comes out as bytes (str is encoded / decoded as UTF-8)."""
    NONE = 2 ** 64 - 1

    def __init__(self, file: GgufFile):
        self._h = lib().mlc_tokenizer_create(file._h)
        if not self._h:
            raise RuntimeError("tokenizer could not be built")
        n, b, e, u = C.c_size_t(), C.c_uint64(), C.c_uint64(), C.c_uint64()
        self._valid = bool(lib().mlc_tokenizer_info(self._h, C.byref(n), C.byref(b), C.byref(e), C.byref(u)))
        self._vocab, self._bos, self._eos, self._unk = n.value, b.value, e.value, u.value

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().mlc_tokenizer_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def valid(self) -> bool:
        return self._valid

    def vocabSize(self) -> int:
        return self._vocab

    def bosId(self) -> int:
        return self._bos

    def eosId(self) -> int:
        return self._eos

    def unkId(self) -> int:
        return self._unk

    def encode(self, text, add_bos: bool = True, add_eos: bool = False) -> list:
        data = text.encode("utf-8") if isinstance(text, str) else bytes(text)
        n = lib().mlc_tokenizer_encode(self._h, data, len(data), int(add_bos), int(add_eos), None, 0)
        ids = (C.c_uint64 * max(n, 1))()
        lib().mlc_tokenizer_encode(self._h, data, len(data), int(add_bos), int(add_eos), ids, n)
        return [int(ids[i]) for i in range(n)]

    def decode_bytes(self, ids) -> bytes:
        arr = (C.c_uint64 * max(len(ids), 1))(*[int(i) for i in ids])
        n = lib().mlc_tokenizer_decode(self._h, arr, len(ids), None, 0)
        buf = C.create_string_buffer(max(n, 1))
        lib().mlc_tokenizer_decode(self._h, arr, len(ids), buf, n)
        return buf.raw[:n]

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    def tokenString(self, token_id: int) -> bytes:
        n = lib().mlc_tokenizer_token_string(self._h, token_id, None, 0)
        buf = C.create_string_buffer(max(n, 1))
        lib().mlc_tokenizer_token_string(self._h, token_id, buf, n)
        return buf.raw[:n]

    def isControlToken(self, token_id: int) -> bool:
        return bool(lib().mlc_tokenizer_token_flags(self._h, token_id) & 1)

    def isEogToken(self, token_id: int) -> bool:
        return bool(lib().mlc_tokenizer_token_flags(self._h, token_id) & 2)


class _ExecutorBase:
    _h = None

    def destroy(self):
        if self._h and _LIB is not None:
            _LIB.mlc_executor_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


class PagedAttentionExecutor(_ExecutorBase):
    """The built-in executor: page state + batched walker over the CUDA kernels."""

    def __init__(self, executor, num_heads, kv_heads, head_dim, n_layers, qkv_seed=0):
        self._ctx = executor
        self.H, self.KVH, self.D, self.L, self.seed = num_heads, kv_heads, head_dim, n_layers, qkv_seed
        self._h = _vp(lib().mlc_paged_executor_create(executor.handle, num_heads, kv_heads, head_dim, n_layers, qkv_seed))
        if not self._h:
            raise ValueError("bad executor shape")

    def attach_page_pool(self, pool: PagePool, page_size_tokens: int = 64):
        self._pool = pool
        assert lib().mlc_executor_attach_page_pool(self._h, pool._h, page_size_tokens) == 0

    def attach_paged_storage(self, storage: PagedKVStorage):
        self._storage = storage
        assert lib().mlc_executor_attach_paged_storage(self._h, storage._h) == 0

    def set_call_order(self, reference_order: bool):
        assert lib().mlc_executor_set_call_order(self._h, 1 if reference_order else 0) == 0

    def assume_context(self, request_id: int, tokens: int) -> bool:
        """Reserve pages for a context whose K/V rows the caller fills in itself; next position = tokens."""
        return lib().mlc_executor_assume_context(self._h, request_id, tokens) == 0

    def attach_model(self, model) -> bool:
        """model: a synth.SyntheticModel (or anything with its fields) whose `device` dict maps tensor names to
        device buffers. Afterwards run_decode returns vocab_size logits per request."""
        dev = model.device
        ptr = lambda name: _vp(int(dev[name].data_ptr()))
        layers = (LayerWeightsC * self.L)()
        for l in range(self.L):
            pre = f"blk.{l}."
            layers[l] = LayerWeightsC(ptr(pre + "attn_norm.weight"), ptr(pre + "attn_qkv.weight"),
                                      ptr(pre + "attn_output.weight"), ptr(pre + "ffn_norm.weight"),
                                      ptr(pre + "ffn_gate_up.weight"), ptr(pre + "ffn_down.weight"))
        desc = ModelDescC(model.hidden_size, model.ffn_inner, model.vocab_size, model.rotary_dim, model.rope_base,
                          model.rope_scale, model.rms_epsilon, 1 if model.lm_head_quant == "q6_k" else 0,
                          ptr("token_embd.weight"), ptr("output_norm.weight"), ptr("output.weight"), layers, self.L)
        self._model = (model, layers)          # the executor keeps the pointers: keep the buffers alive
        ok = lib().mlc_executor_attach_model(self._h, C.byref(desc)) == 0
        if ok:
            self._logit_count = model.vocab_size
        return ok

    def attach_gguf(self, file: GgufFile) -> bool:
        """The decoder of a GGUF file: weights uploaded into device memory the executor owns, then attached like
        attach_model. The reason of a refusal is in self.attach_error."""
        err = C.create_string_buffer(512)
        ok = lib().mlc_executor_attach_gguf(self._h, file._h, err, len(err)) == 0
        self.attach_error = err.value.decode(errors="replace")
        if ok:
            self._logit_count = file.describe()["tensors"]["token_embd.weight"]["shape"][1]
        return ok

    def _logits_rows(self, n, stride):
        """The array the library writes a pass's logits into. With a model attached it is page-locked (the rows then
        come straight from the device) and REUSED by the next call: copy what has to outlive it."""
        if not hasattr(self, "_logit_count"):
            return np.empty((n, stride), np.float32)
        buf = getattr(self, "_logits_buf", None)
        if buf is None or buf.shape[0] < n or buf.shape[1] != stride:
            try:
                import torch
                self._logits_pin = torch.empty((n, stride), dtype=torch.float32).pin_memory()
                buf = self._logits_pin.numpy()
            except Exception:
                buf = np.empty((n, stride), np.float32)
            self._logits_buf = buf
        return buf[:n]

    def run_decode(self, slots):
        """slots: [(request_id, input_token, sequence_position)] -> [(request_id, success, logits or None)]"""
        n = len(slots)
        arr = (RequestSlotC * max(n, 1))(*[RequestSlotC(*s) for s in slots])
        success = (C.c_uint8 * max(n, 1))()
        stride = getattr(self, "_logit_count", self.H * self.D)
        logits = self._logits_rows(max(n, 1), stride)          # rows are returned as views of this one array
        got = lib().mlc_executor_run_decode(self._h, arr, n, success, logits.ctypes.data_as(_fp), stride)
        return [(slots[i][0], bool(success[i]), logits[i] if success[i] else None) for i in range(got)]

    def run_decode_greedy(self, slots):
        """slots as in run_decode -> [token id or None (failed slot)], or None when the executor has no model attached
        (or runs the reference's call order): the argmax of every request's logits, taken on the device."""
        n = len(slots)
        arr = (RequestSlotC * max(n, 1))(*[RequestSlotC(*s) for s in slots])
        toks = (C.c_uint64 * max(n, 1))()
        if lib().mlc_executor_run_decode_greedy(self._h, arr, n, toks) != n or n == 0:
            return None
        return [None if int(t) == 2 ** 64 - 1 else int(t) for t in toks[:n]]

    def run_prefill(self, request_id, tokens):
        toks = (C.c_uint64 * max(len(tokens), 1))(*tokens)
        out = np.zeros(getattr(self, "_logit_count", self.H * self.D), np.float32)
        n = lib().mlc_executor_run_prefill(self._h, request_id, toks, len(tokens), out.ctypes.data_as(_fp), out.size)
        return out[:n].copy()

    def release_request(self, request_id):
        lib().mlc_executor_release_request(self._h, request_id)

    def live_request_count(self) -> int:
        return lib().mlc_executor_live_request_count(self._h)

    def known_position(self, request_id) -> int:
        return lib().mlc_executor_known_position(self._h, request_id)

    def page_state(self, request_id):
        """(page_table, total_tokens) of a tracked request, or None."""
        total = _sz(0)
        n = lib().mlc_executor_page_table(self._h, request_id, None, 0, C.byref(total))
        if n == 0:
            return None
        buf = (C.c_uint32 * n)()
        lib().mlc_executor_page_table(self._h, request_id, buf, n, C.byref(total))
        return [buf[i] for i in range(n)], total.value


class CallbackExecutor(_ExecutorBase):
    """An IBatchedExecutor implemented in Python. Subclass and override run_decode(slots) ->
    [(request_id, success, logits)], run_prefill(request_id, tokens) -> logits, release_request(id)."""

    def __init__(self):
        self._keep = []

        def _decode(user, slots, n, rows):
            out = self.run_decode([(slots[i].request_id, slots[i].input_token, slots[i].sequence_position)
                                   for i in range(n)])
            self._keep = []
            for i, (rid, ok, logits) in enumerate(out[:n]):
                rows[i].request_id = rid
                rows[i].success = 1 if ok else 0
                if ok and logits is not None:
                    a = np.ascontiguousarray(logits, dtype=np.float32)
                    self._keep.append(a)
                    rows[i].logits = a.ctypes.data_as(_fp)
                    rows[i].n_logits = a.size
                else:
                    rows[i].logits = None
                    rows[i].n_logits = 0
            return min(len(out), n)

        def _prefill(user, rid, tokens, n, logits_out):
            a = np.ascontiguousarray(self.run_prefill(rid, [tokens[i] for i in range(n)]), dtype=np.float32)
            self._keep_prefill = a
            logits_out[0] = a.ctypes.data_as(_fp)
            return a.size

        def _release(user, rid):
            self.release_request(rid)

        self._cbs = ExecutorCallbacksC(None, RUN_DECODE_CB(_decode), RUN_PREFILL_CB(_prefill), RELEASE_CB(_release))
        self._h = _vp(lib().mlc_callback_executor_create(C.byref(self._cbs)))


class Scheduler:
    QUEUED, PREFILLING, DECODING, COMPLETE, FAILED = range(5)

    def __init__(self, executor, max_batch_size: int = 8):
        self._exec = executor
        self._h = _vp(lib().mlc_scheduler_create(executor._h, max_batch_size))
        self._token_cb = None

    def __del__(self):
        if getattr(self, "_h", None) and _LIB is not None:
            _LIB.mlc_scheduler_destroy(self._h)
            self._h = None

    def add_request(self, prompt_tokens, max_new_tokens: int = 100, eos_token_id: int = -1) -> int:
        toks = (C.c_uint64 * max(len(prompt_tokens), 1))(*prompt_tokens)
        return lib().mlc_scheduler_add_request(self._h, toks, len(prompt_tokens), max_new_tokens, eos_token_id)

    def set_token_callback(self, fn):
        self._token_cb = TOKEN_CB(lambda user, rid, tok: fn(rid, tok))
        lib().mlc_scheduler_set_token_callback(self._h, self._token_cb, None)

    def set_prefill_chunk_tokens(self, tokens: int):
        """A prompt is fed at most `tokens` at a time, one chunk per tick (0: whole prompts, the reference)."""
        lib().mlc_scheduler_set_prefill_chunk_tokens(self._h, int(tokens))

    def prefill_calls(self) -> int:
        return lib().mlc_scheduler_prefill_calls(self._h)

    def tick(self) -> bool:
        return bool(lib().mlc_scheduler_tick(self._h))

    def run_until_idle(self) -> int:
        return lib().mlc_scheduler_run_until_idle(self._h)

    def empty(self) -> bool:
        return bool(lib().mlc_scheduler_empty(self._h))

    def queued_count(self) -> int:
        return lib().mlc_scheduler_queued_count(self._h)

    def active_count(self) -> int:
        return lib().mlc_scheduler_active_count(self._h)

    def completed_count(self) -> int:
        return lib().mlc_scheduler_completed_count(self._h)

    def stats(self) -> dict:
        a, b, c = _sz(0), _sz(0), _sz(0)
        lib().mlc_scheduler_stats(self._h, C.byref(a), C.byref(b), C.byref(c))
        return {"total_requests_completed": a.value, "total_decode_steps": b.value, "total_tokens_generated": c.value}

    def drain_completed(self) -> list:
        n = lib().mlc_scheduler_drain_completed(self._h)
        out = []
        for i in range(n):
            rid, state, ng = _u32(0), _i(0), _sz(0)
            lib().mlc_scheduler_drained_request(self._h, i, C.byref(rid), C.byref(state), C.byref(ng), None, 0)
            buf = (C.c_uint64 * max(ng.value, 1))()
            lib().mlc_scheduler_drained_request(self._h, i, None, None, None, buf, ng.value)
            out.append({"id": rid.value, "state": state.value, "generated_tokens": [buf[j] for j in range(ng.value)]})
        return out


def hash_qkv_value(seed, request, token, position, layer, tensor, index) -> float:
    return float(lib().mlc_hash_qkv_value(seed, request, token, position, layer, tensor, index))


def hash_qkv_tensor(seed, request, token, position, layer, tensor, n) -> np.ndarray:
    """numpy restatement of the paged executor's Q/K/V stand-in (csrc/batched_executor.cpp):
    n elements of tensor 0 (Q), 1 (K row) or 2 (V row)."""
    M = np.uint64(0xFFFFFFFFFFFFFFFF)

    def mix(x):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & M
        x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & M
        x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & M
        return x ^ (x >> np.uint64(31))

    with np.errstate(over="ignore"):
        h = mix(np.uint64(seed) ^ np.uint64(0xA24BAED4963EE407))
        h = mix(h ^ np.uint64(request))
        h = mix(h ^ np.uint64(token))
        h = mix(h ^ np.uint64(position))
        h = mix(h ^ np.uint64((layer << 8) | tensor))
        hv = mix(h ^ np.arange(n, dtype=np.uint64))
    v = ((hv >> np.uint64(20)) & np.uint64(0x7FF)).astype(np.int64) - 1024
    return (v / 1024.0).astype(np.float32)
