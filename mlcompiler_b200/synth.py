"""Seeded synthetic workloads with the shapes of the benchmark configurations.

The reference measures on no public dataset; these inputs stand in for its
TinyLlama runs (tools/paged_flash_bench.cpp:29-34 uses the same head shape).
Values are N(0,1) rounded once to fp16; the fp16 bit patterns are the ground
truth for the CPU oracle and the GPU alike. Page tables are disjoint slices of
one seeded permutation of the pool, so they are non-contiguous and unordered.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

SHAPE_A = dict(H=32, KVH=4, D=64)    # TinyLlama head shape
SHAPE_B = dict(H=32, KVH=8, D=128)   # wider GQA shape


@dataclass
class PagedCase:
    N: int
    H: int
    KVH: int
    D: int
    P: int
    capacity: int
    seq_lens: np.ndarray          # tokens per request AFTER the new token is written
    pt_flat: np.ndarray
    pt_off: np.ndarray
    q_pos: np.ndarray
    page_ids: np.ndarray          # where the step's new K/V row goes: (page, slot) per request
    slots: np.ndarray
    scale: float
    q: np.ndarray | None = None       # float16 [N, H, D]
    k_new: np.ndarray | None = None   # float16 [N, KVH, D]
    v_new: np.ndarray | None = None
    k_pool: np.ndarray | None = None  # float16 [capacity, P, KVH, D]
    v_pool: np.ndarray | None = None
    meta: dict = field(default_factory=dict)

    @property
    def kv_bytes(self) -> int:
        """Algorithmic KV bytes one attention pass reads: sum_r 2*S_r*KVH*D*2."""
        return int(self.seq_lens.astype(np.int64).sum()) * 2 * self.KVH * self.D * 2

    def tokens_of(self, r: int, pool: np.ndarray) -> np.ndarray:
        """De-paged rows [S_r, KVH, D] of request r in logical token order."""
        S = int(self.seq_lens[r])
        pages = self.pt_flat[self.pt_off[r]:self.pt_off[r + 1]]
        rows = pool[pages].reshape(-1, self.KVH, self.D)
        return rows[:S]


def make_tables(seq_lens, P: int, rng: np.random.Generator, slack: float = 0.10, capacity: int | None = None):
    seq_lens = np.asarray(seq_lens, dtype=np.uint32)
    pages = (seq_lens.astype(np.int64) + P - 1) // P
    total = int(pages.sum())
    if capacity is None:
        capacity = max(int(np.ceil(total * (1.0 + slack))), 1)
    assert capacity >= total
    perm = rng.permutation(capacity).astype(np.uint32)
    pt_off = np.zeros(len(seq_lens) + 1, np.uint32)
    pt_off[1:] = np.cumsum(pages)
    pt_flat = perm[:total].copy()
    return pt_flat, pt_off, capacity


def make_case(seed: int, seq_lens, H: int, KVH: int, D: int, P: int = 64, capacity: int | None = None,
              fill: bool = True, scale: float | None = None, q_pos=None) -> PagedCase:
    rng = np.random.default_rng(seed)
    seq_lens = np.asarray(seq_lens, dtype=np.uint32)
    N = len(seq_lens)
    pt_flat, pt_off, capacity = make_tables(seq_lens, P, rng, capacity=capacity)
    page_ids = np.zeros(N, np.uint32)
    slots = np.zeros(N, np.uint32)
    for r in range(N):
        S = int(seq_lens[r])
        if S:
            page_ids[r] = pt_flat[pt_off[r] + (S - 1) // P]
            slots[r] = (S - 1) % P
    if q_pos is None:
        q_pos = np.where(seq_lens > 0, seq_lens - 1, 0).astype(np.uint32)
    case = PagedCase(N=N, H=H, KVH=KVH, D=D, P=P, capacity=capacity, seq_lens=seq_lens, pt_flat=pt_flat,
                     pt_off=pt_off, q_pos=np.asarray(q_pos, np.uint32), page_ids=page_ids, slots=slots,
                     scale=float(scale if scale is not None else 1.0 / np.sqrt(np.float32(D))))
    if fill:
        case.q = rng.standard_normal((N, H, D), dtype=np.float32).astype(np.float16)
        case.k_new = rng.standard_normal((N, KVH, D), dtype=np.float32).astype(np.float16)
        case.v_new = rng.standard_normal((N, KVH, D), dtype=np.float32).astype(np.float16)
        case.k_pool = rng.standard_normal((capacity, P, KVH, D), dtype=np.float32).astype(np.float16)
        case.v_pool = rng.standard_normal((capacity, P, KVH, D), dtype=np.float32).astype(np.float16)
    return case


def config_lengths(config: int, seed: int | None = None) -> np.ndarray:
    """Context lengths of the numbered benchmark configurations (1-based)."""
    rng = np.random.default_rng(0xBEEF + config if seed is None else seed)
    if config == 1:
        return np.array([512], np.uint32)
    if config == 2:
        return rng.integers(64, 2048, size=32, endpoint=True).astype(np.uint32)
    if config == 3:
        return np.full(4, 32768, np.uint32)
    if config == 4:
        return rng.integers(512, 8192, size=128, endpoint=True).astype(np.uint32)
    raise ValueError(config)


def config_case(config: int, fill: bool = True, seed: int | None = None) -> PagedCase:
    shape = SHAPE_B if config == 4 else SHAPE_A
    lens = config_lengths(config, seed)
    cap = 64 if config == 1 else None
    return make_case(0xBEEF + config if seed is None else seed, lens, P=64, capacity=cap, fill=fill, **shape)


def shard_requests_by_kv_bytes(seq_lens, n_shards: int) -> list[list[int]]:
    """Greedy longest-first bin packing of requests onto shards by KV bytes."""
    order = np.argsort(-np.asarray(seq_lens, dtype=np.int64), kind="stable")
    load = [0] * n_shards
    out: list[list[int]] = [[] for _ in range(n_shards)]
    for r in order:
        i = int(np.argmin(load))
        out[i].append(int(r))
        load[i] += int(seq_lens[r])
    for lst in out:
        lst.sort()
    return out


# ---- synthetic quantised weights for the ops around attention -------------------------------------------
# The reference's walker multiplies activations with GGUF tensors in Q4_0 (projections) and Q6_K (lm_head)
# format. No model file exists here, so weight matrices are drawn directly in the quantised formats: any
# byte pattern with a finite scale is a valid matrix, and scales are chosen so that the de-quantised weights
# have about the spread of a trained projection (standard deviation ~ 1 / sqrt(cols)).
def random_q4_0(rng: np.random.Generator, rows: int, cols: int) -> np.ndarray:
    """uint8 [rows, cols / 32 * 18]: per block an fp16 scale and 16 bytes of nibbles (quantization.cpp:71-74)."""
    assert cols % 32 == 0
    nb = cols // 32
    out = np.zeros((rows, nb, 18), np.uint8)
    # nibbles uniform in 0..15 -> (q - 8) has standard deviation ~4.6; d sets the weight spread
    d = (np.abs(rng.standard_normal((rows, nb))) * 0.3 + 0.7) / (4.6 * np.sqrt(cols))
    out[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    out[:, :, 2:] = rng.integers(0, 256, size=(rows, nb, 16), dtype=np.uint8)
    return out.reshape(rows, nb * 18)


def random_q6_k(rng: np.random.Generator, rows: int, cols: int) -> np.ndarray:
    """uint8 [rows, cols / 256 * 210]: ql[128] | qh[64] | int8 scales[16] | fp16 d (quantization.cpp:142-147)."""
    assert cols % 256 == 0
    nb = cols // 256
    out = np.zeros((rows, nb, 210), np.uint8)
    out[:, :, 0:192] = rng.integers(0, 256, size=(rows, nb, 192), dtype=np.uint8)
    out[:, :, 192:208] = rng.integers(-96, 97, size=(rows, nb, 16)).astype(np.int8).view(np.uint8)
    # 6-bit values (q - 32) have standard deviation ~18.5, scales ~55
    d = (np.abs(rng.standard_normal((rows, nb))) * 0.3 + 0.7) / (18.5 * 55.0 * np.sqrt(cols))
    out[:, :, 208:210] = d.astype(np.float16).view(np.uint8).reshape(rows, nb, 2)
    return out.reshape(rows, nb * 210)


class SyntheticModel:
    """Seeded random weights of a Llama-style decoder in the tensor names and formats the reference's walker
    reads (compiler/runtime/batched_walker.cpp:183-458): Q4_0 token table and mat-vec weights, fp32 norm
    weights, Q6_K (or Q4_0) lm_head. `host` maps tensor name -> numpy array; to_device() fills `device`
    with torch tensors of the same bytes. There is no checkpoint to load in this repository's tests and
    benchmarks, so the values are synthetic; shapes and formats are the model's."""

    def __init__(self, seed, n_layers, num_heads, kv_heads, head_dim, ffn_inner, vocab_size, rotary_dim=None,
                 lm_head_quant="q6_k", rope_base=10000.0, rope_scale=1.0, rms_epsilon=1e-5):
        rng = np.random.default_rng(seed)
        self.n_layers, self.num_heads, self.kv_heads, self.head_dim = n_layers, num_heads, kv_heads, head_dim
        self.hidden_size = num_heads * head_dim
        self.ffn_inner, self.vocab_size = ffn_inner, vocab_size
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        self.lm_head_quant, self.rope_base, self.rope_scale, self.rms_epsilon = lm_head_quant, rope_base, rope_scale, rms_epsilon
        self.qkv_rows = (num_heads + 2 * kv_heads) * head_dim
        h = self.hidden_size
        t = {}
        # embedding rows of unit scale: the generic generator normalises by sqrt(cols), undo that
        emb = random_q4_0(rng, vocab_size, h).reshape(vocab_size, h // 32, 18)
        d = emb[:, :, 0:2].copy().view(np.float16).astype(np.float32) * np.sqrt(h)
        emb[:, :, 0:2] = d.astype(np.float16).view(np.uint8).reshape(vocab_size, h // 32, 2)
        t["token_embd.weight"] = emb.reshape(vocab_size, -1)
        for l in range(n_layers):
            pre = f"blk.{l}."
            t[pre + "attn_norm.weight"] = rng.uniform(0.8, 1.2, h).astype(np.float32)
            t[pre + "attn_qkv.weight"] = random_q4_0(rng, self.qkv_rows, h)
            t[pre + "attn_output.weight"] = random_q4_0(rng, h, h)
            t[pre + "ffn_norm.weight"] = rng.uniform(0.8, 1.2, h).astype(np.float32)
            t[pre + "ffn_gate_up.weight"] = random_q4_0(rng, 2 * ffn_inner, h)
            t[pre + "ffn_down.weight"] = random_q4_0(rng, h, ffn_inner)
        t["output_norm.weight"] = rng.uniform(0.8, 1.2, h).astype(np.float32)
        t["output.weight"] = random_q6_k(rng, vocab_size, h) if lm_head_quant == "q6_k" else random_q4_0(rng, vocab_size, h)
        self.host = t
        self.device = {}

    def weight_bytes(self) -> int:
        return int(sum(a.nbytes for a in self.host.values()))

    def to_device(self, device="cuda"):
        import torch
        self.device = {k: torch.from_numpy(np.ascontiguousarray(v)).to(device) for k, v in self.host.items()}
        return self

    def write_gguf(self, path, split_fused=True, version=3, alignment=32, extra_kv=None):
        """This model as a GGUF file with the keys and tensor names of a Llama checkpoint. split_fused stores
        attn_q / attn_k / attn_v and ffn_gate / ffn_up apart, as real checkpoints do (a loader then rebuilds the fused
        tensors by concatenation, compiler/frontends/gguf_loader.cpp:877-943)."""
        h, D = self.hidden_size, self.head_dim
        kv = [("general.architecture", "string", "llama"), ("general.name", "string", "synthetic"),
              ("general.alignment", "u32", alignment), ("general.quantization_version", "u32", 2),
              ("llama.block_count", "u32", self.n_layers), ("llama.embedding_length", "u32", h),
              ("llama.feed_forward_length", "u32", self.ffn_inner), ("llama.attention.head_count", "u32", self.num_heads),
              ("llama.attention.head_count_kv", "u32", self.kv_heads), ("llama.rope.dimension_count", "u32", self.rotary_dim),
              ("llama.rope.freq_base", "f32", self.rope_base), ("llama.rope.freq_scale", "f32", self.rope_scale),
              ("llama.attention.layer_norm_rms_epsilon", "f32", self.rms_epsilon)] + list(extra_kv or [])
        tensors = []
        q_rows, k_rows = self.num_heads * D, self.kv_heads * D
        for name, a in self.host.items():
            if a.dtype == np.float32:
                tensors.append((name, [a.shape[0]], GGML_F32, a))
                continue
            rows = a.shape[0]
            dtype = GGML_Q6_K if (name == "output.weight" and self.lm_head_quant == "q6_k") else GGML_Q4_0
            cols = a.shape[1] // 210 * 256 if dtype == GGML_Q6_K else a.shape[1] // 18 * 32
            if split_fused and name.endswith("attn_qkv.weight"):
                pre = name[:-len("attn_qkv.weight")]
                for part, r0, r1 in (("attn_q", 0, q_rows), ("attn_k", q_rows, q_rows + k_rows), ("attn_v", q_rows + k_rows, rows)):
                    tensors.append((pre + part + ".weight", [cols, r1 - r0], dtype, a[r0:r1]))
            elif split_fused and name.endswith("ffn_gate_up.weight"):
                pre = name[:-len("ffn_gate_up.weight")]
                tensors.append((pre + "ffn_gate.weight", [cols, rows // 2], dtype, a[:rows // 2]))
                tensors.append((pre + "ffn_up.weight", [cols, rows // 2], dtype, a[rows // 2:]))
            else:
                tensors.append((name, [cols, rows], dtype, a))
        write_gguf(path, kv, tensors, version=version, alignment=alignment)


GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q6_K = 0, 1, 2, 14
_GGUF_TYPES = {"u8": (0, "<B"), "i8": (1, "<b"), "u16": (2, "<H"), "i16": (3, "<h"), "u32": (4, "<I"), "i32": (5, "<i"),
               "f32": (6, "<f"), "bool": (7, "<B"), "u64": (10, "<Q"), "i64": (11, "<q"), "f64": (12, "<d")}


def _gguf_string(s) -> bytes:
    import struct
    b = s if isinstance(s, (bytes, bytearray)) else str(s).encode("utf-8")
    return struct.pack("<Q", len(b)) + bytes(b)


def _gguf_value(kind, value) -> bytes:
    """kind: a scalar name of _GGUF_TYPES, "string", "raw", or ("array", element kind) with a list value."""
    import struct
    if isinstance(kind, tuple):
        elem = kind[1]
        code = 9 if isinstance(elem, tuple) else 8 if elem == "string" else 13 if elem == "raw" else _GGUF_TYPES[elem][0]
        return struct.pack("<IQ", code, len(value)) + b"".join(_gguf_value(elem, v) for v in value)
    if kind in ("string", "raw"):
        return _gguf_string(value)
    return struct.pack(_GGUF_TYPES[kind][1], value)


def write_gguf(path, kv, tensors, version=3, alignment=32, tensor_padding=b"\x00"):
    """A GGUF file (version 2 or 3 layout). kv: (key, kind, value) triples, kinds as in _gguf_value; tensors:
    (name, shape fastest-first, ggml type, numpy array of the stored bytes) - stored in order, each aligned."""
    import struct
    out = bytearray(struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kv)))
    for key, kind, value in kv:
        code = 9 if isinstance(kind, tuple) else 8 if kind == "string" else 13 if kind == "raw" else _GGUF_TYPES[kind][0]
        out += _gguf_string(key) + struct.pack("<I", code) + _gguf_value(kind, value)
    offsets, cursor = [], 0
    blobs = [np.ascontiguousarray(a).view(np.uint8).reshape(-1) for _, _, _, a in tensors]
    for b in blobs:
        offsets.append(cursor)
        cursor = (cursor + b.nbytes + alignment - 1) // alignment * alignment
    for (name, shape, dtype, _), off in zip(tensors, offsets):
        out += _gguf_string(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        out += struct.pack("<IQ", dtype, off)
    out += tensor_padding * ((-len(out)) % alignment)
    with open(path, "wb") as f:
        f.write(out)
        pos = 0
        for b, off in zip(blobs, offsets):
            f.write(tensor_padding * (off - pos))
            f.write(b.tobytes())
            pos = off + b.nbytes
