// Fused QKV split + rotary embedding + fp32 -> fp16 cast (+ optional scatter into the paged pools).
//
// The reference encodes this step as 7 dispatches in one encoder
// (MetalExecutor::encodeQkvSplitRopeCast, compiler/runtime/metal_runtime.mm:7915-8025):
// 3 x strided_copy_f32 (mm:447-457) splitting each fused row [q_rows | k_rows | v_rows],
// 2 x batched_rope (mm:287-314) rotating adjacent pairs (2i, 2i+1) of every Q and K head by the
// request's cos/sin row, 2 x cast_f32_to_f16 (mm:459-466) of K and V; the two
// scatter_kv_paged_batched_f16 dispatches (mm:405-424) follow in the walker
// (compiler/runtime/batched_walker.cpp:299-309). Here it is one launch, one thread per pair, every
// input element read once; with page ids / slots given the fp16 K/V rows go straight into the pools
// and the intermediate fp32 K/V and fp16 staging buffers are optional.
//
// Arithmetic is the reference's, operation for operation in fp32 with no contraction
// (x0*c - x1*s, x0*s + x1*c: quantization.cpp:785-792 / mm:310-313), so results are bit-exact
// against the CPU restatement; the cast is round-to-nearest-even like MSL's half().
#include <cmath>

#include "qkv_rope.hpp"

namespace mlcb {

__global__ void __launch_bounds__(256) qkv_split_rope_cast_kernel(const QkvRopeParams p) {
    const uint32_t pairs_per_row = (p.q_rows + p.k_rows + p.v_rows) >> 1;
    const uint64_t gid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= static_cast<uint64_t>(p.batch) * pairs_per_row) return;
    const uint32_t r = static_cast<uint32_t>(gid / pairs_per_row);
    const uint32_t col = static_cast<uint32_t>(gid - static_cast<uint64_t>(r) * pairs_per_row) << 1;  // even column in the split row
    const float2 x = *reinterpret_cast<const float2*>(p.qkv + static_cast<size_t>(r) * p.qkv_rows + col);
    float y0 = x.x, y1 = x.y;
    const bool is_q = col < p.q_rows;
    const bool is_k = !is_q && col < p.q_rows + p.k_rows;
    const uint32_t c = is_q ? col : (is_k ? col - p.q_rows : col - p.q_rows - p.k_rows);  // column inside its part
    if (is_q || is_k) {
        const uint32_t pair = (c % p.head_dim) >> 1;
        if (pair < p.rotary_pairs) {
            const float cs = p.cos_t[static_cast<size_t>(r) * p.rotary_pairs + pair];
            const float sn = p.sin_t[static_cast<size_t>(r) * p.rotary_pairs + pair];
            y0 = __fsub_rn(__fmul_rn(x.x, cs), __fmul_rn(x.y, sn));
            y1 = __fadd_rn(__fmul_rn(x.x, sn), __fmul_rn(x.y, cs));
        }
    }
    if (is_q) {
        if (p.q) *reinterpret_cast<float2*>(p.q + static_cast<size_t>(r) * p.q_rows + c) = make_float2(y0, y1);
        if (p.q16) *reinterpret_cast<__half2*>(p.q16 + static_cast<size_t>(r) * p.q_rows + c) = __floats2half2_rn(y0, y1);
        return;
    }
    const uint32_t rows = is_k ? p.k_rows : p.v_rows;
    float* f32 = is_k ? p.k : p.v;
    __half* f16 = is_k ? p.k16 : p.v16;
    __half* pool = is_k ? p.k_pool : p.v_pool;
    const __half2 h = __floats2half2_rn(y0, y1);
    if (f32) *reinterpret_cast<float2*>(f32 + static_cast<size_t>(r) * rows + c) = make_float2(y0, y1);
    if (f16) *reinterpret_cast<__half2*>(f16 + static_cast<size_t>(r) * rows + c) = h;
    if (pool) {
        const uint32_t page = p.page_ids[r], slot = p.slots[r];
        if (page >= p.capacity) {
            if (c == 0) atomicOr(p.err, MLC_DEVERR_BAD_PAGE);
        } else if (slot >= p.page_tokens) {
            if (c == 0) atomicOr(p.err, MLC_DEVERR_BAD_SLOT);
        } else {
            // page layout [page][slot][kv_head][dim]: a request's row is `rows` contiguous halves
            *reinterpret_cast<__half2*>(pool + (static_cast<size_t>(page) * p.page_tokens + slot) * rows + c) = h;
        }
    }
}

int launch_qkv_split_rope_cast(mlc_ctx* ctx, const QkvRopeParams& p) {
    const uint64_t pairs = static_cast<uint64_t>(p.batch) * ((p.q_rows + p.k_rows + p.v_rows) >> 1);
    if (pairs == 0) return MLC_OK;
    const unsigned blocks = static_cast<unsigned>((pairs + 255) / 256);
    qkv_split_rope_cast_kernel<<<blocks, 256, 0, ctx->stream>>>(p);
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

// Shared argument rules (metal_runtime.mm:7932-7936 checks only the open pass; the shape rules are
// what the kernels above assume).
int check_qkv_rope_args(mlc_ctx* ctx, const void* qkv, const void* cos_t, const void* sin_t, size_t batch,
                        size_t num_heads, size_t kv_heads, size_t head_dim, size_t qkv_rows, size_t q_rows,
                        size_t k_rows, size_t v_rows, size_t rotary_dim) {
    if (!qkv) return ctx->fail(MLC_ERR_INVALID_ARG, "null qkv buffer");
    if (batch == 0 || head_dim == 0 || num_heads == 0 || kv_heads == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (q_rows != num_heads * head_dim || k_rows != kv_heads * head_dim || v_rows != k_rows)
        return ctx->fail(MLC_ERR_INVALID_ARG, "q_rows / k_rows / v_rows do not match heads * head_dim");
    if (qkv_rows < q_rows + k_rows + v_rows) return ctx->fail(MLC_ERR_INVALID_ARG, "qkv_rows shorter than q + k + v");
    if (head_dim % 2 || qkv_rows % 2) return ctx->fail(MLC_ERR_UNSUPPORTED, "odd head_dim or row stride");
    if (rotary_dim > head_dim || rotary_dim % 2) return ctx->fail(MLC_ERR_INVALID_ARG, "rotary_dim must be even and <= head_dim");
    if (rotary_dim > 0 && (!cos_t || !sin_t)) return ctx->fail(MLC_ERR_INVALID_ARG, "null cos / sin table");
    if (batch * qkv_rows >= (size_t(1) << 32)) return ctx->fail(MLC_ERR_UNSUPPORTED, "batch too large");
    if (reinterpret_cast<uintptr_t>(qkv) % 8) return ctx->fail(MLC_ERR_INVALID_ARG, "qkv must be 8-byte aligned");
    return MLC_OK;
}

}  // namespace mlcb

using namespace mlcb;

extern "C" {

int mlc_encode_qkv_split_rope_cast(mlc_ctx* ctx, const void* qkv, void* q, void* k, void* v, void* k_f16,
                                   void* v_f16, const void* cos_table, const void* sin_table, size_t batch,
                                   size_t num_heads, size_t kv_heads, size_t head_dim, size_t qkv_rows,
                                   size_t q_rows, size_t k_rows, size_t v_rows, size_t rotary_dim) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");  // mm:7935
    int st = check_qkv_rope_args(ctx, qkv, cos_table, sin_table, batch, num_heads, kv_heads, head_dim, qkv_rows,
                                 q_rows, k_rows, v_rows, rotary_dim);
    if (st != MLC_OK) return st;
    if (!q || !k || !v || !k_f16 || !v_f16) return ctx->fail(MLC_ERR_INVALID_ARG, "null output buffer");
    DeviceGuard guard(ctx->device);
    QkvRopeParams p{};
    p.qkv = static_cast<const float*>(qkv);
    p.q = static_cast<float*>(q);
    p.k = static_cast<float*>(k);
    p.v = static_cast<float*>(v);
    p.k16 = static_cast<__half*>(k_f16);
    p.v16 = static_cast<__half*>(v_f16);
    p.cos_t = static_cast<const float*>(cos_table);
    p.sin_t = static_cast<const float*>(sin_table);
    p.err = ctx->d_err;
    p.batch = static_cast<uint32_t>(batch);
    p.head_dim = static_cast<uint32_t>(head_dim);
    p.rotary_pairs = static_cast<uint32_t>(rotary_dim / 2);
    p.qkv_rows = static_cast<uint32_t>(qkv_rows);
    p.q_rows = static_cast<uint32_t>(q_rows);
    p.k_rows = static_cast<uint32_t>(k_rows);
    p.v_rows = static_cast<uint32_t>(v_rows);
    return launch_qkv_split_rope_cast(ctx, p);
}

// computeRotaryCoefficients (compiler/runtime/quantization.cpp:795-823), same float arithmetic.
int mlc_compute_rotary_coefficients(size_t position, size_t rotary_dim, float freq_base, float freq_scale,
                                    float* cos_out, float* sin_out) {
    if (rotary_dim < 2) return MLC_OK;
    if (!cos_out || !sin_out) return MLC_ERR_INVALID_ARG;
    if (freq_base <= 0.0f) freq_base = 10000.0f;
    if (freq_scale == 0.0f) freq_scale = 1.0f;
    const size_t pairs = rotary_dim / 2;
    const float pos = static_cast<float>(position);
    for (size_t i = 0; i < pairs; ++i) {
        const float exponent = static_cast<float>(2 * i) / static_cast<float>(rotary_dim);
        const float inv_freq = std::pow(freq_base, -exponent);
        const float angle = pos * inv_freq * freq_scale;
        cos_out[i] = std::cos(angle);
        sin_out[i] = std::sin(angle);
    }
    return MLC_OK;
}

}  // extern "C"
