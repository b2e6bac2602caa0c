// Parameters and launcher of the fused QKV split + rotary + cast (+ scatter) kernel (qkv_rope.cu).
#pragma once

#include <cuda_fp16.h>

#include "ctx.hpp"

namespace mlcb {

struct QkvRopeParams {
    const float* qkv;        // [batch, qkv_rows]
    float* q;                // [batch, q_rows] fp32, or null
    __half* q16;             // [batch, q_rows] fp16, or null
    float* k;                // [batch, k_rows] fp32, or null
    float* v;                // [batch, v_rows] fp32, or null
    __half* k16;             // [batch, k_rows] fp16, or null
    __half* v16;             // [batch, v_rows] fp16, or null
    __half* k_pool;          // paged pools, or null
    __half* v_pool;
    const uint32_t* page_ids;  // [batch] with the pools
    const uint32_t* slots;
    const float* cos_t;      // [batch, rotary_dim / 2]
    const float* sin_t;
    uint32_t* err;
    uint32_t batch, head_dim, rotary_pairs, qkv_rows, q_rows, k_rows, v_rows;
    uint32_t page_tokens, capacity;
};

int launch_qkv_split_rope_cast(mlc_ctx* ctx, const QkvRopeParams& p);
// The fused Q | K | V projection whose epilogue does what the kernel above does with its result (layer_ops.cu): q16,
// k_pool, v_pool, page_ids, slots, the tables and the sizes of `rope` are used; its qkv, fp32 and unpaged fp16
// outputs are not.
int encode_matvec_qkv_rope(mlc_ctx* ctx, int quant, int input_kind, const void* weights, const void* in, size_t in_stride,
                           size_t cols, size_t row_stride, const QkvRopeParams& rope);
int check_qkv_rope_args(mlc_ctx* ctx, const void* qkv, const void* cos_t, const void* sin_t, size_t batch,
                        size_t num_heads, size_t kv_heads, size_t head_dim, size_t qkv_rows, size_t q_rows,
                        size_t k_rows, size_t v_rows, size_t rotary_dim);

}  // namespace mlcb
