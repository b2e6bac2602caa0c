/* CPU restatement of the other ops of the reference's batched walker step - the ones around attention.
 *
 * TEST INFRASTRUCTURE ONLY. Compiled into oracle/libpaged_oracle.so beside paged_oracle.c; only tests/,
 * __graft_entry__.smoke() and the CPU-baseline leg of bench.py may load it. Every function cites the lines
 * of MLcompiler it follows, and is pinned bit for bit (tests/test_layer_oracle.py) on golden vectors made
 * by running the reference's own CPU code for the same op (tests/golden/make_layer_golden.py).
 *
 * One decode pass of the reference's walker (compiler/runtime/batched_walker.cpp:248-297, 333-458) is, per
 * layer: RMSNorm -> Q4_0 mat-vec (fused QKV) -> split / RoPE / cast -> KV scatter -> paged attention ->
 * Q4_0 mat-vec (output projection) -> add -> RMSNorm -> Q4_0 mat-vec (gate | up) -> SiLU(gate) * up ->
 * Q4_0 mat-vec (down) -> add; then a final RMSNorm and the Q6_K (or Q4_0) lm_head.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

float orc_fp16_to_float(uint16_t h);   /* paged_oracle.c (compiler/runtime/float_convert.hpp:14-76) */

/* rmsNorm, compiler/runtime/operator_backend.cpp:186-204: mean of squares accumulated in fp32 in index
 * order, inv = 1 / sqrt(mean + eps), out = in * inv * gamma. The batched Metal kernel
 * (metal_runtime.mm:166-209) computes the same per row (rsqrt, a tree sum). input/out [batch, length]. */
void orc_rms_norm_batched(const float* in, const float* weight, float eps, uint32_t batch, uint32_t length,
                          float* out) {
    for (uint32_t r = 0; r < batch; ++r) {
        const float* x = in + (size_t)r * length;
        float* y = out + (size_t)r * length;
        float mean_sq = 0.0f;
        for (uint32_t i = 0; i < length; ++i) mean_sq += x[i] * x[i];
        mean_sq = mean_sq / (float)(length > 0 ? length : 1);
        float inv = 1.0f / sqrtf(mean_sq + eps);
        for (uint32_t i = 0; i < length; ++i) y[i] = x[i] * inv * weight[i];
    }
}

/* add_vectors, metal_runtime.mm:44-52; CPU Add node operator_backend.cpp:1144-1200. */
void orc_add(const float* a, const float* b, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

/* feedforward_silu_mul, metal_runtime.mm:32-42; silu() operator_backend.cpp:45-47, used at :847-850. */
void orc_silu_mul(const float* gate, const float* up, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float g = gate[i];
        out[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

/* encodeGateUpSplitSiluMul, metal_runtime.mm:8030-8088: gate_up [batch, rows] holds gate in columns
 * [0, ffn_inner) and up in [ffn_inner, 2 * ffn_inner) of every row (two strided copies), then SiLU(gate) * up.
 * gate / up may be NULL when the caller does not want the copies. */
void orc_gate_up_split_silu_mul(const float* gate_up, uint32_t batch, uint32_t ffn_inner, uint32_t rows,
                                float* gate, float* up, float* out) {
    for (uint32_t r = 0; r < batch; ++r) {
        const float* g = gate_up + (size_t)r * rows;
        const float* u = g + ffn_inner;
        if (gate) memcpy(gate + (size_t)r * ffn_inner, g, (size_t)ffn_inner * sizeof(float));
        if (up) memcpy(up + (size_t)r * ffn_inner, u, (size_t)ffn_inner * sizeof(float));
        orc_silu_mul(g, u, out + (size_t)r * ffn_inner, ffn_inner);
    }
}

/* ---- Q4_0: blocks of 32 weights = fp16 scale d + 16 bytes; weight j < 16 is the low nibble of byte j,
 * weight j + 16 the high nibble, value = d * (nibble - 8). compiler/runtime/quantization.cpp:71-74, 190-215. */
#define ORC_QK4_0 32
#define ORC_BLOCK_Q4_0 18

size_t orc_row_size_q4_0(size_t cols) { return (cols + ORC_QK4_0 - 1) / ORC_QK4_0 * ORC_BLOCK_Q4_0; }

void orc_dequant_row_q4_0(const uint8_t* src, size_t cols, float* dst) {
    size_t nb = (cols + ORC_QK4_0 - 1) / ORC_QK4_0;
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * ORC_BLOCK_Q4_0;
        uint16_t dbits;
        memcpy(&dbits, blk, 2);
        float d = orc_fp16_to_float(dbits);
        size_t base = b * ORC_QK4_0;
        for (size_t j = 0; j < ORC_QK4_0 / 2; ++j) {
            uint8_t byte = blk[2 + j];
            int lo = (int)(byte & 0x0F) - 8, hi = (int)((byte >> 4) & 0x0F) - 8;
            if (base + j < cols) dst[base + j] = d * (float)lo;
            if (base + j + ORC_QK4_0 / 2 < cols) dst[base + j + ORC_QK4_0 / 2] = d * (float)hi;
        }
    }
}

/* dotProductRowQ4_0, quantization.cpp:240-268: acc += d * q * x, low nibble then high nibble of every byte. */
float orc_dot_row_q4_0(const uint8_t* src, size_t cols, const float* vec) {
    size_t nb = (cols + ORC_QK4_0 - 1) / ORC_QK4_0;
    float acc = 0.0f;
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * ORC_BLOCK_Q4_0;
        uint16_t dbits;
        memcpy(&dbits, blk, 2);
        float d = orc_fp16_to_float(dbits);
        size_t base = b * ORC_QK4_0;
        for (size_t j = 0; j < ORC_QK4_0 / 2; ++j) {
            uint8_t byte = blk[2 + j];
            int lo = (int)(byte & 0x0F) - 8, hi = (int)((byte >> 4) & 0x0F) - 8;
            if (base + j < cols) acc += d * (float)lo * vec[base + j];
            if (base + j + ORC_QK4_0 / 2 < cols) acc += d * (float)hi * vec[base + j + ORC_QK4_0 / 2];
        }
    }
    return acc;
}

/* q4_0_matmul_v3_batched, metal_runtime.mm:710-785: out[n, r] = sum_c W[r, c] * in[n, c]; weights
 * [rows] rows of row_stride bytes, in [batch, cols], out [batch, rows]. The sum order here is the CPU
 * row function's (the Metal kernel sums 32 strided partials, then across lanes). */
void orc_matmul_q4_0_batched(const uint8_t* weights, const float* in, uint32_t batch, uint32_t rows, uint32_t cols,
                             size_t row_stride, float* out) {
    for (uint32_t n = 0; n < batch; ++n)
        for (uint32_t r = 0; r < rows; ++r)
            out[(size_t)n * rows + r] = orc_dot_row_q4_0(weights + (size_t)r * row_stride, cols, in + (size_t)n * cols);
}

/* ---- Q6_K: super-blocks of 256 weights = ql[128] | qh[64] | int8 scales[16] | fp16 d (210 bytes);
 * compiler/runtime/quantization.cpp:142-147, 1469-1499. */
#define ORC_QK_K 256
#define ORC_BLOCK_Q6_K 210

size_t orc_row_size_q6_k(size_t cols) { return (cols + ORC_QK_K - 1) / ORC_QK_K * ORC_BLOCK_Q6_K; }

void orc_dequant_row_q6_k(const uint8_t* src, size_t cols, float* dst) {
    size_t nb = (cols + ORC_QK_K - 1) / ORC_QK_K;
    for (size_t b = 0; b < nb; ++b) {
        const uint8_t* blk = src + b * ORC_BLOCK_Q6_K;
        const uint8_t* ql = blk;
        const uint8_t* qh = blk + ORC_QK_K / 2;
        const int8_t* sc = (const int8_t*)(blk + ORC_QK_K / 2 + ORC_QK_K / 4);
        uint16_t dbits;
        memcpy(&dbits, blk + ORC_QK_K / 2 + ORC_QK_K / 4 + ORC_QK_K / 16, 2);
        float d = orc_fp16_to_float(dbits);
        float buf[ORC_QK_K];
        float* y = buf;
        for (int n = 0; n < ORC_QK_K; n += 128) {
            for (int l = 0; l < 32; ++l) {
                int is = l / 16;
                int8_t q1 = (int8_t)((ql[l + 0] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int8_t q3 = (int8_t)((ql[l + 0] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                y[l + 0] = d * (float)sc[is + 0] * (float)q1;
                y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                y[l + 96] = d * (float)sc[is + 6] * (float)q4;
            }
            y += 128;
            ql += 64;
            qh += 32;
            sc += 8;
        }
        size_t elems = cols - b * ORC_QK_K < ORC_QK_K ? cols - b * ORC_QK_K : ORC_QK_K;
        memcpy(dst + b * ORC_QK_K, buf, elems * sizeof(float));
    }
}

/* dotProductRowQ6_K, quantization.cpp:1566-1586: dequantise a super-block, then acc += w * x in index order. */
float orc_dot_row_q6_k(const uint8_t* src, size_t cols, const float* vec) {
    size_t nb = (cols + ORC_QK_K - 1) / ORC_QK_K;
    float acc = 0.0f;
    float tmp[ORC_QK_K];
    size_t offset = 0;
    for (size_t b = 0; b < nb && offset < cols; ++b) {
        size_t elems = cols - offset < ORC_QK_K ? cols - offset : ORC_QK_K;
        orc_dequant_row_q6_k(src + b * ORC_BLOCK_Q6_K, elems, tmp);
        for (size_t i = 0; i < elems; ++i) acc += tmp[i] * vec[offset + i];
        offset += elems;
    }
    return acc;
}

/* q6_k_matmul_v3_batched, metal_runtime.mm:1581-1655: out[n, r] = sum_c W[r, c] * in[n, c]. */
void orc_matmul_q6_k_batched(const uint8_t* weights, const float* in, uint32_t batch, uint32_t rows, uint32_t cols,
                             size_t row_stride, float* out) {
    for (uint32_t n = 0; n < batch; ++n)
        for (uint32_t r = 0; r < rows; ++r)
            out[(size_t)n * rows + r] = orc_dot_row_q6_k(weights + (size_t)r * row_stride, cols, in + (size_t)n * cols);
}
