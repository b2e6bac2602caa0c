// The ops of the batched walker step around attention: batched RMSNorm, residual add, SiLU(gate) * up
// and the quantised (Q4_0 / Q6_K) batched mat-vec.
//
// Reference call sites: compiler/runtime/batched_walker.cpp:248-297 and 333-458 (one decode pass);
// the Metal kernels they dispatch are rms_norm_batched (metal_runtime.mm:166-209), add_vectors
// (mm:44-52), feedforward_silu_mul (mm:32-42), q4_0_matmul_v3_batched (mm:710-785) and
// q6_k_matmul_v3_batched (mm:1581-1655); the block formats are quantization.cpp:71-74 / 142-147.
//
// The mat-vec is a [rows x cols] x [cols x batch] product with batch <= 64: weight rows are the M side of
// mma.sync.m16n8k16, the batch the N side. A block's integers go into the A fragment as exact fp16
// values (nibble - 8, or 6-bit value - 32), the activations into B rounded to fp16, products accumulate
// in fp32 inside the MMA and each 16- or 32-weight group's sum is multiplied by its fp32 scale
// afterwards - so the only rounding beyond the CPU's is that of the activations to fp16.
// A CTA owns 128 weight rows and one slice of the columns; slices of a row tile leave their partial
// sums in a scratch buffer and the last CTA to finish a row tile adds them in slice order (a counter per
// row tile; the order is fixed, so results repeat bit for bit), with the residual add fused there when
// the caller asks for it. Weight bytes are read once from HBM; the activations (L2-resident) are read
// once per row tile.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdint>

#include "ctx.hpp"

namespace mlcb {

// ---------------------------------------------------------------------------------------------------
// RMSNorm, add, SiLU * up
// ---------------------------------------------------------------------------------------------------

// One CTA per row. Sum of squares in fp32 (per-thread strided partials, then a tree), mean = sum / length,
// inv = 1 / sqrt(mean + eps), out = in * inv * weight - the factors in the order of
// operator_backend.cpp:186-204, so that only the order of the sum differs from the CPU code.
__global__ void __launch_bounds__(256) rms_norm_batched_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                                               float eps, uint32_t length, float* __restrict__ out,
                                                               __half* __restrict__ out16) {
    __shared__ float part[8];
    const float* x = in + static_cast<size_t>(blockIdx.x) * length;
    float* y = out + static_cast<size_t>(blockIdx.x) * length;
    float s = 0.0f;
    const bool vec = (length & 3) == 0;
    if (vec) {
        for (uint32_t i = threadIdx.x * 4; i < length; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(x + i);
            s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s); s = fmaf(v.z, v.z, s); s = fmaf(v.w, v.w, s);
        }
    } else {
        for (uint32_t i = threadIdx.x; i < length; i += blockDim.x) s = fmaf(x[i], x[i], s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[i];
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, static_cast<float>(length)), eps)));
    __half* y16 = out16 ? out16 + static_cast<size_t>(blockIdx.x) * length : nullptr;
    if (vec) {
        for (uint32_t i = threadIdx.x * 4; i < length; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(x + i);
            const float4 g = *reinterpret_cast<const float4*>(w + i);
            float4 r;
            r.x = __fmul_rn(__fmul_rn(v.x, inv), g.x);
            r.y = __fmul_rn(__fmul_rn(v.y, inv), g.y);
            r.z = __fmul_rn(__fmul_rn(v.z, inv), g.z);
            r.w = __fmul_rn(__fmul_rn(v.w, inv), g.w);
            *reinterpret_cast<float4*>(y + i) = r;
            if (y16) {
                *reinterpret_cast<__half2*>(y16 + i) = __floats2half2_rn(r.x, r.y);
                *reinterpret_cast<__half2*>(y16 + i + 2) = __floats2half2_rn(r.z, r.w);
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < length; i += blockDim.x) {
            const float r = __fmul_rn(__fmul_rn(x[i], inv), w[i]);
            y[i] = r;
            if (y16) y16[i] = __float2half_rn(r);
        }
    }
}

__global__ void __launch_bounds__(256) add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                  float* __restrict__ out, size_t n4, size_t n) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n4) {
        const float4 x = reinterpret_cast<const float4*>(a)[i], y = reinterpret_cast<const float4*>(b)[i];
        reinterpret_cast<float4*>(out)[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
    if (i < n - n4 * 4) out[n4 * 4 + i] = a[n4 * 4 + i] + b[n4 * 4 + i];   // tail of a count not divisible by 4
}

// silu(g) * u with the CPU code's operations: g / (1 + exp(-g)), then the product
// (operator_backend.cpp:45-47, 847-850). expf here is CUDA's (<= 2 ulp), not libm's.
__device__ __forceinline__ float silu_mul(float g, float u) {
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

// gate_up [batch, rows]: gate = columns [0, inner), up = [inner, 2 * inner). gate / up copies optional.
__global__ void __launch_bounds__(256) gate_up_silu_mul_kernel(const float* __restrict__ gate_up, float* __restrict__ gate,
                                                               float* __restrict__ up, float* __restrict__ out,
                                                               uint32_t batch, uint32_t inner, uint32_t rows) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<size_t>(batch) * inner) return;
    const uint32_t r = static_cast<uint32_t>(i / inner), c = static_cast<uint32_t>(i - static_cast<size_t>(r) * inner);
    const float g = gate_up[static_cast<size_t>(r) * rows + c];
    const float u = gate_up[static_cast<size_t>(r) * rows + inner + c];
    if (gate) gate[i] = g;
    if (up) up[i] = u;
    out[i] = silu_mul(g, u);
}

__global__ void __launch_bounds__(256) silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                                       float* __restrict__ out, size_t n) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = silu_mul(gate[i], up[i]);
}

__device__ __forceinline__ float half_bits_to_float(uint32_t bits) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits)));
}

// Rows of a Q4_0 table picked by token id and dequantised, one CTA per request: what the walker's host
// loop does with dequantizeRowTo before it uploads the residual (batched_walker.cpp:183-208).
// d * (nibble - 8) is a single fp32 product, so the rows equal the CPU's bit for bit. A token id past the
// table gives a row of zeros and a device error bit.
__global__ void __launch_bounds__(256) embedding_q4_0_kernel(const uint8_t* __restrict__ table, size_t row_stride,
                                                             const uint32_t* __restrict__ tokens, uint32_t vocab,
                                                             uint32_t cols, float* __restrict__ out, uint32_t* err) {
    const uint32_t tok = tokens[blockIdx.x];
    float* y = out + static_cast<size_t>(blockIdx.x) * cols;
    if (tok >= vocab) {
        for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) y[i] = 0.0f;
        if (threadIdx.x == 0) atomicOr(err, MLC_DEVERR_BAD_TOKEN);
        return;
    }
    const uint8_t* row = table + static_cast<size_t>(tok) * row_stride;
    for (uint32_t i = threadIdx.x; i < cols / 2; i += blockDim.x) {   // one byte = weights j and j + 16 of a block
        const uint32_t b = i >> 4, j = i & 15;
        const uint8_t* blk = row + static_cast<size_t>(b) * 18;
        const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(blk));
        const uint32_t byte = blk[2 + j];
        y[b * 32 + j] = __fmul_rn(d, static_cast<float>(static_cast<int>(byte & 15u) - 8));
        y[b * 32 + j + 16] = __fmul_rn(d, static_cast<float>(static_cast<int>(byte >> 4) - 8));
    }
}

// ---------------------------------------------------------------------------------------------------
// Quantised batched mat-vec
// ---------------------------------------------------------------------------------------------------

constexpr int kMvRows = 128;        // weight rows per CTA (4 warps x 2 m-tiles of 16)
constexpr int kMvThreads = 128;
constexpr int kMvSliceMax = 512;    // columns per CTA slice at most (a multiple of both block sizes)
constexpr int kXPad = 8;            // halves of padding per activation row in shared memory

enum : int { kQ4_0 = 0, kQ6_K = 1 };
enum : int { kInPlain = 0, kInSiluMul = 1 };

template <int QT> struct QuantFormat;
template <> struct QuantFormat<kQ4_0> {
    static constexpr int kBlockBytes = 18, kBlockWeights = 32;
    static constexpr int kSliceBytesMax = kMvSliceMax / 32 * 18;          // 288
    static constexpr int kPitch = 304;                                     // 76 words: rows g land 12 banks apart
};
template <> struct QuantFormat<kQ6_K> {
    static constexpr int kBlockBytes = 210, kBlockWeights = 256;
    static constexpr int kSliceBytesMax = kMvSliceMax / 256 * 210;        // 420
    static constexpr int kPitch = 464;                                     // 116 words: rows g land 20 banks apart
};

struct MatVecParams {
    const uint8_t* w;        // [rows] rows of row_stride bytes
    const float* x;          // [batch, x_stride] fp32; with kInSiluMul gate at column c, up at column c + cols
    const float* residual;   // [batch, rows] added in the epilogue, or null
    float* out;              // [batch, rows]
    float* partial;          // [slices, batch, rows] when slices > 1
    uint32_t* counters;      // [row tiles], zero between launches
    size_t row_stride;
    uint32_t batch, rows, cols, x_stride;
    uint32_t slice_cols;     // columns per slice (a multiple of the block size)
    uint32_t slices;
};

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Two integers 0..63 in the low bytes of the two halves of `v` -> half2 of (value - bias), exact:
// 0x6400 | n is the fp16 number 1024 + n.
__device__ __forceinline__ uint32_t ints_to_half2(uint32_t v, uint32_t bias_bits) {
    const uint32_t h = v | 0x64006400u;
    __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), *reinterpret_cast<const __half2*>(&bias_bits));
    return *reinterpret_cast<uint32_t*>(&r);
}

// A fragments of one Q4_0 block (two 16-weight groups: low nibbles, high nibbles) for rows g and g + 8 of
// an m-tile. `row` points at the block in shared memory (2-byte aligned), t = lane & 3.
__device__ __forceinline__ void q4_0_fragments(const uint8_t* blk_g, const uint8_t* blk_g8, int t, uint32_t (&lo)[4],
                                               uint32_t (&hi)[4], float& d_g, float& d_g8) {
    const uint16_t* pg = reinterpret_cast<const uint16_t*>(blk_g);
    const uint16_t* p8 = reinterpret_cast<const uint16_t*>(blk_g8);
    d_g = half_bits_to_float(pg[0]);
    d_g8 = half_bits_to_float(p8[0]);
    // weights 2t, 2t+1 are bytes 2t, 2t+1 of the 16 (u16 index 1 + t); weights 2t+8, 2t+9 are u16 index 5 + t
    const uint32_t v[4] = {pg[1 + t], p8[1 + t], pg[5 + t], p8[5 + t]};
    constexpr uint32_t kBias = 0x64086408u;   // 1032 = 1024 + 8
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t l = (v[i] & 0x000Fu) | ((v[i] & 0x0F00u) << 8);
        const uint32_t h = ((v[i] >> 4) & 0x000Fu) | ((v[i] & 0xF000u) << 4);
        lo[i] = ints_to_half2(l, kBias);
        hi[i] = ints_to_half2(h, kBias);
    }
}

// A fragment of 16-weight group j (0..15) of a Q6_K super-block for rows g and g + 8, and the groups' scales
// d * sc[j]. Weight l of a 128-weight half lives in ql / qh as quantization.cpp:1469-1499 lays out.
__device__ __forceinline__ void q6_k_fragment(const uint8_t* blk_g, const uint8_t* blk_g8, int j, int t, uint32_t (&a)[4],
                                              float& s_g, float& s_g8) {
    const int h = j >> 3, quarter = (j & 7) >> 1, sub = j & 1;
    const int ql_off = 64 * h + ((quarter & 1) ? 32 : 0) + 16 * sub;   // q2 / q4 read ql[l + 32]
    const int qh_off = 128 + 32 * h + 16 * sub;
    const int nib_shift = (quarter >> 1) * 4;                           // q3 / q4 take the high nibble
    const int hi_shift = quarter * 2;
    constexpr uint32_t kBias = 0x64206420u;   // 1056 = 1024 + 32
    const uint8_t* rowp[2] = {blk_g, blk_g8};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int l = 2 * t + 8 * k;
            const uint32_t ql = *reinterpret_cast<const uint16_t*>(rowp[r] + ql_off + l);
            const uint32_t qh = *reinterpret_cast<const uint16_t*>(rowp[r] + qh_off + l);
            const uint32_t n0 = ((ql >> nib_shift) & 0xFu) | ((((qh) >> hi_shift) & 3u) << 4);
            const uint32_t n1 = ((ql >> (8 + nib_shift)) & 0xFu) | ((((qh >> 8) >> hi_shift) & 3u) << 4);
            a[r + 2 * k] = ints_to_half2(n0 | (n1 << 16), kBias);
        }
    }
    const float dg = half_bits_to_float(*reinterpret_cast<const uint16_t*>(blk_g + 208));
    const float d8 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(blk_g8 + 208));
    s_g = __fmul_rn(dg, static_cast<float>(static_cast<int8_t>(blk_g[192 + j])));
    s_g8 = __fmul_rn(d8, static_cast<float>(static_cast<int8_t>(blk_g8[192 + j])));
}

template <int QT, int NT, int IN>
__global__ void __launch_bounds__(kMvThreads) quant_matvec_kernel(const MatVecParams p) {
    using F = QuantFormat<QT>;
    constexpr int kXRows = NT * 8;
    extern __shared__ __align__(16) uint8_t smem[];
    __half* xs = reinterpret_cast<__half*>(smem);                                    // [kXRows][slice + pad]
    const uint32_t x_pitch = p.slice_cols + kXPad;
    uint8_t* ws = smem + static_cast<size_t>(kXRows) * x_pitch * sizeof(__half);     // [kMvRows][F::kPitch]
    __shared__ uint32_t ticket;

    const uint32_t tile = blockIdx.x, slice = blockIdx.y;
    const uint32_t row0 = tile * kMvRows;
    const uint32_t c0 = slice * p.slice_cols;
    const uint32_t ncols = min(p.slice_cols, p.cols - c0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

    // weight bytes of this slice: [b0, b1) of every row; copied as the enclosing 16-byte range
    const uint32_t b0 = c0 / F::kBlockWeights * F::kBlockBytes;
    const uint32_t b1 = b0 + ncols / F::kBlockWeights * F::kBlockBytes;
    const uint32_t a0 = b0 & ~15u;
    const uint32_t nvec = (b1 - a0 + 15) >> 4;
    const uint32_t w_shift = b0 - a0;
    for (uint32_t i = tid; i < kMvRows * nvec; i += kMvThreads) {
        const uint32_t r = i / nvec, v = i - r * nvec;
        const uint32_t row = min(row0 + r, p.rows - 1);
        const uint4 d = __ldg(reinterpret_cast<const uint4*>(p.w + static_cast<size_t>(row) * p.row_stride + a0) + v);
        *reinterpret_cast<uint4*>(ws + static_cast<size_t>(r) * F::kPitch + v * 16) = d;
    }
    // activations of this slice, rounded to fp16; rows past the batch are zero
    const uint32_t q4 = ncols >> 2;
    for (uint32_t i = tid; i < kXRows * q4; i += kMvThreads) {
        const uint32_t n = i / q4, c = (i - n * q4) << 2;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n < p.batch) {
            const float* src = p.x + static_cast<size_t>(n) * p.x_stride + c0 + c;
            v = *reinterpret_cast<const float4*>(src);
            if (IN == kInSiluMul) {
                const float4 u = *reinterpret_cast<const float4*>(src + p.cols);
                v = make_float4(silu_mul(v.x, u.x), silu_mul(v.y, u.y), silu_mul(v.z, u.z), silu_mul(v.w, u.w));
            }
        }
        __half2* dst = reinterpret_cast<__half2*>(xs + static_cast<size_t>(n) * x_pitch + c);
        dst[0] = __floats2half2_rn(v.x, v.y);
        dst[1] = __floats2half2_rn(v.z, v.w);
    }
    __syncthreads();

    float acc[2][NT][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[m][n][e] = 0.0f;

    const uint8_t* wrow[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        wrow[m][0] = ws + static_cast<size_t>(warp * 32 + m * 16 + g) * F::kPitch + w_shift;
        wrow[m][1] = wrow[m][0] + 8 * F::kPitch;
    }
    const __half* xrow = xs + static_cast<size_t>(g) * x_pitch + 2 * t;

    if (QT == kQ4_0) {
        const uint32_t nblk = ncols >> 5;
        for (uint32_t b = 0; b < nblk; ++b) {
            uint32_t bl[NT][2], bh[NT][2];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const __half* xp = xrow + static_cast<size_t>(n) * 8 * x_pitch + b * 32;
                bl[n][0] = *reinterpret_cast<const uint32_t*>(xp);
                bl[n][1] = *reinterpret_cast<const uint32_t*>(xp + 8);
                bh[n][0] = *reinterpret_cast<const uint32_t*>(xp + 16);
                bh[n][1] = *reinterpret_cast<const uint32_t*>(xp + 24);
            }
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                uint32_t lo[4], hi[4];
                float dg, d8;
                q4_0_fragments(wrow[m][0] + b * 18, wrow[m][1] + b * 18, t, lo, hi, dg, d8);
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma16816(c, lo, bl[n][0], bl[n][1]);
                    mma16816(c, hi, bh[n][0], bh[n][1]);
                    acc[m][n][0] = fmaf(dg, c[0], acc[m][n][0]);
                    acc[m][n][1] = fmaf(dg, c[1], acc[m][n][1]);
                    acc[m][n][2] = fmaf(d8, c[2], acc[m][n][2]);
                    acc[m][n][3] = fmaf(d8, c[3], acc[m][n][3]);
                }
            }
        }
    } else {
        const uint32_t ngroups = ncols >> 4;
        for (uint32_t j = 0; j < ngroups; ++j) {
            uint32_t bx[NT][2];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const __half* xp = xrow + static_cast<size_t>(n) * 8 * x_pitch + j * 16;
                bx[n][0] = *reinterpret_cast<const uint32_t*>(xp);
                bx[n][1] = *reinterpret_cast<const uint32_t*>(xp + 8);
            }
            const uint32_t blk = (j >> 4) * 210;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                uint32_t a[4];
                float sg, s8;
                q6_k_fragment(wrow[m][0] + blk, wrow[m][1] + blk, static_cast<int>(j & 15), t, a, sg, s8);
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma16816(c, a, bx[n][0], bx[n][1]);
                    acc[m][n][0] = fmaf(sg, c[0], acc[m][n][0]);
                    acc[m][n][1] = fmaf(sg, c[1], acc[m][n][1]);
                    acc[m][n][2] = fmaf(s8, c[2], acc[m][n][2]);
                    acc[m][n][3] = fmaf(s8, c[3], acc[m][n][3]);
                }
            }
        }
    }

    // C fragment: c0, c1 = (row g, batch 2t, 2t + 1); c2, c3 = (row g + 8, same)
    const bool direct = p.slices == 1;
    float* dst = direct ? p.out : p.partial + static_cast<size_t>(slice) * p.batch * p.rows;
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t row = row0 + warp * 32 + m * 16 + g + ((e & 2) ? 8 : 0);
                const uint32_t bn = n * 8 + 2 * t + (e & 1);
                if (row < p.rows && bn < p.batch) {
                    const size_t o = static_cast<size_t>(bn) * p.rows + row;
                    float v = acc[m][n][e];
                    if (direct && p.residual) v = __fadd_rn(p.residual[o], v);
                    dst[o] = v;
                }
            }
    if (direct) return;

    // the last slice of this row tile to arrive adds the partial sums in slice order
    __threadfence();
    __syncthreads();
    if (tid == 0) ticket = atomicAdd(p.counters + tile, 1u);
    __syncthreads();
    if (ticket != p.slices - 1) return;
    __threadfence();
    const uint32_t tile_rows = min(static_cast<uint32_t>(kMvRows), p.rows - row0);
    for (uint32_t i = tid; i < p.batch * tile_rows; i += kMvThreads) {
        const uint32_t bn = i / tile_rows, r = i - bn * tile_rows;
        const size_t o = static_cast<size_t>(bn) * p.rows + row0 + r;
        float s = __ldcg(p.partial + o);
        for (uint32_t k = 1; k < p.slices; ++k) s = __fadd_rn(s, __ldcg(p.partial + static_cast<size_t>(k) * p.batch * p.rows + o));
        if (p.residual) s = __fadd_rn(p.residual[o], s);
        p.out[o] = s;
    }
    if (tid == 0) p.counters[tile] = 0;   // ready for the next launch on this stream
}

template <int QT, int NT, int IN>
static int launch_matvec_nt(mlc_ctx* ctx, const MatVecParams& p, dim3 grid, size_t smem) {
    auto kernel = quant_matvec_kernel<QT, NT, IN>;
    static bool attr_set[16] = {};
    if (ctx->device >= 0 && ctx->device < 16 && !attr_set[ctx->device]) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
        attr_set[ctx->device] = true;
    }
    kernel<<<grid, kMvThreads, smem, ctx->stream>>>(p);
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

template <int QT, int IN>
static int launch_matvec(mlc_ctx* ctx, MatVecParams p) {
    using F = QuantFormat<QT>;
    const uint32_t tiles = (p.rows + kMvRows - 1) / kMvRows;
    // enough CTAs for two per SM where the columns allow it; a slice is a whole number of blocks
    const uint32_t unit = QT == kQ6_K ? 256u : 128u;
    const uint32_t max_slices = (p.cols + unit - 1) / unit;
    uint32_t want = std::max(1u, (2u * static_cast<uint32_t>(ctx->sm_count) + tiles - 1) / tiles);
    want = std::min(want, max_slices);
    uint32_t slice_cols = ((p.cols + want - 1) / want + unit - 1) / unit * unit;
    slice_cols = std::min<uint32_t>(slice_cols, kMvSliceMax);
    p.slice_cols = slice_cols;
    p.slices = (p.cols + slice_cols - 1) / slice_cols;
    const uint32_t nt = (p.batch + 7) / 8;
    const int NT = nt <= 1 ? 1 : (nt <= 2 ? 2 : (nt <= 4 ? 4 : 8));
    if (p.slices > 1) {
        const size_t part_bytes = static_cast<size_t>(p.slices) * p.batch * p.rows * sizeof(float);
        p.partial = static_cast<float*>(mlc_cached_buffer(ctx, "mlc_matvec_partials", part_bytes));
        // counters: one block for any row-tile count this context sees; zeroed when (re)allocated
        const size_t cnt_bytes = std::max<size_t>(4096, static_cast<size_t>(tiles) * 4);
        auto it = ctx->cached.find("mlc_matvec_counters");
        const bool fresh = it == ctx->cached.end() || it->second.second < cnt_bytes;
        p.counters = static_cast<uint32_t*>(mlc_cached_buffer(ctx, "mlc_matvec_counters", cnt_bytes));
        if (!p.partial || !p.counters) return ctx->fail(MLC_ERR_CUDA, "scratch allocation for the mat-vec failed");
        if (fresh) MLCB_CUDA(ctx, cudaMemsetAsync(p.counters, 0, cnt_bytes, ctx->stream));
    }
    const size_t smem = static_cast<size_t>(NT) * 8 * (slice_cols + kXPad) * sizeof(__half) +
                        static_cast<size_t>(kMvRows) * F::kPitch;
    const dim3 grid(tiles, p.slices);
    switch (NT) {
        case 1: return launch_matvec_nt<QT, 1, IN>(ctx, p, grid, smem);
        case 2: return launch_matvec_nt<QT, 2, IN>(ctx, p, grid, smem);
        case 4: return launch_matvec_nt<QT, 4, IN>(ctx, p, grid, smem);
        default: return launch_matvec_nt<QT, 8, IN>(ctx, p, grid, smem);
    }
}

static int check_matvec(mlc_ctx* ctx, int qt, const void* w, const void* in, const void* out, size_t batch, size_t rows,
                        size_t cols, size_t row_stride, size_t x_stride) {
    if (!w || !in || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (batch == 0 || rows == 0 || cols == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    const size_t bw = qt == kQ6_K ? 256 : 32, bb = qt == kQ6_K ? 210 : 18;
    if (cols % bw) return ctx->fail(MLC_ERR_UNSUPPORTED, "cols must be a whole number of quantisation blocks");
    if (row_stride < cols / bw * bb) return ctx->fail(MLC_ERR_INVALID_ARG, "row_stride shorter than a row");
    if (row_stride % 16 || reinterpret_cast<uintptr_t>(w) % 16)
        return ctx->fail(MLC_ERR_UNSUPPORTED, "weights and row_stride must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(in) % 16 || x_stride % 4) return ctx->fail(MLC_ERR_INVALID_ARG, "input must be 16-byte aligned");
    if (batch > 64) return ctx->fail(MLC_ERR_UNSUPPORTED, "batch above 64");
    if (rows >= (1u << 31) || cols >= (1u << 31)) return ctx->fail(MLC_ERR_UNSUPPORTED, "dimension too large");
    return MLC_OK;
}

}  // namespace mlcb

using namespace mlcb;

extern "C" {

int mlc_encode_rms_norm_batched(mlc_ctx* ctx, const void* in, const void* weight, float epsilon, size_t batch,
                                size_t length, void* out, void* out_f16) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!in || !weight || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (batch == 0 || length == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (batch >= (1u << 31) || length >= (1u << 31)) return ctx->fail(MLC_ERR_UNSUPPORTED, "dimension too large");
    if ((length % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                               reinterpret_cast<uintptr_t>(weight)) % 16))
        return ctx->fail(MLC_ERR_INVALID_ARG, "buffers must be 16-byte aligned");
    DeviceGuard guard(ctx->device);
    rms_norm_batched_kernel<<<static_cast<unsigned>(batch), 256, 0, ctx->stream>>>(
        static_cast<const float*>(in), static_cast<const float*>(weight), epsilon, static_cast<uint32_t>(length),
        static_cast<float*>(out), static_cast<__half*>(out_f16));
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

int mlc_encode_add_batched(mlc_ctx* ctx, const void* a, const void* b, void* out, size_t total_elements) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!a || !b || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (total_elements == 0) return MLC_OK;
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) % 16)
        return ctx->fail(MLC_ERR_INVALID_ARG, "buffers must be 16-byte aligned");
    DeviceGuard guard(ctx->device);
    const size_t n4 = total_elements / 4;
    const size_t threads = std::max<size_t>(n4, total_elements - n4 * 4);
    add_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(out), n4, total_elements);
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

int mlc_encode_silu_mul_batched(mlc_ctx* ctx, const void* gate, const void* up, void* out, size_t total_elements) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!gate || !up || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (total_elements == 0) return MLC_OK;
    DeviceGuard guard(ctx->device);
    silu_mul_kernel<<<static_cast<unsigned>((total_elements + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<const float*>(gate), static_cast<const float*>(up), static_cast<float*>(out), total_elements);
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

int mlc_encode_gate_up_split_silu_mul(mlc_ctx* ctx, const void* gate_up, void* gate, void* up, void* out, size_t batch,
                                      size_t ffn_inner, size_t ffn_gate_up_rows) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");   // mm:8035
    if (!gate_up || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (batch == 0 || ffn_inner == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (ffn_gate_up_rows < 2 * ffn_inner) return ctx->fail(MLC_ERR_INVALID_ARG, "row shorter than gate + up");
    if (batch * ffn_gate_up_rows >= (size_t(1) << 32)) return ctx->fail(MLC_ERR_UNSUPPORTED, "batch too large");
    DeviceGuard guard(ctx->device);
    const size_t n = batch * ffn_inner;
    gate_up_silu_mul_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<const float*>(gate_up), static_cast<float*>(gate), static_cast<float*>(up), static_cast<float*>(out),
        static_cast<uint32_t>(batch), static_cast<uint32_t>(ffn_inner), static_cast<uint32_t>(ffn_gate_up_rows));
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

int mlc_encode_embedding_q4_0(mlc_ctx* ctx, const void* table, size_t row_stride, const void* token_ids, size_t batch,
                              size_t cols, size_t vocab, void* out) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!table || !token_ids || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (batch == 0 || cols == 0 || vocab == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (cols % 32) return ctx->fail(MLC_ERR_UNSUPPORTED, "cols must be a whole number of quantisation blocks");
    if (row_stride < cols / 32 * 18 || row_stride % 2 || reinterpret_cast<uintptr_t>(table) % 2)
        return ctx->fail(MLC_ERR_INVALID_ARG, "row_stride shorter than a row, or odd");
    if (batch >= (1u << 31) || cols >= (1u << 31) || vocab >= (size_t(1) << 32)) return ctx->fail(MLC_ERR_UNSUPPORTED, "dimension too large");
    DeviceGuard guard(ctx->device);
    embedding_q4_0_kernel<<<static_cast<unsigned>(batch), 256, 0, ctx->stream>>>(
        static_cast<const uint8_t*>(table), row_stride, static_cast<const uint32_t*>(token_ids), static_cast<uint32_t>(vocab),
        static_cast<uint32_t>(cols), static_cast<float*>(out), ctx->d_err);
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

static int encode_matvec(mlc_ctx* ctx, int qt, int in_mode, const void* weights, const void* in, const void* residual,
                         size_t batch, size_t rows, size_t cols, size_t row_stride, size_t x_stride, void* out) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    int st = check_matvec(ctx, qt, weights, in, out, batch, rows, cols, row_stride, x_stride);
    if (st != MLC_OK) return st;
    if (in_mode == kInSiluMul && x_stride < 2 * cols) return ctx->fail(MLC_ERR_INVALID_ARG, "row shorter than gate + up");
    DeviceGuard guard(ctx->device);
    MatVecParams p{};
    p.w = static_cast<const uint8_t*>(weights);
    p.x = static_cast<const float*>(in);
    p.residual = static_cast<const float*>(residual);
    p.out = static_cast<float*>(out);
    p.row_stride = row_stride;
    p.batch = static_cast<uint32_t>(batch);
    p.rows = static_cast<uint32_t>(rows);
    p.cols = static_cast<uint32_t>(cols);
    p.x_stride = static_cast<uint32_t>(x_stride);
    if (qt == kQ6_K) return in_mode == kInSiluMul ? launch_matvec<kQ6_K, kInSiluMul>(ctx, p) : launch_matvec<kQ6_K, kInPlain>(ctx, p);
    return in_mode == kInSiluMul ? launch_matvec<kQ4_0, kInSiluMul>(ctx, p) : launch_matvec<kQ4_0, kInPlain>(ctx, p);
}

int mlc_encode_matmul_q4_0_batched(mlc_ctx* ctx, const void* weights, const void* in, size_t batch, size_t rows,
                                   size_t cols, size_t row_stride, void* out) {
    return encode_matvec(ctx, kQ4_0, kInPlain, weights, in, nullptr, batch, rows, cols, row_stride, cols, out);
}

int mlc_encode_matmul_q6k_batched(mlc_ctx* ctx, const void* weights, const void* in, size_t batch, size_t rows,
                                  size_t cols, size_t row_stride, void* out) {
    return encode_matvec(ctx, kQ6_K, kInPlain, weights, in, nullptr, batch, rows, cols, row_stride, cols, out);
}

int mlc_encode_matmul_quant_fused(mlc_ctx* ctx, int quant, const void* weights, const void* in, size_t in_stride,
                                  int silu_mul_input, const void* residual, size_t batch, size_t rows, size_t cols,
                                  size_t row_stride, void* out) {
    if (quant != kQ4_0 && quant != kQ6_K) return ctx ? ctx->fail(MLC_ERR_INVALID_ARG, "unknown quantisation") : MLC_ERR_INVALID_ARG;
    return encode_matvec(ctx, quant, silu_mul_input ? kInSiluMul : kInPlain, weights, in, residual, batch, rows, cols,
                         row_stride, in_stride, out);
}

}  // extern "C"
