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
// values (nibble - 8, or 6-bit value - 32), each activation into B as two fp16 numbers (hi = fp16(x),
// lo = fp16(x - hi): 22 bits of x) against the same weight in two MMAs, products accumulate in fp32 inside
// the MMA and each 16- or 32-weight
// group's sum is multiplied by its fp32 scale afterwards - so results differ from the CPU's fp32 loop by
// the order of the sums, not by the precision of the operands.
// A CTA owns 64 weight rows and one slice of the columns (8 warps: 4 m-tiles x 2 halves of every chunk); the slices of a row tile are the CTAs of one
// thread-block cluster, which add their partial tiles through distributed shared memory in slice order
// (fixed, so results repeat bit for bit), with the residual add fused there when the caller asks for it.
// Weight bytes are read once from HBM; the activations (L2-resident) are read once per row tile.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <vector>

#include "ctx.hpp"
#include "qkv_rope.hpp"
#include "tcgen05_util.hpp"

namespace mlcb {

// Every kernel of this file is launched as a programmatic dependent of the kernel before it on the stream
// (MLC_B200_LAYER_PDL=0 in the environment turns that off): its CTAs may start while that kernel drains, and
// wait (griddepcontrol.wait) before they touch anything a kernel writes. What runs before the wait reads only
// weights, which no kernel writes.
static bool layer_pdl() {
    static const bool on = [] {
        const char* e = std::getenv("MLC_B200_LAYER_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

template <typename... KArgs, typename... Args>
static cudaError_t launch_layer_kernel(mlc_ctx* ctx, void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem,
                                       unsigned cluster, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (layer_pdl()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ void dependent_launch_gate() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------------
// RMSNorm, add, SiLU * up
// ---------------------------------------------------------------------------------------------------

// One CTA per row. Sum of squares in fp32 (per-thread strided partials, then a tree), mean = sum / length,
// inv = 1 / sqrt(mean + eps), out = in * inv * weight - the factors in the order of
// operator_backend.cpp:186-204, so that only the order of the sum differs from the CPU code.
__global__ void __launch_bounds__(256) rms_norm_batched_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                                               float eps, uint32_t length, float* __restrict__ out,
                                                               __half* __restrict__ out16, uint32_t* __restrict__ packed) {
    __shared__ float part[8];
    // Rows of up to 4096 columns stay in registers between the two passes, and their norm weights - which no
    // kernel writes - are fetched before the wait for the kernel in front.
    constexpr int kKeep = 4;
    const bool vec = (length & 3) == 0;
    const bool keep = vec && length <= 256u * 4u * kKeep && blockDim.x == 256;
    float4 gk[kKeep], vk[kKeep];
    if (keep) {
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            const uint32_t i = (threadIdx.x + j * 256u) * 4u;
            if (i < length) gk[j] = __ldg(reinterpret_cast<const float4*>(w + i));
        }
    }
    dependent_launch_gate();
    const float* x = in + static_cast<size_t>(blockIdx.x) * length;
    float* y = out ? out + static_cast<size_t>(blockIdx.x) * length : nullptr;
    float s = 0.0f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            const uint32_t i = (threadIdx.x + j * 256u) * 4u;
            if (i < length) vk[j] = *reinterpret_cast<const float4*>(x + i);
        }
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            const uint32_t i = (threadIdx.x + j * 256u) * 4u;
            if (i < length) {
                const float4 v = vk[j];
                s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s); s = fmaf(v.z, v.z, s); s = fmaf(v.w, v.w, s);
            }
        }
    } else if (vec) {
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
    auto emit = [&](uint32_t i, const float4& v, const float4& g) {
        float4 r;
        r.x = __fmul_rn(__fmul_rn(v.x, inv), g.x);
        r.y = __fmul_rn(__fmul_rn(v.y, inv), g.y);
        r.z = __fmul_rn(__fmul_rn(v.z, inv), g.z);
        r.w = __fmul_rn(__fmul_rn(v.w, inv), g.w);
        if (y) *reinterpret_cast<float4*>(y + i) = r;
        if (packed) {   // the mat-vec kernel's operand format: {hi0, hi1}, {lo0, lo1} per pair of columns
            const __half2 h01 = __floats2half2_rn(r.x, r.y), h23 = __floats2half2_rn(r.z, r.w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const __half2 l01 = __floats2half2_rn(r.x - f01.x, r.y - f01.y), l23 = __floats2half2_rn(r.z - f23.x, r.w - f23.y);
            *reinterpret_cast<uint4*>(packed + static_cast<size_t>(blockIdx.x) * length + i) =
                make_uint4(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&l01),
                           *reinterpret_cast<const uint32_t*>(&h23), *reinterpret_cast<const uint32_t*>(&l23));
        }
        if (y16) {
            *reinterpret_cast<__half2*>(y16 + i) = __floats2half2_rn(r.x, r.y);
            *reinterpret_cast<__half2*>(y16 + i + 2) = __floats2half2_rn(r.z, r.w);
        }
    };
    if (keep) {
#pragma unroll
        for (int j = 0; j < kKeep; ++j) {
            const uint32_t i = (threadIdx.x + j * 256u) * 4u;
            if (i < length) emit(i, vk[j], gk[j]);
        }
    } else if (vec) {
        for (uint32_t i = threadIdx.x * 4; i < length; i += blockDim.x * 4)
            emit(i, *reinterpret_cast<const float4*>(x + i), *reinterpret_cast<const float4*>(w + i));
    } else {
        for (uint32_t i = threadIdx.x; i < length; i += blockDim.x) {
            const float r = __fmul_rn(__fmul_rn(x[i], inv), w[i]);
            if (y) y[i] = r;
            if (y16) y16[i] = __float2half_rn(r);
        }
    }
}

__global__ void __launch_bounds__(256) add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                  float* __restrict__ out, size_t n4, size_t n) {
    dependent_launch_gate();
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
    dependent_launch_gate();
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
    dependent_launch_gate();
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = silu_mul(gate[i], up[i]);
}

// Index of the first maximum of every request's logits, one CTA per request. The logits lie as the walker's lm_head
// leaves them: groups of `group_rows` vocabulary rows, each group a [batch, rows of the group] array (group_rows >=
// vocab: one plain [batch, vocab] array). A thread looks at indices tid, tid + 256, ... in rising order and keeps the
// first maximum it sees; between threads the larger value wins and, among equals, the lower index - what a host
// loop `if (x[i] > x[best]) best = i` returns for finite values.
__global__ void __launch_bounds__(256) argmax_rows_kernel(const float* __restrict__ logits, uint32_t batch, uint32_t vocab,
                                                          uint32_t group_rows, uint32_t* __restrict__ out) {
    __shared__ float s_val[8];
    __shared__ uint32_t s_idx[8];
    dependent_launch_gate();
    const uint32_t n = blockIdx.x;
    float best = -INFINITY;
    uint32_t best_i = 0xFFFFFFFFu;
    for (uint32_t r0 = 0; r0 < vocab; r0 += group_rows) {
        const uint32_t nr = min(group_rows, vocab - r0);
        const float* row = logits + static_cast<size_t>(batch) * r0 + static_cast<size_t>(n) * nr;
        for (uint32_t c = threadIdx.x; c < nr; c += blockDim.x) {
            const float v = row[c];
            if (v > best || best_i == 0xFFFFFFFFu) { best = v; best_i = r0 + c; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t i = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (i != 0xFFFFFFFFu && (best_i == 0xFFFFFFFFu || v > best || (v == best && i < best_i))) { best = v; best_i = i; }
    }
    if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) {
            const float v = s_val[w];
            const uint32_t i = s_idx[w];
            if (i != 0xFFFFFFFFu && (best_i == 0xFFFFFFFFu || v > best || (v == best && i < best_i))) { best = v; best_i = i; }
        }
        out[n] = best_i;
    }
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
    dependent_launch_gate();
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

// Weight rows per CTA (the kernel's ROWS): 64 - 4 m-tiles of 16, each worked on by two warps (half the columns
// each) - or 128 - one m-tile per warp. Every row tile reads the activations again (through L2), so the tall
// tile pays where a matrix has more row tiles than the GPU holds at once, and costs CTAs where it has few.
constexpr int kMvThreads = 256;
constexpr int kMvChunk = 256;       // columns staged in shared memory at a time (a multiple of both block sizes)
constexpr int kXPadWords = 4;       // words of padding per activation row in shared memory: rows land 4 banks apart
constexpr int kMvStages = 2;        // chunks in flight per CTA

enum : int { kQ4_0 = 0, kQ6_K = 1 };
enum : int { kInPlain = 0, kInSiluMul = 1, kInPacked = 2 };   // kInPacked: the input already holds {hi, lo} words

template <int QT> struct QuantFormat;
template <> struct QuantFormat<kQ4_0> {
    static constexpr int kBlockBytes = 18, kBlockWeights = 32;
};
template <> struct QuantFormat<kQ6_K> {
    static constexpr int kBlockBytes = 210, kBlockWeights = 256;
};

struct MatVecParams {
    const uint8_t* w;        // [rows] rows of row_stride bytes
    const float* x;          // [batch, x_stride] fp32; with kInSiluMul gate at column c, up at column c + cols
    const float* residual;   // [batch, rows] added in the epilogue, or null
    float* out;              // [batch, rows]
    size_t row_stride;
    uint32_t batch, rows, cols, x_stride;
    uint32_t slice_cols;     // columns per slice (a multiple of the block size)
    uint32_t chunk_cols;     // columns staged in shared memory at a time
    uint32_t w_pitch;        // bytes between weight rows in shared memory
    uint32_t rope_mode;      // 1: the rows are a fused Q | K | V projection and the epilogue finishes them (see `rope`)
    QkvRopeParams rope;      // where Q (fp16) and the K / V page rows go, the rotary tables, the pass's (page, slot) per request
    uint32_t pair_inner;     // 0, or: rows = gate rows [0, pair_inner) then up rows [pair_inner, 2 pair_inner); a row tile is
                             // half gate rows, half the up rows that go with them, and out gets SiLU(gate) * up as operand words
    uint32_t slices;         // CTAs per cluster
    uint32_t aligned16;      // weights and row_stride on 16-byte boundaries: vector copies
};

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The first cluster barrier publishes every CTA's partial sums (release / acquire); the second only keeps a
// CTA's shared memory alive until its readers are done and orders nothing.
// The same with a zero accumulator coming in: d = a . b (no registers to clear beforehand).
__device__ __forceinline__ void mma16816_zero(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    const float z = 0.0f;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(z));
}

__device__ __forceinline__ void cluster_sync_publish() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}

// 16 bytes at `local_smem_addr` of CTA `rank` of this cluster.
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}


// Shared memory of one pipeline stage: the chunk's activations as fp32 words [kXRows][chunk + 4] (turned in
// place into {hi, lo} fp16 pairs), with SiLU input a second such array for the `up` half, then the chunk's
// weight bytes [ROWS][w_pitch].
template <int QT, int NT, int IN, int ROWS>
__global__ void __launch_bounds__(kMvThreads) quant_matvec_kernel(const MatVecParams p) {
    using F = QuantFormat<QT>;
    constexpr int kMvRows = ROWS;
    constexpr int MT = ROWS / 64;           // m-tiles per warp: they share the warp's activation fragments
    constexpr int kRedPitch = ROWS + 4;     // floats per batch row of a partial tile: lanes t land 8 banks apart
    constexpr int kXRows = NT * 8;
    constexpr int kXArrays = IN == kInSiluMul ? 2 : 1;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t x_pitch = p.chunk_cols + kXPadWords;                  // words
    const uint32_t x_bytes = kXRows * x_pitch * 4;
    const uint32_t stage_bytes = kXArrays * x_bytes + kMvRows * p.w_pitch;

    // The CTAs of a cluster share a row tile and split its columns: blockIdx.x = tile * slices + slice, and the
    // slice is the CTA's rank in the cluster.
    const uint32_t S = p.slices;
    const uint32_t tile = blockIdx.x / S, slice = blockIdx.x - tile * S;
    const uint32_t row0 = tile * kMvRows;
    constexpr uint32_t kPairHalf = kMvRows / 2;
    // weight row behind row r of the tile (rows past the matrix repeat its last row; their sums are never stored)
    auto weight_row = [&](uint32_t r) -> uint32_t {
        if (!p.pair_inner) return min(row0 + r, p.rows - 1);
        const uint32_t up = r >= kPairHalf ? 1u : 0u;
        return up * p.pair_inner + min(tile * kPairHalf + r - up * kPairHalf, p.pair_inner - 1);
    };
    const uint32_t c_begin = min(slice * p.slice_cols, p.cols), c_end = min(c_begin + p.slice_cols, p.cols);
    const uint32_t n_chunks = (c_end - c_begin + p.chunk_cols - 1) / p.chunk_cols;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int mt = warp & 3, kh = warp >> 2;   // the warp's group of MT m-tiles and its half of every chunk's columns

    // Every byte of a chunk arrives by cp.async, issued at once: one round trip to L2 / HBM per chunk, and the
    // next chunk's is under way while this one is computed.
    auto issue_weights = [&](uint32_t chunk) {
        if (chunk < n_chunks) {
            uint8_t* st = smem + (chunk % kMvStages) * stage_bytes;
            const uint32_t c0 = c_begin + chunk * p.chunk_cols;
            const uint32_t ncols = min(p.chunk_cols, c_end - c0);
            const uint32_t b0 = c0 / F::kBlockWeights * F::kBlockBytes;
            const uint32_t b1 = b0 + ncols / F::kBlockWeights * F::kBlockBytes;
            uint8_t* ws = st + kXArrays * x_bytes;
            if (p.aligned16) {
                // 16 lanes across a row's 16-byte vectors (a chunk's row is at most 15 of them), 16 rows per pass
                const uint32_t a0 = b0 & ~15u, nvec = (b1 - a0 + 15) >> 4;
                const uint32_t v = tid & 15;
                if (v < nvec) {
#pragma unroll
                    for (uint32_t r = tid >> 4; r < kMvRows; r += kMvThreads / 16) {
                        const uint32_t row = weight_row(r);
                        const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(ws + r * p.w_pitch + v * 16));
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                                     "l"(p.w + static_cast<size_t>(row) * p.row_stride + a0 + v * 16) : "memory");
                    }
                }
            } else {
                // rows that do not start on 16-byte boundaries (a Q6_K row of 256 columns is 210 bytes): 2-byte copies
                const uint32_t n16 = (b1 - b0) >> 1, w_shift = b0 & 15u;
                for (uint32_t i = tid; i < kMvRows * n16; i += kMvThreads) {
                    const uint32_t r = i / n16, v = i - r * n16;
                    const uint32_t row = weight_row(r);
                    const uint16_t d = __ldg(reinterpret_cast<const uint16_t*>(p.w + static_cast<size_t>(row) * p.row_stride + b0) + v);
                    *reinterpret_cast<uint16_t*>(ws + static_cast<size_t>(r) * p.w_pitch + w_shift + v * 2) = d;
                }
            }
        }
    };
    auto issue_activations = [&](uint32_t chunk) {
        if (chunk < n_chunks) {
            uint8_t* st = smem + (chunk % kMvStages) * stage_bytes;
            const uint32_t c0 = c_begin + chunk * p.chunk_cols;
            const uint32_t ncols = min(p.chunk_cols, c_end - c0);
            // 64 lanes across a row's float4 (a chunk is at most 256 columns), 4 batch rows per pass
            const uint32_t cq = tid & 63;
            if (cq < (ncols >> 2)) {
                const float* src = p.x + static_cast<size_t>(tid >> 6) * p.x_stride + c0 + cq * 4;
                uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(st + ((tid >> 6) * x_pitch + cq * 4) * 4));
                for (uint32_t n = tid >> 6; n < p.batch; n += kMvThreads / 64) {
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
                    if (IN == kInSiluMul)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + x_bytes), "l"(src + p.cols) : "memory");
                    src += static_cast<size_t>(kMvThreads / 64) * p.x_stride;
                    dst += (kMvThreads / 64) * x_pitch * 4;
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");   // one group per chunk index, empty or not
    };

    float acc[MT][NT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[m][n][e] = 0.0f;

    // Launched as a programmatic dependent of the kernel before it: the first chunk's weights (never written by
    // any kernel) are on their way while that kernel finishes; its output - this kernel's activations - is
    // touched only after the wait. Without the launch attribute both instructions do nothing.
    static_assert(kMvStages == 2, "the prologue below issues exactly one chunk");
    issue_weights(0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    issue_activations(0);

    for (uint32_t chunk = 0; chunk < n_chunks; ++chunk) {
        issue_weights(chunk + 1);            // into the stage the previous iteration finished with
        issue_activations(chunk + 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(kMvStages - 1) : "memory");
        __syncthreads();
        uint8_t* st = smem + (chunk % kMvStages) * stage_bytes;
        uint32_t* xw = reinterpret_cast<uint32_t*>(st);
        const uint8_t* ws = st + kXArrays * x_bytes;
        const uint32_t c0 = c_begin + chunk * p.chunk_cols;
        const uint32_t ncols = min(p.chunk_cols, c_end - c0);
        const uint32_t w_shift = (c0 / F::kBlockWeights * F::kBlockBytes) & 15u;

        // Activations in place, two columns at a time: fp32 (x0, x1) -> the words {hi0, hi1} and {lo0, lo1} with
        // hi = fp16(x), lo = fp16(x - hi): 22 bits of x, so the products lose nothing that fp32 keeps. Rows past
        // the batch become zero.
        if (IN == kInPacked) {
            // the words came in ready; only the rows past the batch need their zeros
            const uint32_t cq = tid & 63;
            if (cq < (ncols >> 2))
                for (uint32_t n = p.batch + (tid >> 6); n < kXRows; n += kMvThreads / 64)
                    *reinterpret_cast<uint4*>(xw + n * x_pitch + cq * 4) = make_uint4(0u, 0u, 0u, 0u);
        } else {
            const uint32_t cq = tid & 63;
            if (cq < (ncols >> 2)) {
#pragma unroll 2
                for (uint32_t n = tid >> 6; n < kXRows; n += kMvThreads / 64) {
                    uint4* wp = reinterpret_cast<uint4*>(xw + n * x_pitch + cq * 4);
                    uint4 o = make_uint4(0u, 0u, 0u, 0u);
                    if (n < p.batch) {
                        float4 w = *reinterpret_cast<const float4*>(wp);
                        if (IN == kInSiluMul) {
                            const float4 u = *reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(wp) + x_bytes);
                            w = make_float4(silu_mul(w.x, u.x), silu_mul(w.y, u.y), silu_mul(w.z, u.z), silu_mul(w.w, u.w));
                        }
                        const __half2 h01 = __floats2half2_rn(w.x, w.y), h23 = __floats2half2_rn(w.z, w.w);
                        const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
                        const __half2 l01 = __floats2half2_rn(w.x - f01.x, w.y - f01.y);
                        const __half2 l23 = __floats2half2_rn(w.z - f23.x, w.w - f23.y);
                        o = make_uint4(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&l01),
                                       *reinterpret_cast<const uint32_t*>(&h23), *reinterpret_cast<const uint32_t*>(&l23));
                    }
                    *wp = o;
                }
            }
        }
        __syncthreads();

        // Lane t of a quad owns a contiguous run of columns, so its B words are one or two 16-byte loads and its
        // weights a few adjacent bytes: k slots (2t, 2t + 1) and (2t + 8, 2t + 9) of an MMA are two column pairs of
        // that run, once against the {hi, hi} words and once against the {lo, lo} words, with the same A registers.
        const uint8_t* wg = ws + (mt * MT * 16 + g) * p.w_pitch + w_shift;
        const uint32_t* xrow = xw + g * x_pitch;

        if (QT == kQ4_0) {
            // columns [8t, 8t + 8) of a block: low (t < 2) or high nibbles of bytes [8 (t & 1), 8 (t & 1) + 8).
            // 0x6400 | n is the fp16 number 1024 + n, 0x6400 | (n << 4) is 1024 + 16 n: one fused multiply-add
            // takes either to n - 8 exactly.
            const bool high = t >= 2;
            const uint32_t nib_mask = high ? 0x00F000F0u : 0x000F000Fu;
            const __half2 mul = high ? __floats2half2_rn(0.0625f, 0.0625f) : __floats2half2_rn(1.0f, 1.0f);
            const __half2 add = high ? __floats2half2_rn(-72.0f, -72.0f) : __floats2half2_rn(-1032.0f, -1032.0f);
            const uint32_t byte_off = 2 + 8 * (t & 1);
            const uint32_t nblk = ncols >> 5, half0 = (nblk + 1) >> 1;
            const uint32_t b_lo = kh ? half0 : 0u, b_hi = kh ? nblk : half0;
            for (uint32_t b = b_lo; b < b_hi; ++b) {
                uint4 bx[NT][2];   // words of columns 8t .. 8t + 7: {hi, lo} x 4 pairs
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint4* xp = reinterpret_cast<const uint4*>(xrow + n * 8 * x_pitch + b * 32 + 8 * t);
                    bx[n][0] = xp[0];
                    bx[n][1] = xp[1];
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint8_t* bg = wg + m * 16 * p.w_pitch + b * 18;
                    const uint8_t* b8 = bg + 8 * p.w_pitch;
                    const float dg = half_bits_to_float(*reinterpret_cast<const uint16_t*>(bg));
                    const float d8 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b8));
                    uint32_t ag[4], a8[4];   // pair p = columns 8t + 2p, 8t + 2p + 1
#pragma unroll
                    for (int pr = 0; pr < 4; ++pr) {
                        const uint32_t vg = *reinterpret_cast<const uint16_t*>(bg + byte_off + 2 * pr);
                        const uint32_t v8 = *reinterpret_cast<const uint16_t*>(b8 + byte_off + 2 * pr);
                        const uint32_t hg = (__byte_perm(vg, 0u, 0x4140) & nib_mask) | 0x64006400u;
                        const uint32_t h8 = (__byte_perm(v8, 0u, 0x4140) & nib_mask) | 0x64006400u;
                        const __half2 rg = __hfma2(*reinterpret_cast<const __half2*>(&hg), mul, add);
                        const __half2 r8 = __hfma2(*reinterpret_cast<const __half2*>(&h8), mul, add);
                        ag[pr] = *reinterpret_cast<const uint32_t*>(&rg);
                        a8[pr] = *reinterpret_cast<const uint32_t*>(&r8);
                    }
                    const uint32_t a01[4] = {ag[0], a8[0], ag[1], a8[1]}, a23[4] = {ag[2], a8[2], ag[3], a8[3]};
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        float c[4];
                        mma16816_zero(c, a01, bx[n][0].y, bx[n][0].w);   // the small terms first: lo words
                        mma16816(c, a23, bx[n][1].y, bx[n][1].w);
                        mma16816(c, a01, bx[n][0].x, bx[n][0].z);
                        mma16816(c, a23, bx[n][1].x, bx[n][1].z);
                        acc[m][n][0] = fmaf(dg, c[0], acc[m][n][0]);
                        acc[m][n][1] = fmaf(dg, c[1], acc[m][n][1]);
                        acc[m][n][2] = fmaf(d8, c[2], acc[m][n][2]);
                        acc[m][n][3] = fmaf(d8, c[3], acc[m][n][3]);
                    }
                }
            }
        } else {
            // columns [4t, 4t + 4) of a 16-weight group; weight l of a 128-weight half sits in ql / qh as
            // quantization.cpp:1469-1499 lays out
            const uint32_t ngroups = ncols >> 4, half0 = (ngroups + 1) >> 1;
            const uint32_t j_lo = kh ? half0 : 0u, j_hi = kh ? ngroups : half0;
            const __half2 bias = __floats2half2_rn(1056.0f, 1056.0f);   // 1024 + 32
            for (uint32_t j = j_lo; j < j_hi; ++j) {
                uint4 bx[NT];
#pragma unroll
                for (int n = 0; n < NT; ++n) bx[n] = *reinterpret_cast<const uint4*>(xrow + n * 8 * x_pitch + j * 16 + 4 * t);
                const uint32_t blk = (j >> 4) * 210, jj = j & 15;
                const uint32_t h = jj >> 3, quarter = (jj & 7) >> 1, sub = jj & 1;
                const uint32_t ql_off = 64 * h + ((quarter & 1) ? 32 : 0) + 16 * sub + 4 * t;   // q2 / q4 read ql[l + 32]
                const uint32_t qh_off = 128 + 32 * h + 16 * sub + 4 * t;
                const uint32_t nib_shift = (quarter >> 1) * 4, hi_shift = quarter * 2;          // q3 / q4: high nibble
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint8_t* bg = wg + m * 16 * p.w_pitch + blk;
                    const uint8_t* b8 = bg + 8 * p.w_pitch;
                    const float sg = __fmul_rn(half_bits_to_float(*reinterpret_cast<const uint16_t*>(bg + 208)),
                                               static_cast<float>(static_cast<int8_t>(bg[192 + jj])));
                    const float s8 = __fmul_rn(half_bits_to_float(*reinterpret_cast<const uint16_t*>(b8 + 208)),
                                               static_cast<float>(static_cast<int8_t>(b8[192 + jj])));
                    uint32_t a[4];   // {row g pair 0, row g + 8 pair 0, row g pair 1, row g + 8 pair 1}
#pragma unroll
                    for (int pr = 0; pr < 2; ++pr) {
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const uint8_t* bp = r ? b8 : bg;
                            const uint32_t lo2 = *reinterpret_cast<const uint16_t*>(bp + ql_off + 2 * pr);
                            const uint32_t hi2 = *reinterpret_cast<const uint16_t*>(bp + qh_off + 2 * pr);
                            const uint32_t q2 = ((lo2 >> nib_shift) & 0x0F0Fu) | (((hi2 >> hi_shift) & 0x0303u) << 4);
                            const uint32_t hw = __byte_perm(q2, 0u, 0x4140) | 0x64006400u;
                            const __half2 rr = __hsub2(*reinterpret_cast<const __half2*>(&hw), bias);
                            a[2 * pr + r] = *reinterpret_cast<const uint32_t*>(&rr);
                        }
                    }
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        float c[4];
                        mma16816_zero(c, a, bx[n].y, bx[n].w);
                        mma16816(c, a, bx[n].x, bx[n].z);
                        acc[m][n][0] = fmaf(sg, c[0], acc[m][n][0]);
                        acc[m][n][1] = fmaf(sg, c[1], acc[m][n][1]);
                        acc[m][n][2] = fmaf(s8, c[2], acc[m][n][2]);
                        acc[m][n][3] = fmaf(s8, c[3], acc[m][n][3]);
                    }
                }
            }
        }
        __syncthreads();   // this stage may be refilled by the next iteration's issue
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

    // Every warp leaves its partial tile (its m-tile, its half of the columns) in shared memory:
    // red[kh][batch][row], C fragment c0, c1 = (row g, batch 2t, 2t + 1), c2, c3 = (row g + 8, same).
    // The column slices of a row tile are the CTAs of one cluster: after the cluster barrier CTA s adds rows
    // [s * ROWS / S, (s + 1) * ROWS / S) of all partial tiles, slice by slice and half by half, through
    // distributed shared memory - no round trip through L2, and the order is fixed, so results repeat bit for
    // bit. The second barrier keeps every CTA's tiles alive until their readers are done.
    float* red = reinterpret_cast<float*>(smem);   // [2 column halves][kXRows][kRedPitch], over the first stage
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t lrow = (mt * MT + m) * 16 + g + ((e & 2) ? 8 : 0);
                const uint32_t bn = n * 8 + 2 * t + (e & 1);
                red[(kh * kXRows + bn) * kRedPitch + lrow] = acc[m][n][e];
            }
    if (S > 1) cluster_sync_publish(); else __syncthreads();
    const uint32_t red_base = static_cast<uint32_t>(__cvta_generic_to_shared(red));
    // Rows [lrow, lrow + 4) of batch row bn, added up over the cluster's 2 S partial tiles (slice 0's two column
    // halves, slice 1's, ...). T lanes share the work: lane j takes partials j, j + T, ... - requested four at a time
    // before the first is used, so that a lane waits for one round trip through distributed shared memory per four
    // partials and not for one per partial - and the lanes' sums meet in a butterfly. With T = 1 that is the plain
    // sum in slice order; for a given launch shape T is fixed, so results repeat bit for bit.
    auto sum_tiles = [&](bool valid, uint32_t bn, uint32_t lrow, uint32_t j, uint32_t T) -> float4 {
        const uint32_t addr = red_base + (bn * kRedPitch + lrow) * 4;
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        bool have = false;
        if (valid) {
            for (uint32_t q0 = j; q0 < 2 * S; q0 += 4 * T) {
                float4 part[4];
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    const uint32_t q = q0 + u * T;
                    if (q < 2 * S) part[u] = ld_cluster_f4(addr + (q & 1u) * (kXRows * kRedPitch * 4), q >> 1);
                }
#pragma unroll
                for (uint32_t u = 0; u < 4; ++u) {
                    if (q0 + u * T >= 2 * S) continue;
                    const float4 v = part[u];
                    sum = have ? make_float4(__fadd_rn(sum.x, v.x), __fadd_rn(sum.y, v.y), __fadd_rn(sum.z, v.z), __fadd_rn(sum.w, v.w)) : v;
                    have = true;
                }
            }
        }
        for (uint32_t off = T >> 1; off; off >>= 1) {   // every lane of the warp takes part
            const float4 o = make_float4(__shfl_xor_sync(0xffffffffu, sum.x, off), __shfl_xor_sync(0xffffffffu, sum.y, off),
                                         __shfl_xor_sync(0xffffffffu, sum.z, off), __shfl_xor_sync(0xffffffffu, sum.w, off));
            sum = make_float4(__fadd_rn(sum.x, o.x), __fadd_rn(sum.y, o.y), __fadd_rn(sum.z, o.z), __fadd_rn(sum.w, o.w));
        }
        return sum;
    };
    // lanes per work item: as many (a power of two up to 8, at most one per partial) as leave every item a lane
    auto lanes_per_item = [&](uint32_t items) {
        uint32_t T = 1;
        while (T < 8 && items * T * 2 <= kMvThreads && T * 2 <= 2 * S) T *= 2;
        return T;
    };
    if (p.pair_inner) {
        // CTA s finishes gate rows [s * share, (s + 1) * share) of the tile and the up rows that go with them
        const uint32_t share = ((kPairHalf + S - 1) / S + 3u) & ~3u, rs4 = share >> 2;
        const uint32_t items = kXRows * rs4, T = lanes_per_item(items);
        for (uint32_t base = 0; base < items * T; base += kMvThreads) {
            const uint32_t w = base + tid, i = w / T, j = w - i * T;
            const uint32_t bn = i / rs4, lrow = slice * share + ((i - bn * rs4) << 2);
            const uint32_t col = tile * kPairHalf + lrow;   // column of the [batch, pair_inner] output
            const bool valid = w < items * T && bn < p.batch && lrow < kPairHalf && col < p.pair_inner;
            const float4 gt = sum_tiles(valid, bn, lrow, j, T), up = sum_tiles(valid, bn, lrow + kPairHalf, j, T);
            if (!valid || j != 0) continue;
            const float4 r = make_float4(silu_mul(gt.x, up.x), silu_mul(gt.y, up.y), silu_mul(gt.z, up.z), silu_mul(gt.w, up.w));
            const __half2 h01 = __floats2half2_rn(r.x, r.y), h23 = __floats2half2_rn(r.z, r.w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const __half2 l01 = __floats2half2_rn(r.x - f01.x, r.y - f01.y), l23 = __floats2half2_rn(r.z - f23.x, r.w - f23.y);
            *reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(p.out) + static_cast<size_t>(bn) * p.pair_inner + col) =
                make_uint4(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&l01),
                           *reinterpret_cast<const uint32_t*>(&h23), *reinterpret_cast<const uint32_t*>(&l23));
        }
    } else {
        const uint32_t share = ((kMvRows + S - 1) / S + 3u) & ~3u;   // rows this CTA adds up: a multiple of 4, the last CTA's may be short
        const uint32_t rs4 = share >> 2;                             // float4 per batch row in this CTA's share
        const bool vec_out = (p.rows & 3u) == 0;
        const uint32_t items = kXRows * rs4, T = lanes_per_item(items);
        for (uint32_t base = 0; base < items * T; base += kMvThreads) {
            const uint32_t w = base + tid, i = w / T, j = w - i * T;
            const uint32_t bn = i / rs4, lrow = slice * share + ((i - bn * rs4) << 2);
            const bool valid = w < items * T && bn < p.batch && lrow < kMvRows && row0 + lrow < p.rows;
            float4 sum = sum_tiles(valid, bn, lrow, j, T);
            if (!valid || j != 0) continue;
            if (p.rope_mode) {
                // Rows row0 + lrow .. + 3 of request bn are two adjacent pairs of one head of Q, K or V: rotate
                // (Q and K, inside the rotary dimensions), round to fp16, write Q to its buffer and K / V into the
                // request's (page, slot) of the pools - the arithmetic of qkv_split_rope_cast_kernel, pair by pair.
                const QkvRopeParams& q = p.rope;
                const uint32_t col = row0 + lrow;
                const bool is_q = col < q.q_rows, is_k = !is_q && col < q.q_rows + q.k_rows;
                const uint32_t c = is_q ? col : (is_k ? col - q.q_rows : col - q.q_rows - q.k_rows);
                float v[4] = {sum.x, sum.y, sum.z, sum.w};
                if (is_q || is_k) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint32_t pair = ((c + 2 * j) % q.head_dim) >> 1;
                        if (pair < q.rotary_pairs) {
                            const float cs = q.cos_t[static_cast<size_t>(bn) * q.rotary_pairs + pair];
                            const float sn = q.sin_t[static_cast<size_t>(bn) * q.rotary_pairs + pair];
                            const float x0 = v[2 * j], x1 = v[2 * j + 1];
                            v[2 * j] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
                            v[2 * j + 1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
                        }
                    }
                }
                const __half2 h01 = __floats2half2_rn(v[0], v[1]), h23 = __floats2half2_rn(v[2], v[3]);
                const uint2 packed = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
                if (is_q) {
                    *reinterpret_cast<uint2*>(q.q16 + static_cast<size_t>(bn) * q.q_rows + c) = packed;
                } else {
                    const uint32_t page = q.page_ids[bn], slot = q.slots[bn];
                    if (page >= q.capacity) {
                        if (c == 0) atomicOr(q.err, MLC_DEVERR_BAD_PAGE);
                    } else if (slot >= q.page_tokens) {
                        if (c == 0) atomicOr(q.err, MLC_DEVERR_BAD_SLOT);
                    } else {
                        __half* pool = is_k ? q.k_pool : q.v_pool;
                        *reinterpret_cast<uint2*>(pool + (static_cast<size_t>(page) * q.page_tokens + slot) * q.k_rows + c) = packed;
                    }
                }
                continue;
            }
            const size_t o = static_cast<size_t>(bn) * p.rows + row0 + lrow;
            if (vec_out) {
                if (p.residual) {
                    const float4 r = *reinterpret_cast<const float4*>(p.residual + o);
                    sum = make_float4(__fadd_rn(r.x, sum.x), __fadd_rn(r.y, sum.y), __fadd_rn(r.z, sum.z), __fadd_rn(r.w, sum.w));
                }
                *reinterpret_cast<float4*>(p.out + o) = sum;
            } else {
                const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (row0 + lrow + e < p.rows) p.out[o + e] = p.residual ? __fadd_rn(p.residual[o + e], vals[e]) : vals[e];
            }
        }
    }
    if (S > 1) cluster_sync_relaxed();
}

// How many clusters of S CTAs of `kernel` (threads, dynamic shared memory) the device holds at once; cached.
// Clusters are placed inside one GPC each, so this is often less than (CTAs that fit) / S - and a launch that
// needs one cluster more than fit runs as two waves.
static uint32_t max_active_clusters(mlc_ctx* ctx, const void* kernel, unsigned threads, size_t smem, unsigned S) {
    struct Entry { const void* f; size_t smem; unsigned S; int dev; uint32_t n; };
    static std::vector<Entry> cache;
    for (const Entry& e : cache)
        if (e.f == kernel && e.smem == smem && e.S == S && e.dev == ctx->device) return e.n;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(S * 64);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = std::max(1, ctx->sm_count / static_cast<int>(S));   // a guess; only the choice of S depends on it
    }
    cache.push_back({kernel, smem, S, ctx->device, static_cast<uint32_t>(n)});
    return static_cast<uint32_t>(n);
}

static uint32_t weight_pitch(uint32_t chunk_bytes) {
    // room for the enclosing 16-byte range of a chunk, and rows 4 banks apart (pitch / 4 = 4 mod 8)
    uint32_t p = (chunk_bytes + 16 + 15) / 16 * 16;
    while ((p / 4) % 8 != 4) p += 16;
    return p;
}

// Column slices (= CTAs per cluster, 8 at most, never less than one block per slice): the most slices whose
// clusters - one per row tile - are all resident at once; if even unsliced tiles do not fit one wave, the
// slicing that leaves the fewest chunks per CTA per wave. A slice is worked through in chunks of kMvChunk columns.
template <int QT, int NT, int IN, int ROWS = 64>
static int launch_matvec_nt(mlc_ctx* ctx, MatVecParams p) {
    using F = QuantFormat<QT>;
    constexpr int kMvRows = ROWS;
    auto kernel = quant_matvec_kernel<QT, NT, IN, ROWS>;
    static bool attr_set[16] = {};
    if (ctx->device >= 0 && ctx->device < 16 && !attr_set[ctx->device]) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[ctx->device] = true;
    }
    const uint32_t tiles = p.pair_inner ? (p.pair_inner + kMvRows / 2 - 1) / (kMvRows / 2) : (p.rows + kMvRows - 1) / kMvRows;
    const uint32_t unit = F::kBlockWeights;
    size_t smem = 0;
    auto shape = [&](uint32_t S) {
        p.slices = S;
        p.slice_cols = ((p.cols + S - 1) / S + unit - 1) / unit * unit;
        p.chunk_cols = std::min<uint32_t>(p.slice_cols, kMvChunk);
        p.w_pitch = weight_pitch(p.chunk_cols / F::kBlockWeights * F::kBlockBytes);
        const size_t stage = static_cast<size_t>(IN == kInSiluMul ? 2 : 1) * NT * 8 * (p.chunk_cols + kXPadWords) * 4 +
                             static_cast<size_t>(kMvRows) * p.w_pitch;
        smem = std::max(stage * kMvStages, static_cast<size_t>(2) * NT * 8 * (ROWS + 4) * sizeof(float));
    };
    uint32_t best_S = 1;
    uint64_t best_cost = ~0ull;
    for (uint32_t S = 8; S >= 1; --S) {
        if (S > 1 && p.cols / S < unit) continue;
        shape(S);
        const uint32_t fit = max_active_clusters(ctx, reinterpret_cast<const void*>(kernel), kMvThreads, smem, S);
        const uint64_t waves = (tiles + fit - 1) / fit;
        const uint64_t chunks = (p.slice_cols + p.chunk_cols - 1) / p.chunk_cols;
        const uint64_t cost = waves * (chunks + 1);   // + 1: what a wave costs beside its chunks
        if (cost < best_cost) best_cost = cost, best_S = S;
    }
    shape(best_S);
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, kernel, tiles * best_S, kMvThreads, smem, best_S, p));
    ++ctx->launches;
    return MLC_OK;
}

template <int QT, int IN>
static int launch_matvec(mlc_ctx* ctx, MatVecParams p) {
    const uint32_t nt = (p.batch + 7) / 8;
    if (nt <= 1) return launch_matvec_nt<QT, 1, IN>(ctx, p);
    if (nt <= 2) return launch_matvec_nt<QT, 2, IN>(ctx, p);
    if (nt <= 4) {
        // measured at 32 requests: 11264 x 2048 30 -> 27 us and 32000 x 2048 65 -> 51 us with the tall tile,
        // 2048 x 5632 16 -> 20 us; Q6_K's rows are too wide for two tall CTAs per SM
        if (QT == kQ4_0 && p.rows >= 8192) return launch_matvec_nt<QT, 4, IN, 128>(ctx, p);
        return launch_matvec_nt<QT, 4, IN>(ctx, p);
    }
    return launch_matvec_nt<QT, 8, IN>(ctx, p);
}

// ---------------------------------------------------------------------------------------------------
// The same mat-vec on the fifth-generation tensor cores (batch <= 32, 16-byte aligned rows)
// ---------------------------------------------------------------------------------------------------
// mma.sync reaches a fraction of the tensor cores' rate on this GPU, and the kernel above keeps that pipe
// occupied most of the time. Here the products run as tcgen05.mma with the accumulator in tensor memory:
//   A = 128 weight rows x 64 columns, the block integers as exact fp16 values, written by 8 dequantising warps
//       into shared memory in the K-major 128-byte-swizzle layout (4 slots in flight);
//   B = the chunk's activations [64 x 256 columns] in the same layout: rows 0..31 the requests' hi parts,
//       rows 32..63 their lo parts - one MMA of N = 64 instead of two of N = 32 (an MMA of this size costs
//       about the same to issue whatever its N);
//   D = one 128 x 64 fp32 tile of tensor memory per scale group (a Q4_0 block of 32 columns: 2 MMAs; a Q6_K
//       group of 16 columns: 1), 8 tiles in flight;
//   4 epilogue warps (thread = weight row) read each finished tile (tcgen05.ld), add its hi and lo halves and
//   add that, times the row's fp32 scale of the group, to 32 accumulators in registers - the same arithmetic
//   as above, group by group.
// One warp issues the MMAs. Rings are handed over with mbarriers (every wait bounded: a wait that runs out
// sets the device error word and the roles wind down). Column slices are CTAs of a cluster and add up through
// distributed shared memory as above. A CTA owns one 128-row tile.
constexpr int kTcRows = 128;
constexpr int kTcN = 32;            // requests (the batch, padded)
constexpr int kTcND = 2 * kTcN;     // MMA N: the hi activations of the 32 requests, then their lo parts
constexpr int kTcChunk = 256;       // columns per chunk: 4 atoms of 64
constexpr int kTcRawStages = 3;
constexpr int kTcSlots = 4;         // A atoms in flight
constexpr int kTcBufs = 8;          // D tiles in flight (64 columns of tensor memory each: all 512)
constexpr int kTcDequantThreads = 256;
constexpr int kTcThreads = 128 + kTcDequantThreads + 32;   // epilogue | dequantise + load | MMA issue
constexpr uint32_t kTcAtomABytes = kTcRows * 128;          // 16 KiB
constexpr uint32_t kTcAtomBBytes = kTcND * 128;            // 8 KiB: rows 0..31 hi, rows 32..63 lo
constexpr uint32_t kTcBBytes = 4 * kTcAtomBBytes;          // a chunk's activations

struct TcBars {
    uint64_t raw_full[kTcRawStages], raw_empty[kTcRawStages], raw_done[kTcRawStages];
    uint64_t a_full[kTcSlots], a_empty[kTcSlots];
    uint64_t d_full[kTcBufs], d_empty[kTcBufs];
    uint64_t b_full[2], b_empty[2];
    uint32_t tmem_slot, abort;
};

struct TcParams {
    const uint8_t* w;
    const float* x;          // fp32 [batch, x_stride] (kInPlain / kInSiluMul) or the packed words (kInPacked)
    const float* residual;
    float* out;
    uint32_t* err;
    size_t row_stride;
    uint32_t batch, rows, cols, x_stride;
    uint32_t slice_cols, slices, w_pitch;
};

template <int QT, int IN>
__global__ void __launch_bounds__(kTcThreads) quant_matvec_tc_kernel(const TcParams p) {
    using F = QuantFormat<QT>;
    constexpr int kGroupCols = QT == kQ4_0 ? 32 : 16;            // columns that share one fp32 scale
    constexpr int kGroupsPerAtom = 64 / kGroupCols;
    constexpr int kStepsPerGroup = kGroupCols / 16;
    extern __shared__ __align__(1024) uint8_t smem_unaligned[];
    // the swizzled tiles need 1024-byte alignment: the launch asks for 1 KiB more than the layout takes
    uint8_t* smem = smem_unaligned + ((1024u - (tc::smem_u32(smem_unaligned) & 1023u)) & 1023u);
    const uint32_t base = tc::smem_u32(smem);
    const uint32_t sB = base;                                    // two buffers of a chunk's activations
    const uint32_t sA = sB + 2 * kTcBBytes;                      // kTcSlots atoms
    uint8_t* raw = smem + 2 * kTcBBytes + kTcSlots * kTcAtomABytes;
    const uint32_t raw_bytes = kTcRows * p.w_pitch;
    TcBars& bars = *reinterpret_cast<TcBars*>(raw + kTcRawStages * raw_bytes);
    float* red = reinterpret_cast<float*>(raw);                  // [32][128 + 4], over the raw ring once it is done

    const uint32_t S = p.slices;
    const uint32_t tile = blockIdx.x / S, slice = blockIdx.x - tile * S;
    const uint32_t row0 = tile * kTcRows;
    const uint32_t c_begin = min(slice * p.slice_cols, p.cols), c_end = min(c_begin + p.slice_cols, p.cols);
    const uint32_t n_chunks = (c_end - c_begin + kTcChunk - 1) / kTcChunk;
    const uint32_t tid = threadIdx.x, warp = tid >> 5;

    if (tid == 0) {
        for (int i = 0; i < kTcRawStages; ++i) {
            tc::mbar_init(tc::smem_u32(&bars.raw_full[i]), kTcDequantThreads);
            tc::mbar_init(tc::smem_u32(&bars.raw_empty[i]), 128);
            tc::mbar_init(tc::smem_u32(&bars.raw_done[i]), kTcDequantThreads);
        }
        for (int i = 0; i < kTcSlots; ++i) {
            tc::mbar_init(tc::smem_u32(&bars.a_full[i]), kTcDequantThreads);
            tc::mbar_init(tc::smem_u32(&bars.a_empty[i]), 1);
        }
        for (int i = 0; i < kTcBufs; ++i) {
            tc::mbar_init(tc::smem_u32(&bars.d_full[i]), 1);
            tc::mbar_init(tc::smem_u32(&bars.d_empty[i]), 128);
        }
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(tc::smem_u32(&bars.b_full[i]), kTcDequantThreads);
            tc::mbar_init(tc::smem_u32(&bars.b_empty[i]), 1);
        }
        bars.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // rows of B past the batch stay zero for the whole kernel
    for (uint32_t i = tid; i < 2 * kTcBBytes / 16; i += kTcThreads) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 12) tc::tmem_alloc(tc::smem_u32(&bars.tmem_slot), kTcBufs * kTcND);
    tc::fence_proxy_async_smem();
    tc::fence_before();
    __syncthreads();
    tc::fence_after();
    const uint32_t tmem = bars.tmem_slot;

    // A wait that ran out: timeout bit plus where (0x6x = this kernel: 0 dequantise, 1 MMA, 2 epilogue) and the chunk.
    auto give_up = [&](uint32_t where, uint32_t chunk) {
        bars.abort = 1;
        if (atomicCAS(p.err, 0u, MLC_DEVERR_WAIT_TIMEOUT | ((0x60u + where) << 8) | (chunk << 16)) != 0u)
            atomicOr(p.err, MLC_DEVERR_WAIT_TIMEOUT);
    };

    float acc[kTcN];
#pragma unroll
    for (int n = 0; n < kTcN; ++n) acc[n] = 0.0f;

    if (warp >= 4 && warp < 12) {
        // ---------------- weight loads, activation conversion, dequantisation ----------------
        const uint32_t dt = tid - 128;                     // 0..255
        const uint32_t drow = dt & 127, dhalf = dt >> 7;   // this thread's weight row, and which 32 columns of an atom
        uint32_t a_off[4];                                 // its four 16-byte chunks inside an A atom
#pragma unroll
        for (int c = 0; c < 4; ++c) a_off[c] = tc::sw128_offset(drow, dhalf * 32 + c * 8);
        auto issue_raw = [&](uint32_t chunk) {
            if (chunk < n_chunks) {
                uint8_t* ws = raw + (chunk % kTcRawStages) * raw_bytes;
                const uint32_t c0 = c_begin + chunk * kTcChunk;
                const uint32_t ncols = min(static_cast<uint32_t>(kTcChunk), c_end - c0);
                const uint32_t b0 = c0 / F::kBlockWeights * F::kBlockBytes;
                const uint32_t b1 = b0 + ncols / F::kBlockWeights * F::kBlockBytes;
                const uint32_t a0 = b0 & ~15u, nvec = (b1 - a0 + 15) >> 4;
                const uint32_t v = dt & 15;
                if (v < nvec) {
#pragma unroll
                    for (uint32_t r = dt >> 4; r < kTcRows; r += kTcDequantThreads / 16) {
                        const uint32_t row = min(row0 + r, p.rows - 1);
                        const uint32_t dst = tc::smem_u32(ws + r * p.w_pitch + v * 16);
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst),
                                     "l"(p.w + static_cast<size_t>(row) * p.row_stride + a0 + v * 16) : "memory");
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        // this thread's share of a chunk's activations: 8 x 4 columns (request n = e * 4 + dt / 64, columns 4 (dt % 64) ..)
        constexpr int kXU = IN == kInSiluMul ? 8 : 1;
        float4 xv[8], xu[kXU];
        auto load_x = [&](uint32_t chunk) {
            const uint32_t c0 = c_begin + chunk * kTcChunk;
            const uint32_t ncols = chunk < n_chunks ? min(static_cast<uint32_t>(kTcChunk), c_end - c0) : 0u;
            const uint32_t cq = dt & 63;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t n = e * 4 + (dt >> 6);
                xv[e] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (IN == kInSiluMul) xu[e % kXU] = xv[e];
                if (n < p.batch && cq * 4 < ncols) {
                    const float* src = p.x + static_cast<size_t>(n) * p.x_stride + c0 + cq * 4;
                    xv[e] = __ldcg(reinterpret_cast<const float4*>(src));
                    if (IN == kInSiluMul) xu[e % kXU] = __ldcg(reinterpret_cast<const float4*>(src + p.cols));
                }
            }
        };
        uint32_t x_off[8];                                 // where its 8 float4 of a chunk go in a B plane
#pragma unroll
        for (int e = 0; e < 8; ++e)
            x_off[e] = ((dt & 63) >> 4) * kTcAtomBBytes + tc::sw128_offset(e * 4 + (dt >> 6), ((dt & 63) & 15) * 4);
        // the lo row of request n is row 32 + n of the tile: 4 groups of 8 rows = 4096 bytes further, same swizzle
        auto store_x = [&](uint32_t bb) {
            uint8_t* bdst = smem + bb * kTcBBytes;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t n = e * 4 + (dt >> 6);
                uint32_t h01, h23, l01, l23;
                if (IN == kInPacked) {   // {hi0, hi1}, {lo0, lo1}, {hi2, hi3}, {lo2, lo3}
                    h01 = __float_as_uint(xv[e].x); l01 = __float_as_uint(xv[e].y);
                    h23 = __float_as_uint(xv[e].z); l23 = __float_as_uint(xv[e].w);
                } else {
                    float4 w = xv[e];
                    if (IN == kInSiluMul) {
                        const float4 u = xu[e % kXU];
                        w = make_float4(silu_mul(w.x, u.x), silu_mul(w.y, u.y), silu_mul(w.z, u.z), silu_mul(w.w, u.w));
                    }
                    const __half2 a = __floats2half2_rn(w.x, w.y), b = __floats2half2_rn(w.z, w.w);
                    const float2 fa = __half22float2(a), fb = __half22float2(b);
                    const __half2 la = __floats2half2_rn(w.x - fa.x, w.y - fa.y), lb = __floats2half2_rn(w.z - fb.x, w.w - fb.y);
                    h01 = *reinterpret_cast<const uint32_t*>(&a); h23 = *reinterpret_cast<const uint32_t*>(&b);
                    l01 = *reinterpret_cast<const uint32_t*>(&la); l23 = *reinterpret_cast<const uint32_t*>(&lb);
                }
                const uint32_t off = x_off[e];
                if (n < p.batch) {
                    *reinterpret_cast<uint2*>(bdst + off) = make_uint2(h01, h23);
                    *reinterpret_cast<uint2*>(bdst + 4096 + off) = make_uint2(l01, l23);
                }
            }
        };

        // Weights never change: their first chunks are on their way before the kernel in front of this one has
        // finished; its output - the activations - is touched only after the wait.
        for (uint32_t c = 0; c < kTcRawStages; ++c) issue_raw(c);
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        asm volatile("griddepcontrol.wait;" ::: "memory");
        load_x(0);
        if (n_chunks > 0) {
            store_x(0);
            tc::fence_proxy_async_smem();
            tc::mbar_arrive(tc::smem_u32(&bars.b_full[0]));
        }
        load_x(1);

        uint32_t atom_count = 0;
        bool ok = true;
        for (uint32_t chunk = 0; chunk < n_chunks && ok; ++chunk) {
            const uint32_t stage = chunk % kTcRawStages;
            const uint32_t c0 = c_begin + chunk * kTcChunk;
            const uint32_t ncols = min(static_cast<uint32_t>(kTcChunk), c_end - c0);
            asm volatile("cp.async.wait_group %0;" ::"n"(kTcRawStages - 1) : "memory");
            tc::mbar_arrive(tc::smem_u32(&bars.raw_full[stage]));
            if (!tc::mbar_wait_bounded(tc::smem_u32(&bars.raw_full[stage]), (chunk / kTcRawStages) & 1u)) { give_up(0, chunk); ok = false; break; }
            const uint8_t* wrow = raw + stage * raw_bytes + drow * p.w_pitch + ((c0 / F::kBlockWeights * F::kBlockBytes) & 15u);
            const uint32_t n_atoms = (ncols + 63) >> 6;
            for (uint32_t a = 0; a < n_atoms; ++a, ++atom_count) {
                const uint32_t slot = atom_count % kTcSlots;
                if (atom_count >= kTcSlots &&
                    !tc::mbar_wait_bounded(tc::smem_u32(&bars.a_empty[slot]), ((atom_count / kTcSlots) - 1) & 1u)) { give_up(0, chunk); ok = false; break; }
                uint8_t* dstA = smem + 2 * kTcBBytes + slot * kTcAtomABytes;
                const uint32_t col = a * 64 + dhalf * 32;          // this thread's 32 columns inside the chunk
                uint4 out4[4];
                if (col < ncols) {
                    if (QT == kQ4_0) {
                        // 0x6400 | n is the fp16 number 1024 + n, 0x6400 | (n << 4) is 1024 + 16 n: one fused
                        // multiply-add takes either to n - 8 exactly
                        const uint8_t* blk = wrow + (col >> 5) * 18 + 2;
                        const __half2 m1 = __floats2half2_rn(1.0f, 1.0f), a1 = __floats2half2_rn(-1032.0f, -1032.0f);
                        const __half2 m2 = __floats2half2_rn(0.0625f, 0.0625f), a2 = __floats2half2_rn(-72.0f, -72.0f);
                        uint32_t lo[8], hi[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const uint32_t v = __byte_perm(*reinterpret_cast<const uint16_t*>(blk + 2 * i), 0u, 0x4140);
                            const uint32_t l = (v & 0x000F000Fu) | 0x64006400u, h = (v & 0x00F000F0u) | 0x64006400u;
                            const __half2 rl = __hfma2(*reinterpret_cast<const __half2*>(&l), m1, a1);
                            const __half2 rh = __hfma2(*reinterpret_cast<const __half2*>(&h), m2, a2);
                            lo[i] = *reinterpret_cast<const uint32_t*>(&rl);
                            hi[i] = *reinterpret_cast<const uint32_t*>(&rh);
                        }
                        out4[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);   // columns 0..7: low nibbles of bytes 0..7
                        out4[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                        out4[2] = make_uint4(hi[0], hi[1], hi[2], hi[3]);   // columns 16..23: their high nibbles
                        out4[3] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                    } else {
                        // 32 columns = two 16-weight groups jj, jj + 1 of the super-block (quantization.cpp:1469-1499)
                        const uint8_t* sb = wrow + (col >> 8) * 210;
                        const uint32_t jj = (col & 255) >> 4;
                        const __half2 bias = __floats2half2_rn(1056.0f, 1056.0f);
#pragma unroll
                        for (int gq = 0; gq < 2; ++gq) {
                            const uint32_t j = jj + gq, h = j >> 3, quarter = (j & 7) >> 1, sub = j & 1;
                            const uint32_t ql_off = 64 * h + ((quarter & 1) ? 32 : 0) + 16 * sub, qh_off = 128 + 32 * h + 16 * sub;
                            const uint32_t nib_shift = (quarter >> 1) * 4, hi_shift = quarter * 2;
                            uint32_t wv[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const uint32_t l2 = *reinterpret_cast<const uint16_t*>(sb + ql_off + 2 * i);
                                const uint32_t h2 = *reinterpret_cast<const uint16_t*>(sb + qh_off + 2 * i);
                                const uint32_t q2 = ((l2 >> nib_shift) & 0x0F0Fu) | (((h2 >> hi_shift) & 0x0303u) << 4);
                                const uint32_t hw = __byte_perm(q2, 0u, 0x4140) | 0x64006400u;
                                const __half2 rr = __hsub2(*reinterpret_cast<const __half2*>(&hw), bias);
                                wv[i] = *reinterpret_cast<const uint32_t*>(&rr);
                            }
                            out4[2 * gq] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                            out4[2 * gq + 1] = make_uint4(wv[4], wv[5], wv[6], wv[7]);
                        }
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(dstA + a_off[c]) = out4[c];
                }
                tc::fence_proxy_async_smem();
                tc::mbar_arrive(tc::smem_u32(&bars.a_full[slot]));
            }
            if (!ok) break;
            // the next chunk's activations into the other B buffer, free once the MMAs of the chunk before this one have run
            if (chunk + 1 < n_chunks) {
                const uint32_t nb = (chunk + 1) & 1u;
                if (chunk >= 1 && !tc::mbar_wait_bounded(tc::smem_u32(&bars.b_empty[nb]), (((chunk + 1) >> 1) - 1) & 1u)) { give_up(0, chunk); ok = false; break; }
                store_x(nb);
                tc::fence_proxy_async_smem();
                tc::mbar_arrive(tc::smem_u32(&bars.b_full[nb]));
                load_x(chunk + 2);
            }
            // refill this raw stage once every dequantising thread is done with it and the epilogue has its scales
            tc::mbar_arrive(tc::smem_u32(&bars.raw_done[stage]));
            if (chunk + kTcRawStages < n_chunks &&
                !(tc::mbar_wait_bounded(tc::smem_u32(&bars.raw_done[stage]), (chunk / kTcRawStages) & 1u) &&
                  tc::mbar_wait_bounded(tc::smem_u32(&bars.raw_empty[stage]), (chunk / kTcRawStages) & 1u))) { give_up(0, chunk); ok = false; break; }
            issue_raw(chunk + kTcRawStages);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp == 12) {
        // ---------------- MMA issue: the whole warp walks the loop, one elected lane issues ----------------
        constexpr uint32_t idesc = tc::idesc_f16_kmajor(kTcRows, kTcND);
        const uint64_t desc = tc::smem_desc_sw128(0, 16, 1024);
        uint32_t atom_count = 0, group_count = 0;
        bool ok = true;
        for (uint32_t chunk = 0; chunk < n_chunks && ok; ++chunk) {
            const uint32_t c0 = c_begin + chunk * kTcChunk;
            const uint32_t ncols = min(static_cast<uint32_t>(kTcChunk), c_end - c0);
            ok = tc::mbar_wait_bounded(tc::smem_u32(&bars.b_full[chunk & 1u]), (chunk >> 1) & 1u);
            if (!ok) { give_up(1, chunk); break; }
            const uint32_t n_atoms = (ncols + 63) >> 6;
            for (uint32_t a = 0; a < n_atoms && ok; ++a, ++atom_count) {
                const uint32_t slot = atom_count % kTcSlots;
                ok = tc::mbar_wait_bounded(tc::smem_u32(&bars.a_full[slot]), (atom_count / kTcSlots) & 1u);
                if (!ok) { give_up(1, chunk); break; }
                tc::fence_after();
                // descriptors of this atom's first 16-column step; the start address field counts 16-byte units
                const uint64_t a_desc = desc | ((sA + slot * kTcAtomABytes) >> 4);
                const uint64_t b_desc = desc | ((sB + (chunk & 1u) * kTcBBytes + a * kTcAtomBBytes) >> 4);
                const uint32_t groups = min(static_cast<uint32_t>(kGroupsPerAtom), (ncols - a * 64 + kGroupCols - 1) / kGroupCols);
                for (uint32_t gi = 0; gi < groups; ++gi, ++group_count) {
                    const uint32_t buf = group_count % kTcBufs;
                    if (group_count >= kTcBufs) {
                        ok = tc::mbar_wait_bounded(tc::smem_u32(&bars.d_empty[buf]), ((group_count / kTcBufs) - 1) & 1u);
                        if (!ok) { give_up(1, chunk); break; }
                        tc::fence_after();
                    }
                    if (tc::elect_one()) {
                        const uint32_t d = tmem + buf * kTcND;
#pragma unroll
                        for (int ks = 0; ks < kStepsPerGroup; ++ks) {
                            const uint32_t kstep = gi * kStepsPerGroup + ks;   // 16-column step inside the atom
                            tc::mma_f16(d, a_desc + 2 * kstep, b_desc + 2 * kstep, idesc, ks == 0 ? 0u : 1u);   // 32 bytes = 2 units
                        }
                        tc::commit(tc::smem_u32(&bars.d_full[buf]));
                    }
                    __syncwarp();
                }
                if (ok && tc::elect_one()) tc::commit(tc::smem_u32(&bars.a_empty[slot]));
                __syncwarp();
            }
            if (ok && tc::elect_one()) tc::commit(tc::smem_u32(&bars.b_empty[chunk & 1u]));
            __syncwarp();
        }
        // the last commits' arrivals land in this CTA's shared memory: see them before it is given up
        if (ok && n_chunks > 0) {
            const uint32_t last = n_chunks - 1;
            if (!tc::mbar_wait_bounded(tc::smem_u32(&bars.b_empty[last & 1u]), (last >> 1) & 1u)) give_up(1, last);
        }
    } else if (warp < 4) {
        // ---------------- epilogue: thread = weight row, TMEM lane = tid ----------------
        const uint32_t lane_base = (warp * 32u) << 16;
        uint32_t group_count = 0;
        bool ok = true;
        for (uint32_t chunk = 0; chunk < n_chunks && ok; ++chunk) {
            const uint32_t stage = chunk % kTcRawStages;
            const uint32_t c0 = c_begin + chunk * kTcChunk;
            const uint32_t ncols = min(static_cast<uint32_t>(kTcChunk), c_end - c0);
            ok = tc::mbar_wait_bounded(tc::smem_u32(&bars.raw_full[stage]), (chunk / kTcRawStages) & 1u);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; give_up(2, chunk); break; }
            // this row's scales of the chunk
            const uint8_t* wrow = raw + stage * raw_bytes + tid * p.w_pitch + ((c0 / F::kBlockWeights * F::kBlockBytes) & 15u);
            constexpr int kGroupsPerChunk = kTcChunk / kGroupCols;
            float scale[kGroupsPerChunk];
            const uint32_t n_groups = ncols / kGroupCols;
            if (QT == kQ4_0) {
#pragma unroll
                for (int i = 0; i < kGroupsPerChunk; ++i)
                    scale[i] = static_cast<uint32_t>(i) < n_groups ? half_bits_to_float(*reinterpret_cast<const uint16_t*>(wrow + i * 18)) : 0.0f;
            } else {
                const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(wrow + 208));
#pragma unroll
                for (int i = 0; i < kGroupsPerChunk; ++i)
                    scale[i] = static_cast<uint32_t>(i) < n_groups ? __fmul_rn(d, static_cast<float>(static_cast<int8_t>(wrow[192 + i]))) : 0.0f;
            }
            tc::mbar_arrive(tc::smem_u32(&bars.raw_empty[stage]));
#pragma unroll
            for (int gi = 0; gi < kGroupsPerChunk; ++gi) {
                if (static_cast<uint32_t>(gi) >= n_groups) break;
                const uint32_t buf = group_count % kTcBufs;
                ok = tc::mbar_wait_bounded(tc::smem_u32(&bars.d_full[buf]), (group_count / kTcBufs) & 1u);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; give_up(2, chunk); break; }
                tc::fence_after();
                uint32_t vh[32], vl[32];
                tc::tmem_ld32(tmem + lane_base + buf * kTcND, vh);
                tc::tmem_ld32(tmem + lane_base + buf * kTcND + kTcN, vl);
                tc::tmem_wait_ld();
                tc::fence_before();
                tc::mbar_arrive(tc::smem_u32(&bars.d_empty[buf]));
                ++group_count;
                const float sc = scale[gi];
#pragma unroll
                for (int n = 0; n < kTcN; ++n) acc[n] = fmaf(sc, __fadd_rn(__uint_as_float(vl[n]), __uint_as_float(vh[n])), acc[n]);
            }
            if (!ok) break;
        }
    }

    // ---------------- every role is done: partial tile to shared memory, tensor memory back ----------------
    tc::fence_before();
    __syncthreads();
    tc::fence_after();
    if (warp == 12) tc::tmem_dealloc(tmem, kTcBufs * kTcND);
    constexpr uint32_t kPitch = kTcRows + 4;
    if (warp < 4) {
#pragma unroll
        for (int n = 0; n < kTcN; ++n) red[n * kPitch + tid] = bars.abort ? 0.0f : acc[n];
    }
    if (S > 1) cluster_sync_publish(); else __syncthreads();
    const uint32_t r4n = kTcRows >> 2, items = p.batch * r4n;
    const uint32_t red_base = tc::smem_u32(red);
    const bool vec_out = (p.rows & 3u) == 0;
    for (uint32_t i = slice + S * tid; i < items; i += S * kTcThreads) {
        const uint32_t bn = i / r4n, lrow = (i - bn * r4n) << 2;
        if (row0 + lrow >= p.rows) continue;
        const uint32_t addr = red_base + (bn * kPitch + lrow) * 4;
        float4 sum = ld_cluster_f4(addr, 0);
        for (uint32_t k = 1; k < S; ++k) {
            const float4 v = ld_cluster_f4(addr, k);
            sum = make_float4(__fadd_rn(sum.x, v.x), __fadd_rn(sum.y, v.y), __fadd_rn(sum.z, v.z), __fadd_rn(sum.w, v.w));
        }
        const size_t o = static_cast<size_t>(bn) * p.rows + row0 + lrow;
        if (vec_out) {
            if (p.residual) {
                const float4 r = *reinterpret_cast<const float4*>(p.residual + o);
                sum = make_float4(__fadd_rn(r.x, sum.x), __fadd_rn(r.y, sum.y), __fadd_rn(r.z, sum.z), __fadd_rn(r.w, sum.w));
            }
            *reinterpret_cast<float4*>(p.out + o) = sum;
        } else {
            const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (row0 + lrow + e < p.rows) p.out[o + e] = p.residual ? __fadd_rn(p.residual[o + e], vals[e]) : vals[e];
        }
    }
    if (S > 1) cluster_sync_relaxed();
}

// Which kernel: MLC_B200_MATVEC=tcgen05 in the environment selects the tensor-memory kernel for batches of up to
// 32 requests; the default is the mma.sync kernel, which is the faster of the two as they stand (both are
// bound by the instructions around the tensor-core work - dequantising, converting, scaling - and by
// per-launch latency, not by the tensor cores or HBM).
static bool matvec_tc_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("MLC_B200_MATVEC");
        return e && e[0] == 't';
    }();
    return on;
}

template <int QT, int IN>
static int launch_matvec_tc(mlc_ctx* ctx, const MatVecParams& mp) {
    using F = QuantFormat<QT>;
    TcParams p{};
    p.w = mp.w;
    p.x = mp.x;
    p.residual = mp.residual;
    p.out = mp.out;
    p.err = ctx->d_err;
    p.row_stride = mp.row_stride;
    p.batch = mp.batch;
    p.rows = mp.rows;
    p.cols = mp.cols;
    p.x_stride = mp.x_stride;
    // column slices (CTAs per cluster, a slice a whole number of atoms): the most whose clusters - one per 128-row
    // tile - are all resident at once, else none
    const uint32_t tiles = (mp.rows + kTcRows - 1) / kTcRows;
    const uint32_t unit = std::max<uint32_t>(F::kBlockWeights, 64);
    p.w_pitch = weight_pitch(kTcChunk / F::kBlockWeights * F::kBlockBytes);
    const size_t smem = 2 * kTcBBytes + kTcSlots * kTcAtomABytes + static_cast<size_t>(kTcRawStages) * kTcRows * p.w_pitch +
                        sizeof(TcBars) + 1024;   // slack for the 1024-byte alignment of the tiles
    auto kernel = quant_matvec_tc_kernel<QT, IN>;
    static bool attr_set[16] = {};
    if (ctx->device >= 0 && ctx->device < 16 && !attr_set[ctx->device]) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[ctx->device] = true;
    }
    uint32_t S = 1;
    for (uint32_t c = 8; c > 1; c >>= 1) {
        if (mp.cols / c < unit) continue;
        if (tiles <= max_active_clusters(ctx, reinterpret_cast<const void*>(kernel), kTcThreads, smem, c)) { S = c; break; }
    }
    p.slices = S;
    p.slice_cols = ((mp.cols + S - 1) / S + unit - 1) / unit * unit;
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, kernel, tiles * S, kTcThreads, smem, S, p));
    ++ctx->launches;
    return MLC_OK;
}

static int check_matvec(mlc_ctx* ctx, int qt, const void* w, const void* in, const void* out, size_t batch, size_t rows,
                        size_t cols, size_t row_stride, size_t x_stride) {
    if (!w || !in || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (batch == 0 || rows == 0 || cols == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    const size_t bw = qt == kQ6_K ? 256 : 32, bb = qt == kQ6_K ? 210 : 18;
    if (cols % bw) return ctx->fail(MLC_ERR_UNSUPPORTED, "cols must be a whole number of quantisation blocks");
    if (row_stride < cols / bw * bb) return ctx->fail(MLC_ERR_INVALID_ARG, "row_stride shorter than a row");
    if (row_stride % 2 || reinterpret_cast<uintptr_t>(w) % 2) return ctx->fail(MLC_ERR_INVALID_ARG, "weights and row_stride must be even");
    if (reinterpret_cast<uintptr_t>(in) % 16 || x_stride % 4) return ctx->fail(MLC_ERR_INVALID_ARG, "input must be 16-byte aligned");
    if (rows % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 16) return ctx->fail(MLC_ERR_INVALID_ARG, "output must be 16-byte aligned");
    if (batch > 64) return ctx->fail(MLC_ERR_UNSUPPORTED, "batch above 64");
    if (rows >= (1u << 31) || cols >= (1u << 31)) return ctx->fail(MLC_ERR_UNSUPPORTED, "dimension too large");
    return MLC_OK;
}

}  // namespace mlcb

using namespace mlcb;

extern "C" {

static int encode_rms_norm(mlc_ctx* ctx, const void* in, const void* weight, float epsilon, size_t batch, size_t length,
                           void* out, void* out_f16, void* packed) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!in || !weight || (!out && !packed)) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (batch == 0 || length == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (batch >= (1u << 31) || length >= (1u << 31)) return ctx->fail(MLC_ERR_UNSUPPORTED, "dimension too large");
    if (packed && length % 4) return ctx->fail(MLC_ERR_UNSUPPORTED, "packed output needs a length divisible by 4");
    if ((length % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) |
                               reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(packed)) % 16))
        return ctx->fail(MLC_ERR_INVALID_ARG, "buffers must be 16-byte aligned");
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, rms_norm_batched_kernel, static_cast<unsigned>(batch), 256, 0, 1,
                                       static_cast<const float*>(in), static_cast<const float*>(weight), epsilon,
                                       static_cast<uint32_t>(length), static_cast<float*>(out), static_cast<__half*>(out_f16),
                                       static_cast<uint32_t*>(packed)));
    ++ctx->launches;
    return MLC_OK;
}

int mlc_encode_rms_norm_batched(mlc_ctx* ctx, const void* in, const void* weight, float epsilon, size_t batch,
                                size_t length, void* out, void* out_f16) {
    if (ctx && !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    return encode_rms_norm(ctx, in, weight, epsilon, batch, length, out, out_f16, nullptr);
}

int mlc_encode_rms_norm_batched_packed(mlc_ctx* ctx, const void* in, const void* weight, float epsilon, size_t batch,
                                       size_t length, void* out, void* packed) {
    if (ctx && !packed) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    return encode_rms_norm(ctx, in, weight, epsilon, batch, length, out, nullptr, packed);
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
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, add_kernel, static_cast<unsigned>((threads + 255) / 256), 256, 0, 1,
                                       static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(out), n4,
                                       total_elements));
    ++ctx->launches;
    return MLC_OK;
}

int mlc_encode_silu_mul_batched(mlc_ctx* ctx, const void* gate, const void* up, void* out, size_t total_elements) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!gate || !up || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (total_elements == 0) return MLC_OK;
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, silu_mul_kernel, static_cast<unsigned>((total_elements + 255) / 256), 256, 0, 1,
                                       static_cast<const float*>(gate), static_cast<const float*>(up), static_cast<float*>(out),
                                       total_elements));
    ++ctx->launches;
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
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, gate_up_silu_mul_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0, 1,
                                       static_cast<const float*>(gate_up), static_cast<float*>(gate), static_cast<float*>(up),
                                       static_cast<float*>(out), static_cast<uint32_t>(batch), static_cast<uint32_t>(ffn_inner),
                                       static_cast<uint32_t>(ffn_gate_up_rows)));
    ++ctx->launches;
    return MLC_OK;
}

int mlc_encode_argmax_rows(mlc_ctx* ctx, const void* logits, size_t batch, size_t vocab, size_t group_rows, void* out_ids) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (!logits || !out_ids) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (batch == 0 || vocab == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (batch >= (1u << 31) || vocab >= (size_t(1) << 32)) return ctx->fail(MLC_ERR_UNSUPPORTED, "dimension too large");
    if (group_rows == 0 || group_rows > vocab) group_rows = vocab;
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, argmax_rows_kernel, static_cast<unsigned>(batch), 256, 0, 1,
                                       static_cast<const float*>(logits), static_cast<uint32_t>(batch), static_cast<uint32_t>(vocab),
                                       static_cast<uint32_t>(group_rows), static_cast<uint32_t*>(out_ids)));
    ++ctx->launches;
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
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, embedding_q4_0_kernel, static_cast<unsigned>(batch), 256, 0, 1,
                                       static_cast<const uint8_t*>(table), row_stride, static_cast<const uint32_t*>(token_ids),
                                       static_cast<uint32_t>(vocab), static_cast<uint32_t>(cols), static_cast<float*>(out), ctx->d_err));
    ++ctx->launches;
    return MLC_OK;
}

static int encode_matvec(mlc_ctx* ctx, int qt, int in_mode, const void* weights, const void* in, const void* residual,
                         size_t batch, size_t rows, size_t cols, size_t row_stride, size_t x_stride, void* out,
                         size_t pair_inner = 0, const QkvRopeParams* rope = nullptr) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    int st = check_matvec(ctx, qt, weights, in, out, batch, rows, cols, row_stride, x_stride);
    if (st != MLC_OK) return st;
    if (in_mode == kInSiluMul && x_stride < 2 * cols) return ctx->fail(MLC_ERR_INVALID_ARG, "row shorter than gate + up");
    if (residual && rows % 4 == 0 && reinterpret_cast<uintptr_t>(residual) % 16)
        return ctx->fail(MLC_ERR_INVALID_ARG, "residual must be 16-byte aligned");
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
    p.aligned16 = (row_stride % 16 == 0 && reinterpret_cast<uintptr_t>(weights) % 16 == 0) ? 1u : 0u;
    p.pair_inner = static_cast<uint32_t>(pair_inner);
    if (rope) {
        p.rope_mode = 1;
        p.rope = *rope;
    }
    const bool tcore = !pair_inner && !rope && matvec_tc_enabled() && p.aligned16 && batch <= static_cast<size_t>(kTcN);
#define MLCB_MATVEC_DISPATCH(QT, IN) (tcore ? launch_matvec_tc<QT, IN>(ctx, p) : launch_matvec<QT, IN>(ctx, p))
    if (qt == kQ6_K) {
        if (in_mode == kInSiluMul) return MLCB_MATVEC_DISPATCH(kQ6_K, kInSiluMul);
        return in_mode == kInPacked ? MLCB_MATVEC_DISPATCH(kQ6_K, kInPacked) : MLCB_MATVEC_DISPATCH(kQ6_K, kInPlain);
    }
    if (in_mode == kInSiluMul) return MLCB_MATVEC_DISPATCH(kQ4_0, kInSiluMul);
    return in_mode == kInPacked ? MLCB_MATVEC_DISPATCH(kQ4_0, kInPacked) : MLCB_MATVEC_DISPATCH(kQ4_0, kInPlain);
#undef MLCB_MATVEC_DISPATCH
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
                                  int input_kind, const void* residual, size_t batch, size_t rows, size_t cols,
                                  size_t row_stride, void* out) {
    if (quant != kQ4_0 && quant != kQ6_K) return ctx ? ctx->fail(MLC_ERR_INVALID_ARG, "unknown quantisation") : MLC_ERR_INVALID_ARG;
    if (input_kind < kInPlain || input_kind > kInPacked)
        return ctx ? ctx->fail(MLC_ERR_INVALID_ARG, "unknown input kind") : MLC_ERR_INVALID_ARG;
    return encode_matvec(ctx, quant, input_kind, weights, in, residual, batch, rows, cols, row_stride, in_stride, out);
}

int mlc_encode_matmul_gate_up_silu_packed(mlc_ctx* ctx, int quant, const void* weights, const void* in, size_t in_stride,
                                          int input_kind, size_t batch, size_t ffn_inner, size_t cols, size_t row_stride,
                                          void* packed) {
    if (quant != kQ4_0 && quant != kQ6_K) return ctx ? ctx->fail(MLC_ERR_INVALID_ARG, "unknown quantisation") : MLC_ERR_INVALID_ARG;
    if (input_kind != kInPlain && input_kind != kInPacked)
        return ctx ? ctx->fail(MLC_ERR_INVALID_ARG, "input kind must be 0 or 2") : MLC_ERR_INVALID_ARG;
    if (ctx && (ffn_inner == 0 || ffn_inner % 4)) return ctx->fail(MLC_ERR_UNSUPPORTED, "ffn_inner must be a positive multiple of 4");
    if (ctx && ffn_inner >= (size_t(1) << 30)) return ctx->fail(MLC_ERR_UNSUPPORTED, "dimension too large");
    return encode_matvec(ctx, quant, input_kind, weights, in, nullptr, batch, 2 * ffn_inner, cols, row_stride, in_stride, packed,
                         ffn_inner);
}

}  // extern "C"

namespace mlcb {

int encode_matvec_qkv_rope(mlc_ctx* ctx, int quant, int input_kind, const void* weights, const void* in, size_t in_stride,
                           size_t cols, size_t row_stride, const QkvRopeParams& rope) {
    if (quant != kQ4_0 && quant != kQ6_K) return ctx->fail(MLC_ERR_INVALID_ARG, "unknown quantisation");
    if (input_kind != kInPlain && input_kind != kInPacked) return ctx->fail(MLC_ERR_INVALID_ARG, "input kind must be 0 or 2");
    const size_t rows = static_cast<size_t>(rope.q_rows) + rope.k_rows + rope.v_rows;
    if (rope.head_dim % 4 || reinterpret_cast<uintptr_t>(rope.q16) % 16 || reinterpret_cast<uintptr_t>(rope.k_pool) % 8 ||
        reinterpret_cast<uintptr_t>(rope.v_pool) % 8)
        return ctx->fail(MLC_ERR_UNSUPPORTED, "head_dim must be a multiple of 4, q 16-byte and the pools 8-byte aligned");
    // `out` of the plain form is not written in this mode; q stands in for the pointer checks
    return encode_matvec(ctx, quant, input_kind, weights, in, nullptr, rope.batch, rows, cols, row_stride, in_stride, rope.q16, 0,
                         &rope);
}

}  // namespace mlcb
