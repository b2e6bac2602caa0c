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

#include "ctx.hpp"

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
                                                               __half* __restrict__ out16) {
    __shared__ float part[8];
    dependent_launch_gate();
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

constexpr int kMvRows = 64;         // weight rows per CTA: 4 m-tiles of 16, each worked on by two warps (half the columns each)
constexpr int kMvThreads = 256;
constexpr int kMvChunk = 256;       // columns staged in shared memory at a time (a multiple of both block sizes)
constexpr int kXPadWords = 4;       // words of padding per activation row in shared memory: rows land 4 banks apart
constexpr int kMvStages = 2;        // chunks in flight per CTA

enum : int { kQ4_0 = 0, kQ6_K = 1 };
enum : int { kInPlain = 0, kInSiluMul = 1 };

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
    uint32_t slices;         // CTAs per cluster
    uint32_t aligned16;      // weights and row_stride on 16-byte boundaries: vector copies
};

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// 16 bytes at `local_smem_addr` of CTA `rank` of this cluster.
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

constexpr int kRedPitch = 68;    // floats per batch row of a partial tile (64 rows + 4): lanes t land 8 banks apart

// Shared memory of one pipeline stage: the chunk's activations as fp32 words [kXRows][chunk + 4] (turned in
// place into {hi, lo} fp16 pairs), with SiLU input a second such array for the `up` half, then the chunk's
// weight bytes [128][w_pitch].
template <int QT, int NT, int IN>
__global__ void __launch_bounds__(kMvThreads) quant_matvec_kernel(const MatVecParams p) {
    using F = QuantFormat<QT>;
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
    const uint32_t c_begin = min(slice * p.slice_cols, p.cols), c_end = min(c_begin + p.slice_cols, p.cols);
    const uint32_t n_chunks = (c_end - c_begin + p.chunk_cols - 1) / p.chunk_cols;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int mt = warp & 3, kh = warp >> 2;   // the warp's m-tile and its half of every chunk's columns

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
                        const uint32_t row = min(row0 + r, p.rows - 1);
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
                    const uint32_t row = min(row0 + r, p.rows - 1);
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

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.0f;

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
        {
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
        const uint8_t* wg = ws + (mt * 16 + g) * p.w_pitch + w_shift;
        const uint8_t* w8 = wg + 8 * p.w_pitch;
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
                const uint8_t* bg = wg + b * 18;
                const uint8_t* b8 = w8 + b * 18;
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
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma16816(c, a01, bx[n][0].y, bx[n][0].w);   // the small terms first: lo words
                    mma16816(c, a23, bx[n][1].y, bx[n][1].w);
                    mma16816(c, a01, bx[n][0].x, bx[n][0].z);
                    mma16816(c, a23, bx[n][1].x, bx[n][1].z);
                    acc[n][0] = fmaf(dg, c[0], acc[n][0]);
                    acc[n][1] = fmaf(dg, c[1], acc[n][1]);
                    acc[n][2] = fmaf(d8, c[2], acc[n][2]);
                    acc[n][3] = fmaf(d8, c[3], acc[n][3]);
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
                const uint8_t* bg = wg + blk;
                const uint8_t* b8 = w8 + blk;
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
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma16816(c, a, bx[n].y, bx[n].w);
                    mma16816(c, a, bx[n].x, bx[n].z);
                    acc[n][0] = fmaf(sg, c[0], acc[n][0]);
                    acc[n][1] = fmaf(sg, c[1], acc[n][1]);
                    acc[n][2] = fmaf(s8, c[2], acc[n][2]);
                    acc[n][3] = fmaf(s8, c[3], acc[n][3]);
                }
            }
        }
        __syncthreads();   // this stage may be refilled by the next iteration's issue
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

    // Every warp leaves its partial tile (its m-tile, its half of the columns) in shared memory:
    // red[kh][batch][row], C fragment c0, c1 = (row g, batch 2t, 2t + 1), c2, c3 = (row g + 8, same).
    // The column slices of a row tile are the CTAs of one cluster: after the cluster barrier CTA s adds rows
    // [s * 64 / S, (s + 1) * 64 / S) of all 2 S partial tiles, slice by slice and half by half, through
    // distributed shared memory - no round trip through L2, and the order is fixed, so results repeat bit for
    // bit. The second barrier keeps every CTA's tiles alive until their readers are done.
    float* red = reinterpret_cast<float*>(smem);   // [2][kXRows][kRedPitch], over the first stage
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t lrow = mt * 16 + g + ((e & 2) ? 8 : 0);
            const uint32_t bn = n * 8 + 2 * t + (e & 1);
            red[(kh * kXRows + bn) * kRedPitch + lrow] = acc[n][e];
        }
    if (S > 1) cluster_sync_all(); else __syncthreads();
    const uint32_t rs4 = (kMvRows / S) >> 2;                 // float4 per batch row in this CTA's share
    const uint32_t red_base = static_cast<uint32_t>(__cvta_generic_to_shared(red));
    const bool vec_out = (p.rows & 3u) == 0;
    for (uint32_t i = tid; i < kXRows * rs4; i += kMvThreads) {
        const uint32_t bn = i / rs4, lrow = slice * (kMvRows / S) + ((i - bn * rs4) << 2);
        if (bn >= p.batch || row0 + lrow >= p.rows) continue;
        const uint32_t addr0 = red_base + (bn * kRedPitch + lrow) * 4;
        const uint32_t addr1 = addr0 + kXRows * kRedPitch * 4;
        float4 sum = ld_cluster_f4(addr0, 0);
        for (uint32_t k = 0; k < S; ++k) {
            if (k) {
                const float4 v = ld_cluster_f4(addr0, k);
                sum = make_float4(__fadd_rn(sum.x, v.x), __fadd_rn(sum.y, v.y), __fadd_rn(sum.z, v.z), __fadd_rn(sum.w, v.w));
            }
            const float4 v = ld_cluster_f4(addr1, k);
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
    if (S > 1) cluster_sync_all();
}

static uint32_t weight_pitch(uint32_t chunk_bytes) {
    // room for the enclosing 16-byte range of a chunk, and rows 4 banks apart (pitch / 4 = 4 mod 8)
    uint32_t p = (chunk_bytes + 16 + 15) / 16 * 16;
    while ((p / 4) % 8 != 4) p += 16;
    return p;
}

template <int QT, int NT, int IN>
static int launch_matvec_nt(mlc_ctx* ctx, const MatVecParams& p, unsigned ctas, size_t smem) {
    auto kernel = quant_matvec_kernel<QT, NT, IN>;
    static bool attr_set[16] = {};
    if (ctx->device >= 0 && ctx->device < 16 && !attr_set[ctx->device]) {
        MLCB_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[ctx->device] = true;
    }
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, kernel, ctas, kMvThreads, smem, p.slices, p));
    ++ctx->launches;
    return MLC_OK;
}

template <int QT, int IN>
static int launch_matvec(mlc_ctx* ctx, MatVecParams p) {
    using F = QuantFormat<QT>;
    const uint32_t tiles = (p.rows + kMvRows - 1) / kMvRows;
    // Column slices (= CTAs per cluster): as many as it takes to put two CTAs on every SM, 8 at most, and never
    // slices of less than one block. A slice is worked through in chunks of kMvChunk columns.
    uint32_t S = 1;
    while (S < 8 && tiles * S < 2u * static_cast<uint32_t>(ctx->sm_count) && p.cols / (2 * S) >= F::kBlockWeights) S *= 2;
    const uint32_t unit = F::kBlockWeights;
    p.slices = S;
    p.slice_cols = ((p.cols + S - 1) / S + unit - 1) / unit * unit;
    p.chunk_cols = std::min<uint32_t>(p.slice_cols, kMvChunk);
    p.w_pitch = weight_pitch(p.chunk_cols / F::kBlockWeights * F::kBlockBytes);
    const uint32_t nt = (p.batch + 7) / 8;
    const int NT = nt <= 1 ? 1 : (nt <= 2 ? 2 : (nt <= 4 ? 4 : 8));
    const size_t stage = static_cast<size_t>(IN == kInSiluMul ? 2 : 1) * NT * 8 * (p.chunk_cols + kXPadWords) * 4 +
                         static_cast<size_t>(kMvRows) * p.w_pitch;
    const size_t smem = std::max(stage * kMvStages, static_cast<size_t>(2) * NT * 8 * kRedPitch * sizeof(float));
    const unsigned ctas = tiles * S;
    switch (NT) {
        case 1: return launch_matvec_nt<QT, 1, IN>(ctx, p, ctas, smem);
        case 2: return launch_matvec_nt<QT, 2, IN>(ctx, p, ctas, smem);
        case 4: return launch_matvec_nt<QT, 4, IN>(ctx, p, ctas, smem);
        default: return launch_matvec_nt<QT, 8, IN>(ctx, p, ctas, smem);
    }
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
    MLCB_CUDA(ctx, launch_layer_kernel(ctx, rms_norm_batched_kernel, static_cast<unsigned>(batch), 256, 0, 1,
                                       static_cast<const float*>(in), static_cast<const float*>(weight), epsilon,
                                       static_cast<uint32_t>(length), static_cast<float*>(out), static_cast<__half*>(out_f16)));
    ++ctx->launches;
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
                         size_t batch, size_t rows, size_t cols, size_t row_stride, size_t x_stride, void* out) {
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
