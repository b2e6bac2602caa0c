// General paged decode-attention kernel: any head_dim <= 256, any page size, any
// head grouping, fp32 or fp16 Q/O, fp32 arithmetic throughout.
//
// Same contract as the reference's MSL kernel paged_flash_attention
// (compiler/runtime/metal_runtime.mm:2216-2335): online softmax over the
// request's pages, GQA map kv_h = h*KVH/H (mm:2237), causal rule kv_pos > q_pos
// masked (mm:2286), seq_len == 0 or a fully masked row gives zeros (mm:2254,
// 2333). It is the kernel behind shapes the TMA/tensor-core kernel does not take
// (page sizes that are not a multiple of its tile, head_dim other than 64/128,
// more than 16 query heads per KV head) and behind mlc_ctx_set_attention_kernel(1).
//
// Mapping: one CTA per (request, query head); its 4 warps take tokens
// round-robin, the 32 lanes of a warp split head_dim; the dot product is
// finished with warp shuffles, each warp keeps its own (m, l, o) and the four
// states are merged through shared memory with the log-sum-exp rule.
#include <cuda_fp16.h>

#include "attn_internal.hpp"

namespace mlcb {

static constexpr int kGenWarps = 4;
static constexpr int kGenMaxPerLane = 8;  // head_dim <= 256

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, size_t i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p, size_t i) { return __half2float(p[i]); }

template <typename QT, typename OT>
__global__ void __launch_bounds__(kGenWarps * 32)
paged_attention_general_kernel(const QT* __restrict__ q, const __half* __restrict__ k_pages,
                               const __half* __restrict__ v_pages, OT* __restrict__ o,
                               const uint32_t* __restrict__ pt_flat,
                               const uint32_t* __restrict__ pt_off,
                               const uint32_t* __restrict__ eff_len,  // tokens each request attends to
                               uint32_t H, uint32_t KVH, uint32_t D, uint32_t P, float scale,
                               uint32_t capacity, uint32_t* __restrict__ err,
                               float* __restrict__ o_partial, float* __restrict__ ml_partial) {
    const uint32_t req = blockIdx.x / H, head = blockIdx.x % H;
    const uint32_t kv_h = static_cast<uint32_t>((static_cast<uint64_t>(head) * KVH) / H);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t S = eff_len[req];
    const uint32_t pt_base = pt_off[req];
    const size_t row = (static_cast<size_t>(req) * H + head) * D;
    const size_t page_elems = static_cast<size_t>(P) * KVH * D;

    float qv[kGenMaxPerLane], acc[kGenMaxPerLane];
#pragma unroll
    for (int i = 0; i < kGenMaxPerLane; ++i) {
        uint32_t d = lane + 32 * i;
        qv[i] = d < D ? load_as_float<QT>(q, row + d) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (uint32_t pos = warp; pos < S; pos += kGenWarps) {
        uint32_t page = pt_flat[pt_base + pos / P];
        if (page >= capacity) {
            if (lane == 0) atomicOr(err, MLC_DEVERR_BAD_PAGE);
            continue;
        }
        size_t base = static_cast<size_t>(page) * page_elems +
                      static_cast<size_t>(pos % P) * (static_cast<size_t>(KVH) * D) +
                      static_cast<size_t>(kv_h) * D;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < kGenMaxPerLane; ++i) {
            uint32_t d = lane + 32 * i;
            if (d < D) dot += qv[i] * __half2float(k_pages[base + d]);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        float s = dot * scale;
        float m_new = fmaxf(m, s);
        float alpha = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        float p = expf(s - m_new);
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < kGenMaxPerLane; ++i) {
            uint32_t d = lane + 32 * i;
            if (d < D) acc[i] = acc[i] * alpha + p * __half2float(v_pages[base + d]);
        }
        m = m_new;
    }

    __shared__ float s_m[kGenWarps], s_l[kGenWarps];
    __shared__ float s_o[kGenWarps][kGenMaxPerLane * 32];
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < kGenMaxPerLane; ++i) s_o[warp][lane + 32 * i] = acc[i];
    __syncthreads();
    float mstar = -INFINITY;
#pragma unroll
    for (int w = 0; w < kGenWarps; ++w) mstar = fmaxf(mstar, s_m[w]);
    float wgt[kGenWarps], lsum = 0.0f;
#pragma unroll
    for (int w = 0; w < kGenWarps; ++w) {
        wgt[w] = (s_m[w] == -INFINITY) ? 0.0f : expf(s_m[w] - mstar);
        lsum += s_l[w] * wgt[w];
    }
    float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
    if (o_partial && threadIdx.x == 0) {  // split-KV partial: un-normalised o plus (m, l)
        ml_partial[(static_cast<size_t>(req) * H + head) * 2] = mstar;
        ml_partial[(static_cast<size_t>(req) * H + head) * 2 + 1] = lsum;
    }
    for (uint32_t d = threadIdx.x; d < D; d += blockDim.x) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kGenWarps; ++w) v += s_o[w][d] * wgt[w];
        if (o_partial) {
            o_partial[row + d] = v;
            continue;
        }
        v *= inv;
        if constexpr (sizeof(OT) == 4) o[row + d] = v;
        else o[row + d] = __float2half_rn(v);
    }
}

int launch_attention_general(mlc_ctx* ctx, const AttnArgs& a, const uint32_t* d_pt_flat,
                             const uint32_t* d_pt_off, const uint32_t* d_eff_len) {
    dim3 grid(static_cast<unsigned>(a.batch * a.H)), block(kGenWarps * 32);
    uint32_t cap32 = a.capacity ? static_cast<uint32_t>(a.capacity) : 0xFFFFFFFFu;
    auto kp = static_cast<const __half*>(a.k_pages);
    auto vp = static_cast<const __half*>(a.v_pages);
#define MLCB_GEN_LAUNCH(QT, OT)                                                                   \
    paged_attention_general_kernel<QT, OT><<<grid, block, 0, ctx->stream>>>(                       \
        static_cast<const QT*>(a.q), kp, vp, static_cast<OT*>(a.o), d_pt_flat, d_pt_off, d_eff_len, \
        static_cast<uint32_t>(a.H), static_cast<uint32_t>(a.KVH), static_cast<uint32_t>(a.D),       \
        static_cast<uint32_t>(a.P), a.scale, cap32, ctx->d_err, a.o_partial, a.ml_partial)
    if (a.q_dtype == MLC_F32 && a.o_dtype == MLC_F32) MLCB_GEN_LAUNCH(float, float);
    else if (a.q_dtype == MLC_F32) MLCB_GEN_LAUNCH(float, __half);
    else if (a.o_dtype == MLC_F32) MLCB_GEN_LAUNCH(__half, float);
    else MLCB_GEN_LAUNCH(__half, __half);
#undef MLCB_GEN_LAUNCH
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

}  // namespace mlcb
