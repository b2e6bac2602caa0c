// Log-sum-exp combine of gathered split-KV partials, and CUDA-graph bracketing of a
// pass.
//
// The reference has neither: its kernel walks a whole sequence in one threadgroup
// (compiler/runtime/metal_runtime.mm:2260-2331) and its pass is one Metal command
// buffer (metal_runtime.hpp:181-183). The combine applies between partials the
// rule the reference applies between tiles (mm:2304-2329):
//   m* = max_k m_k, w_k = exp(m_k - m*), l = sum_k l_k w_k, O = sum_k o_k w_k / l.
#include <cuda_fp16.h>

#include "attn_internal.hpp"

namespace mlcb {

// One thread per (row, 4 consecutive d): o_parts [parts, rows, D] un-normalised,
// ml_parts [parts, rows, 2] (m in natural-log units).
template <typename OT>
__global__ void lse_combine_kernel(const float* __restrict__ o_parts, const float* __restrict__ ml_parts,
                                   uint32_t parts, size_t rows, uint32_t D, OT* __restrict__ out) {
    const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint32_t vec_per_row = D / 4;
    if (gid >= rows * vec_per_row) return;
    const size_t row = gid / vec_per_row;
    const uint32_t d0 = static_cast<uint32_t>(gid % vec_per_row) * 4;
    float mstar = -INFINITY;
    for (uint32_t k = 0; k < parts; ++k) mstar = fmaxf(mstar, ml_parts[(static_cast<size_t>(k) * rows + row) * 2]);
    float l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t k = 0; k < parts; ++k) {
        const float2 ml = *reinterpret_cast<const float2*>(ml_parts + (static_cast<size_t>(k) * rows + row) * 2);
        const float w = (ml.x == -INFINITY) ? 0.f : expf(ml.x - mstar);
        l += ml.y * w;
        const float4 v = *reinterpret_cast<const float4*>(o_parts + (static_cast<size_t>(k) * rows + row) * D + d0);
        acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    if constexpr (sizeof(OT) == 4) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + row * D + d0) = acc;
    } else {
        __half2* dst = reinterpret_cast<__half2*>(reinterpret_cast<__half*>(out) + row * D + d0);
        dst[0] = __floats2half2_rn(acc.x, acc.y);
        dst[1] = __floats2half2_rn(acc.z, acc.w);
    }
}

}  // namespace mlcb

using namespace mlcb;

struct mlc_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;  // kernel nodes recorded during the capture
};

extern "C" {

int mlc_encode_lse_combine(mlc_ctx* ctx, const float* o_parts, const float* ml_parts, size_t parts,
                           size_t rows, size_t head_dim, void* out, int o_dtype) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!o_parts || !ml_parts || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (parts == 0 || rows == 0 || head_dim == 0 || head_dim % 4 != 0) return ctx->fail(MLC_ERR_INVALID_ARG, "bad dimensions");
    if (o_dtype != MLC_F32 && o_dtype != MLC_F16) return ctx->fail(MLC_ERR_INVALID_ARG, "dtype must be MLC_F32 or MLC_F16");
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    DeviceGuard guard(ctx->device);
    const size_t total = rows * (head_dim / 4);
    const int threads = 128;
    const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
    if (o_dtype == MLC_F32)
        lse_combine_kernel<float><<<blocks, threads, 0, ctx->stream>>>(o_parts, ml_parts, static_cast<uint32_t>(parts), rows,
                                                                       static_cast<uint32_t>(head_dim), static_cast<float*>(out));
    else
        lse_combine_kernel<__half><<<blocks, threads, 0, ctx->stream>>>(o_parts, ml_parts, static_cast<uint32_t>(parts), rows,
                                                                        static_cast<uint32_t>(head_dim), static_cast<__half*>(out));
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

int mlc_graph_begin_capture(mlc_ctx* ctx) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "capture needs an open pass");
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    MLCB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    ctx->launches_at_capture = ctx->launches;
    return MLC_OK;
}

int mlc_graph_end_capture(mlc_ctx* ctx, mlc_graph** out) {
    if (!ctx || !out) return MLC_ERR_INVALID_ARG;
    *out = nullptr;
    if (!ctx->capturing) return ctx->fail(MLC_ERR_INVALID_ARG, "no capture in progress");
    DeviceGuard guard(ctx->device);
    ctx->capturing = false;
    auto* g = new mlc_graph();
    g->kernels = ctx->launches - ctx->launches_at_capture;  // recorded, not run
    ctx->launches = ctx->launches_at_capture;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
        if (g->graph) cudaGraphDestroy(g->graph);
        delete g;
        return ctx->fail(MLC_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    }
    *out = g;
    return MLC_OK;
}

int mlc_graph_launch(mlc_ctx* ctx, mlc_graph* graph) {
    if (!ctx || !graph || !graph->exec) return MLC_ERR_INVALID_ARG;
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, cudaGraphLaunch(graph->exec, ctx->stream));
    ctx->launches += graph->kernels;
    return MLC_OK;
}

void mlc_graph_destroy(mlc_ctx* ctx, mlc_graph* graph) {
    if (!graph) return;
    if (ctx) {
        DeviceGuard guard(ctx->device);
        cudaStreamSynchronize(ctx->stream);
    }
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    if (graph->graph) cudaGraphDestroy(graph->graph);
    delete graph;
}

}  // extern "C"
