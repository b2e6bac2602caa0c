// Split-KV across GPUs: exchange of the per-rank partials over NVLink peer memory, fused with
// the log-sum-exp combine. One kernel per step and rank replaces "NCCL all-gather + combine":
//
//   1. push    CTA b < world copies this rank's (o, m, l) partial with plain 16-byte stores into
//              slot `rank` of peer (rank+1+b)%world's gather buffer (its own included), then
//              publishes: __threadfence_system, CTA barrier, one system-scope store of the step's
//              sequence number into that peer's flag word for this rank;
//   2. wait    every CTA polls its OWN memory's flag words (ld.acquire.sys) until all `world`
//              ranks have published this step - bounded: after kMaxPolls polls the kernel records
//              MLC_DEVERR_WAIT_TIMEOUT, skips the combine and returns (the context stays usable);
//   3. combine the merge rule of the reference kernel between tiles (metal_runtime.mm:2304-2329),
//              applied between ranks, read from the local gather buffer with L1-bypassing loads.
//
// The reference has one device (metal_runtime.mm:5774-5777) and no counterpart. The partial is
// ~33 KiB per rank at the long-context workload, so the exchange is latency-bound: what this
// removes is the collective's launch and protocol latency plus one kernel boundary.
//
// Buffers are double-buffered by step parity. A peer can only be one step ahead (its step s+1
// needs this rank's push of s+1, which this rank issues after its own combine of s in stream
// order), so parity s+2 is never written before this rank has read parity s. The step counter
// lives in device memory and is advanced by the last CTA to finish, so the call can be captured
// in a CUDA graph. Peer pointers come from cudaIpc handles of plain cudaMalloc memory; loads from
// peer memory are never issued (pushes only), and no TMA or multicast is involved.
//
// The grid never exceeds the SM count (one small CTA each), so every CTA of a launch is resident
// while it polls. Ranks are separate processes on separate GPUs; nothing here waits on another
// kernel of the same GPU.
#include <cuda_fp16.h>

#include <cmath>
#include <cstring>
#include <vector>

#include "ctx.hpp"

namespace mlcb {

constexpr int kMaxRanks = 16;
constexpr uint32_t kMaxPolls = 1u << 20;  // default limit; ~1 us per system-scope poll: about a second

struct ExchangeParams {
    const float* o_part;    // [rows, D]
    const float* ml_part;   // [rows, 2]
    char* peer[kMaxRanks];  // base of every rank's gather buffer as mapped into this process
    char* local;            // this rank's own gather buffer (= peer[rank])
    void* out;
    uint32_t* err;
    uint32_t* seq;          // step counter (local)
    uint32_t* done;         // CTAs finished in this launch (local)
    size_t slot_floats;     // floats per (parity, rank) slot = max_rows * (D + 2)
    size_t flags_off;       // byte offset of the flag words [2][world] (max_units = 1)
    uint32_t max_units;
    uint32_t rank, world, rows, D;
    uint32_t max_polls;     // limit of the flag wait (mlc_ctx_set_wait_limit, default kMaxPolls)
    unsigned long long* trace;   // optional: 8 %globaltimer stamps of CTA 0 (MLC_B200_TRACE=1), else null
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <typename OT>
__global__ void __launch_bounds__(256) exchange_lse_combine_kernel(const ExchangeParams p) {
    __shared__ uint32_t s_step;
    __shared__ int s_ok;
    auto stamp = [&](int i) {
        if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            p.trace[i] = t;
        }
    };
    stamp(0);
    if (threadIdx.x == 0) {
        s_step = *reinterpret_cast<volatile uint32_t*>(p.seq);
        s_ok = 1;
    }
    __syncthreads();
    const uint32_t step = s_step, parity = step & 1u, stamp_value = step + 1u;  // never 0: zeroed flags match nothing
    const size_t o_floats = static_cast<size_t>(p.rows) * p.D, ml_floats = static_cast<size_t>(p.rows) * 2;

    // ---- 1. push this rank's partial into one peer's buffer ----
    if (blockIdx.x < p.world) {
        const uint32_t dst_rank = (p.rank + 1u + blockIdx.x) % p.world;
        float* dst = reinterpret_cast<float*>(p.peer[dst_rank]) + (static_cast<size_t>(parity) * p.world + p.rank) * p.slot_floats;
        const float4* so = reinterpret_cast<const float4*>(p.o_part);
        float4* d4 = reinterpret_cast<float4*>(dst);
        for (size_t i = threadIdx.x; i < o_floats / 4; i += blockDim.x) d4[i] = so[i];
        const float2* sm = reinterpret_cast<const float2*>(p.ml_part);
        float2* d2 = reinterpret_cast<float2*>(dst + o_floats);
        for (size_t i = threadIdx.x; i < ml_floats / 2; i += blockDim.x) d2[i] = sm[i];
        __threadfence_system();
        __syncthreads();
        stamp(1);
        if (threadIdx.x == 0) {
            uint32_t* flag = reinterpret_cast<uint32_t*>(p.peer[dst_rank] + p.flags_off) +
                             (static_cast<size_t>(parity) * p.world + p.rank) * p.max_units;
            st_release_sys(flag, stamp_value);
        }
        stamp(2);
    }

    // ---- 2. wait (bounded) until every rank's partial of this step is in local memory ----
    if (threadIdx.x < p.world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(p.local + p.flags_off) +
                               (static_cast<size_t>(parity) * p.world + threadIdx.x) * p.max_units;
        bool seen = false;
        for (uint32_t i = 0; i < p.max_polls; ++i) {
            if (static_cast<int32_t>(ld_acquire_sys(flag) - stamp_value) >= 0) {
                seen = true;
                break;
            }
            __nanosleep(200);
        }
        if (!seen) {
            s_ok = 0;
            atomicOr(p.err, MLC_DEVERR_WAIT_TIMEOUT | (0x50u << 8) | (threadIdx.x << 16));
        }
    }
    __syncthreads();
    stamp(3);

    // ---- 3. combine: m* = max_k m_k, w_k = exp(m_k - m*), O = sum_k o_k w_k / sum_k l_k w_k ----
    if (s_ok) {
        const float* base = reinterpret_cast<const float*>(p.local) + static_cast<size_t>(parity) * p.world * p.slot_floats;
        const uint32_t vec_per_row = p.D / 4;
        const size_t total = static_cast<size_t>(p.rows) * vec_per_row;
        for (size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; gid < total;
             gid += static_cast<size_t>(gridDim.x) * blockDim.x) {
            const size_t row = gid / vec_per_row;
            const uint32_t d0 = static_cast<uint32_t>(gid % vec_per_row) * 4;
            float mstar = -INFINITY;
            for (uint32_t k = 0; k < p.world; ++k)
                mstar = fmaxf(mstar, __ldcg(base + k * p.slot_floats + o_floats + row * 2));
            float l = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t k = 0; k < p.world; ++k) {
                const float* slot = base + k * p.slot_floats;
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(slot + o_floats + row * 2));
                const float w = (ml.x == -INFINITY) ? 0.f : expf(ml.x - mstar);
                l += ml.y * w;
                const float4 v = __ldcg(reinterpret_cast<const float4*>(slot + row * p.D + d0));
                acc.x += v.x * w; acc.y += v.y * w; acc.z += v.z * w; acc.w += v.w * w;
            }
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
            if constexpr (sizeof(OT) == 4) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + row * p.D + d0) = acc;
            } else {
                __half2* dst = reinterpret_cast<__half2*>(reinterpret_cast<__half*>(p.out) + row * p.D + d0);
                dst[0] = __floats2half2_rn(acc.x, acc.y);
                dst[1] = __floats2half2_rn(acc.z, acc.w);
            }
        }
    }

    // ---- the last CTA to finish advances the step counter (graph replays need no host argument) ----
    __syncthreads();
    stamp(4);
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.done, 1u) == gridDim.x - 1) {
            *p.done = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(p.seq) = step + 1u;
        }
    }
}

}  // namespace mlcb

using namespace mlcb;

struct mlc_exchange {
    int rank = 0, world = 1;
    size_t max_rows = 0, D = 0, slot_floats = 0, flags_off = 0, bytes = 0;
    char* local = nullptr;
    char* peer[kMaxRanks] = {};
    bool attached = false;
    bool by_pointer = false;   // peers given as addresses of this process (nothing to close)
};

extern "C" {

int mlc_exchange_layout(int world, size_t max_rows, size_t head_dim, size_t* slot_floats, size_t* flags_offset,
                        size_t* total_bytes) {
    if (world < 1 || world > kMaxRanks || max_rows == 0 || head_dim == 0 || head_dim % 4) return MLC_ERR_INVALID_ARG;
    // rounded up to whole 16-byte vectors: every (parity, rank) slot then starts on a 16-byte boundary
    // whatever the parity of max_rows (the kernel moves the o rows as float4)
    const size_t slot = (max_rows * (head_dim + 2) + 3) / 4 * 4;
    const size_t flags = ((2 * static_cast<size_t>(world) * slot * 4 + 255) / 256) * 256;
    if (slot_floats) *slot_floats = slot;
    if (flags_offset) *flags_offset = flags;
    // behind the flag words [2 parities][world] (256 bytes): the slots of the fused attention + exchange
    // kernel, [2 parities][world] of max_rows * (head_dim * 8 + 16) bytes - every float travels beside a
    // 4-byte step stamp, so that a row is known to be complete from its own bytes, without a flag behind a
    // fence - then the step counter and the CTA count (256 bytes)
    const size_t ll_slot = max_rows * (head_dim * 8 + 16);
    const size_t ll_bytes = ((2 * static_cast<size_t>(world) * ll_slot + 255) / 256) * 256;
    if (total_bytes) *total_bytes = flags + 256 + ll_bytes + 256;
    return MLC_OK;
}

int mlc_exchange_create(mlc_ctx* ctx, int rank, int world, size_t max_rows, size_t head_dim, mlc_exchange** out) {
    if (!ctx || !out) return MLC_ERR_INVALID_ARG;
    *out = nullptr;
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return ctx->fail(MLC_ERR_INVALID_ARG, "rank / world out of range (at most %d ranks)", kMaxRanks);
    if (max_rows == 0 || head_dim == 0 || head_dim % 4) return ctx->fail(MLC_ERR_INVALID_ARG, "head_dim must be a positive multiple of 4");
    DeviceGuard guard(ctx->device);
    auto* ex = new mlc_exchange();
    ex->rank = rank;
    ex->world = world;
    ex->max_rows = max_rows;
    ex->D = head_dim;
    mlc_exchange_layout(world, max_rows, head_dim, &ex->slot_floats, &ex->flags_off, &ex->bytes);
    // plain cudaMalloc: the block is exported whole through a cudaIpc handle
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ex->local), ex->bytes);
    if (e == cudaSuccess) e = cudaMemset(ex->local, 0, ex->bytes);
    if (e != cudaSuccess) {
        if (ex->local) cudaFree(ex->local);
        delete ex;
        return ctx->fail(MLC_ERR_OOM, "exchange buffer: %s", cudaGetErrorString(e));
    }
    ++ctx->allocations;
    ex->peer[rank] = ex->local;
    ex->attached = world == 1;
    *out = ex;
    return MLC_OK;
}

int mlc_exchange_handle(mlc_ctx* ctx, mlc_exchange* ex, void* handle_out) {
    if (!ctx || !ex || !handle_out) return MLC_ERR_INVALID_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == MLC_IPC_HANDLE_BYTES, "handle size");
    DeviceGuard guard(ctx->device);
    cudaIpcMemHandle_t h;
    MLCB_CUDA(ctx, cudaIpcGetMemHandle(&h, ex->local));
    std::memcpy(handle_out, &h, sizeof(h));
    return MLC_OK;
}

int mlc_exchange_attach(mlc_ctx* ctx, mlc_exchange* ex, const void* handles) {
    if (!ctx || !ex || !handles) return MLC_ERR_INVALID_ARG;
    if (ex->attached) return ctx->fail(MLC_ERR_INVALID_ARG, "exchange already attached");
    DeviceGuard guard(ctx->device);
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const char*>(handles) + static_cast<size_t>(r) * MLC_IPC_HANDLE_BYTES, sizeof(h));
        void* ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int k = 0; k < r; ++k)
                if (k != ex->rank && ex->peer[k]) {
                    cudaIpcCloseMemHandle(ex->peer[k]);
                    ex->peer[k] = nullptr;
                }
            return ctx->fail(MLC_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d: %s", r, cudaGetErrorString(e));
        }
        ex->peer[r] = static_cast<char*>(ptr);
    }
    ex->attached = true;
    return MLC_OK;
}

int mlc_exchange_attach_pointers(mlc_ctx* ctx, mlc_exchange* ex, void* const* bases) {
    if (!ctx || !ex || !bases) return MLC_ERR_INVALID_ARG;
    if (ex->attached) return ctx->fail(MLC_ERR_INVALID_ARG, "exchange already attached");
    for (int r = 0; r < ex->world; ++r)
        if (r != ex->rank && !bases[r]) return ctx->fail(MLC_ERR_INVALID_ARG, "null gather buffer for rank %d", r);
    for (int r = 0; r < ex->world; ++r)
        if (r != ex->rank) ex->peer[r] = static_cast<char*>(bases[r]);
    ex->by_pointer = true;
    ex->attached = true;
    return MLC_OK;
}

void* mlc_exchange_local_buffer(const mlc_exchange* ex) { return ex ? ex->local : nullptr; }

}  // extern "C"

namespace mlcb {
// What the fused attention + exchange kernel needs to know about an exchange object (attn_decode_tma.cu).
bool exchange_describe(const mlc_exchange* ex, ExchangeView* v) {
    if (!ex || !ex->attached) return false;
    for (int r = 0; r < ex->world; ++r) v->peer[r] = ex->peer[r];
    v->local = ex->local;
    v->seq = reinterpret_cast<uint32_t*>(ex->local + ex->bytes - 256);
    v->done = v->seq + 1;
    v->slot_floats = ex->slot_floats;
    v->flags_off = ex->flags_off;
    v->ll_off = ex->flags_off + 256;
    v->ll_slot_bytes = ex->max_rows * (ex->D * 8 + 16);
    v->rank = static_cast<uint32_t>(ex->rank);
    v->world = static_cast<uint32_t>(ex->world);
    v->max_rows = ex->max_rows;
    v->D = ex->D;
    return true;
}
}  // namespace mlcb

extern "C" {

int mlc_exchange_read_trace(mlc_ctx* ctx, unsigned long long* out8) {
    if (!ctx || !out8 || !ctx->d_trace) return MLC_ERR_INVALID_ARG;
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    MLCB_CUDA(ctx, cudaMemcpy(out8, ctx->d_trace + ctx->trace_words - 8, 64, cudaMemcpyDeviceToHost));
    return MLC_OK;
}

size_t mlc_exchange_slot_floats(const mlc_exchange* ex) { return ex ? ex->slot_floats : 0; }

int mlc_encode_exchange_lse_combine(mlc_ctx* ctx, mlc_exchange* ex, const float* o_partial, const float* ml_partial,
                                    size_t rows, void* out, int o_dtype) {
    if (!ctx || !ex) return MLC_ERR_INVALID_ARG;
    if (!ex->attached) return ctx->fail(MLC_ERR_INVALID_ARG, "exchange not attached to its peers");
    if (!o_partial || !ml_partial || !out) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (rows == 0 || rows > ex->max_rows) return ctx->fail(MLC_ERR_INVALID_ARG, "rows %zu outside 1..%zu", rows, ex->max_rows);
    if (o_dtype != MLC_F16 && o_dtype != MLC_F32) return ctx->fail(MLC_ERR_INVALID_ARG, "o dtype must be MLC_F16 or MLC_F32");
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (reinterpret_cast<uintptr_t>(o_partial) % 16 || reinterpret_cast<uintptr_t>(ml_partial) % 8 ||
        reinterpret_cast<uintptr_t>(out) % 16)
        return ctx->fail(MLC_ERR_INVALID_ARG, "buffers must be 16-byte aligned");
    DeviceGuard guard(ctx->device);
    ExchangeParams p{};
    p.o_part = o_partial;
    p.ml_part = ml_partial;
    for (int r = 0; r < ex->world; ++r) p.peer[r] = ex->peer[r];
    p.local = ex->local;
    p.out = out;
    p.err = ctx->d_err;
    p.seq = reinterpret_cast<uint32_t*>(ex->local + ex->bytes - 256);
    p.max_units = 1;
    p.done = p.seq + 1;
    p.slot_floats = ex->slot_floats;
    p.flags_off = ex->flags_off;
    p.rank = static_cast<uint32_t>(ex->rank);
    p.world = static_cast<uint32_t>(ex->world);
    p.rows = static_cast<uint32_t>(rows);
    p.D = static_cast<uint32_t>(ex->D);
    p.max_polls = ctx->wait_limit ? ctx->wait_limit : kMaxPolls;
    // stamps of the exchange go behind the decode kernel's in the trace buffer (its last 8 words)
    p.trace = ctx->d_trace ? ctx->d_trace + ctx->trace_words - 8 : nullptr;
    const size_t total = rows * (ex->D / 4);
    size_t blocks = (total + 255) / 256;
    if (blocks < static_cast<size_t>(ex->world)) blocks = ex->world;
    // every CTA polls: all of them must be resident at once
    if (blocks > static_cast<size_t>(ctx->sm_count)) blocks = ctx->sm_count;
    if (o_dtype == MLC_F32)
        exchange_lse_combine_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(p);
    else
        exchange_lse_combine_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(p);
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

void mlc_exchange_destroy(mlc_ctx* ctx, mlc_exchange* ex) {
    if (!ex) return;
    if (ctx) {
        DeviceGuard guard(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        for (int r = 0; r < ex->world; ++r)
            if (r != ex->rank && ex->peer[r] && !ex->by_pointer) cudaIpcCloseMemHandle(ex->peer[r]);
        if (ex->local) cudaFree(ex->local);
    }
    delete ex;
}

}  // extern "C"
