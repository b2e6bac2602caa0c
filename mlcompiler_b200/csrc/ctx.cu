// Context, buffer helpers and pass bracketing of the C ABI.
//
// Stands in for the device-API part of the reference's MetalExecutor singleton
// (compiler/runtime/metal_runtime.hpp:181-183, 693-703): scratch buffers,
// name-keyed cached buffers, upload/download and the begin/flush bracket that
// the reference maps onto one Metal command buffer and that maps here onto one
// CUDA stream.
#include "ctx.hpp"

#include <cstdlib>
#include <cstring>

namespace mlcb {

static constexpr size_t kStageAlign = 256;

bool stage_reserve(mlc_ctx* ctx, size_t bytes, void** host, void** dev) {
    size_t need = (bytes + kStageAlign - 1) / kStageAlign * kStageAlign;
    if (need == 0) need = kStageAlign;
    for (auto& c : ctx->stage) {
        if (c.cap - c.used >= need) {
            *host = c.host + c.used;
            *dev = c.dev + c.used;
            c.used += need;
            return true;
        }
    }
    StageChunk c;
    size_t last = ctx->stage.empty() ? (size_t(1) << 20) : ctx->stage.back().cap * 2;
    c.cap = need > last ? need : last;
    if (cudaHostAlloc(reinterpret_cast<void**>(&c.host), c.cap, cudaHostAllocDefault) != cudaSuccess) {
        ctx->last_error = "cudaHostAlloc failed for the staging area";
        return false;
    }
    if (cudaMalloc(reinterpret_cast<void**>(&c.dev), c.cap) != cudaSuccess) {
        cudaFreeHost(c.host);
        ctx->last_error = "cudaMalloc failed for the staging area";
        return false;
    }
    ctx->allocations += 2;
    c.used = need;
    *host = c.host;
    *dev = c.dev;
    ctx->stage.push_back(c);
    return true;
}

bool stage_commit(mlc_ctx* ctx, void* host, void* dev, size_t bytes) {
    if (bytes == 0) return true;
    cudaError_t e = cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) {
        ctx->last_error = std::string("staging copy failed: ") + cudaGetErrorString(e);
        return false;
    }
    return true;
}

void* stage_to_device(mlc_ctx* ctx, const void* host, size_t bytes) {
    void *h = nullptr, *d = nullptr;
    if (!stage_reserve(ctx, bytes, &h, &d)) return nullptr;
    if (bytes) std::memcpy(h, host, bytes);
    if (!stage_commit(ctx, h, d, bytes)) return nullptr;
    return d;
}

void stage_reset(mlc_ctx* ctx) {
    for (auto& c : ctx->stage) c.used = 0;
}

int ensure_workspace(mlc_ctx* ctx, size_t bytes, size_t counters) {
    if ((bytes > ctx->work_bytes || counters > ctx->n_counters) && ctx->capturing)
        return ctx->fail(MLC_ERR_UNSUPPORTED, "workspace must grow: run the step once outside the capture first");
    if (bytes > ctx->work_bytes) {
        MLCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->d_work) cudaFree(ctx->d_work);
        ctx->d_work = nullptr;
        size_t want = bytes + bytes / 2;
        if (cudaMalloc(&ctx->d_work, want) != cudaSuccess) {
            ctx->work_bytes = 0;
            return ctx->fail(MLC_ERR_OOM, "split-KV workspace of %zu bytes unavailable", want);
        }
        ctx->work_bytes = want;
        ++ctx->allocations;
    }
    if (counters > ctx->n_counters) {
        MLCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->d_counters) cudaFree(ctx->d_counters);
        ctx->d_counters = nullptr;
        size_t want = counters * 2;
        if (cudaMalloc(reinterpret_cast<void**>(&ctx->d_counters), want * 4) != cudaSuccess) {
            ctx->n_counters = 0;
            return ctx->fail(MLC_ERR_OOM, "split-KV counters unavailable");
        }
        // Counters start at zero and every launch leaves them at zero again.
        MLCB_CUDA(ctx, cudaMemsetAsync(ctx->d_counters, 0, want * 4, ctx->stream));
        ctx->n_counters = want;
        ++ctx->allocations;
    }
    return MLC_OK;
}

void reset_after_device_error(mlc_ctx* ctx) {
    cudaMemset(ctx->d_err, 0, 4);
    if (ctx->d_counters && ctx->n_counters) cudaMemset(ctx->d_counters, 0, ctx->n_counters * 4);
    for (uint32_t* block : ctx->ext_counter_block)
        if (block) cudaMemset(block, 0, kExtCounterBytes);
}

size_t resolve_capacity(const mlc_ctx* ctx, const void* pool, size_t claimed, size_t page_bytes) {
    if (claimed) return claimed;
    auto it = ctx->allocs.find(pool);
    if (it != ctx->allocs.end() && page_bytes) return it->second / page_bytes;
    return 0;
}

}  // namespace mlcb

using namespace mlcb;

extern "C" {

int mlc_ctx_create(int device, void* stream, mlc_ctx** out) {
    if (!out) return MLC_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0 || device < 0 || device >= count) {
        cudaGetLastError();
        return MLC_ERR_NO_DEVICE;
    }
    DeviceGuard guard(device);
    auto* ctx = new mlc_ctx();
    ctx->device = device;
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        delete ctx;
        return MLC_ERR_CUDA;
    }
    ctx->sm_count = prop.multiProcessorCount;
    if (stream) {
        ctx->stream = static_cast<cudaStream_t>(stream);
    } else {
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete ctx;
            return MLC_ERR_CUDA;
        }
        ctx->own_stream = true;
    }
    if (cudaMalloc(reinterpret_cast<void**>(&ctx->d_err), 4) != cudaSuccess ||
        cudaMemset(ctx->d_err, 0, 4) != cudaSuccess) {
        delete ctx;
        return MLC_ERR_CUDA;
    }
    if (const char* t = std::getenv("MLC_B200_TRACE"); t && *t == '1') {
        ctx->trace_words = size_t(1) << 16;
        if (cudaMalloc(reinterpret_cast<void**>(&ctx->d_trace), ctx->trace_words * 8) != cudaSuccess) ctx->d_trace = nullptr;
        else cudaMemset(ctx->d_trace, 0, ctx->trace_words * 8);
    }
    *out = ctx;
    return MLC_OK;
}

// Copies the phase stamps of the last traced decode launch: [ctas][4 warps][8] u64
// nanosecond timestamps. Returns the number of CTAs, 0 when tracing is off.
uint32_t mlc_ctx_read_trace(mlc_ctx* ctx, unsigned long long* out, size_t max_words, int previous) {
    if (!ctx || !ctx->d_trace || !out) return 0;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    size_t words = static_cast<size_t>(ctx->trace_ctas) * 32;
    if (words > max_words) words = max_words;
    const uint32_t half = previous ? 1u - ctx->trace_parity : ctx->trace_parity;
    cudaMemcpy(out, ctx->d_trace + half * (ctx->trace_words / 2), words * 8, cudaMemcpyDeviceToHost);
    return ctx->trace_ctas;
}

void mlc_ctx_destroy(mlc_ctx* ctx) {
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    destroy_plan_cache(ctx);
    destroy_tmap_cache(ctx);
    destroy_pass_args(ctx);
    for (auto& kv : ctx->allocs) cudaFree(const_cast<void*>(kv.first));
    for (auto& c : ctx->stage) {
        cudaFreeHost(c.host);
        cudaFree(c.dev);
    }
    if (ctx->d_work) cudaFree(ctx->d_work);
    if (ctx->d_counters) cudaFree(ctx->d_counters);
    if (ctx->d_err) cudaFree(ctx->d_err);
    if (ctx->h_err) cudaFreeHost(ctx->h_err);
    if (ctx->d_trace) cudaFree(ctx->d_trace);
    for (cudaEvent_t e : ctx->pass_events) cudaEventDestroy(e);
    if (ctx->h2d_stream) cudaStreamDestroy(ctx->h2d_stream);
    if (ctx->d2h_stream) cudaStreamDestroy(ctx->d2h_stream);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int mlc_ctx_available(const mlc_ctx* ctx) { return ctx && ctx->device >= 0 ? 1 : 0; }

const char* mlc_last_error(const mlc_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

void* mlc_ctx_stream(const mlc_ctx* ctx) { return ctx ? ctx->stream : nullptr; }

uint64_t mlc_ctx_launch_count(const mlc_ctx* ctx) { return ctx ? ctx->launches : 0; }

uint64_t mlc_ctx_alloc_count(const mlc_ctx* ctx) { return ctx ? ctx->allocations : 0; }

int mlc_ctx_set_wait_limit(mlc_ctx* ctx, uint32_t polls) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    ctx->wait_limit = polls;
    return MLC_OK;
}

int mlc_ctx_set_attention_kernel(mlc_ctx* ctx, int which) {
    if (!ctx || which < 0 || which > 1) return MLC_ERR_INVALID_ARG;
    ctx->force_general = which;
    return MLC_OK;
}

int mlc_device_error_word(mlc_ctx* ctx, uint32_t* word) {
    if (!ctx || !word) return MLC_ERR_INVALID_ARG;
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    MLCB_CUDA(ctx, cudaMemcpy(word, ctx->d_err, 4, cudaMemcpyDeviceToHost));
    if (*word) reset_after_device_error(ctx);
    return MLC_OK;
}

void* mlc_alloc(mlc_ctx* ctx, size_t bytes) {
    if (!ctx || bytes == 0) return nullptr;
    DeviceGuard guard(ctx->device);
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        ctx->last_error = "cudaMalloc failed";
        return nullptr;
    }
    ctx->allocs[p] = bytes;
    ++ctx->allocations;
    return p;
}

void mlc_free(mlc_ctx* ctx, void* buffer) {
    if (!ctx || !buffer) return;
    auto it = ctx->allocs.find(buffer);
    if (it == ctx->allocs.end()) return;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(buffer);
    ctx->allocs.erase(it);
}

size_t mlc_buffer_bytes(const mlc_ctx* ctx, const void* buffer) {
    if (!ctx) return 0;
    auto it = ctx->allocs.find(buffer);
    return it == ctx->allocs.end() ? 0 : it->second;
}

int mlc_upload(mlc_ctx* ctx, void* buffer, const void* src, size_t bytes, size_t dst_offset) {
    if (!ctx || !buffer || (!src && bytes)) return MLC_ERR_INVALID_ARG;
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, cudaMemcpyAsync(static_cast<char*>(buffer) + dst_offset, src, bytes,
                                   cudaMemcpyHostToDevice, ctx->stream));
    MLCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MLC_OK;
}

int mlc_download(mlc_ctx* ctx, const void* buffer, void* dst, size_t bytes, size_t src_offset) {
    if (!ctx || !buffer || (!dst && bytes)) return MLC_ERR_INVALID_ARG;
    DeviceGuard guard(ctx->device);
    MLCB_CUDA(ctx, cudaMemcpyAsync(dst, static_cast<const char*>(buffer) + src_offset, bytes,
                                   cudaMemcpyDeviceToHost, ctx->stream));
    MLCB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MLC_OK;
}

void* mlc_cached_buffer(mlc_ctx* ctx, const char* name, size_t bytes) {
    if (!ctx || !name) return nullptr;
    auto it = ctx->cached.find(name);
    if (it != ctx->cached.end() && it->second.second >= bytes) return it->second.first;
    if (it != ctx->cached.end()) {
        mlc_free(ctx, it->second.first);
        ctx->cached.erase(it);
    }
    void* p = mlc_alloc(ctx, bytes ? bytes : 1);
    if (!p) return nullptr;
    ctx->cached[name] = {p, bytes};
    return p;
}

int mlc_pass_begin(mlc_ctx* ctx) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    ctx->pass_open = true;
    return MLC_OK;
}

int mlc_pass_is_open(const mlc_ctx* ctx) { return ctx && ctx->pass_open ? 1 : 0; }

int mlc_pass_flush(mlc_ctx* ctx) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return MLC_OK;  // the reference's flush is a no-op without an open CB
    DeviceGuard guard(ctx->device);
    ctx->pass_open = false;
    // the error word travels behind the pass's kernels, so one synchronisation covers both
    if (!ctx->h_err) {
        if (cudaHostAlloc(reinterpret_cast<void**>(&ctx->h_err), 4, cudaHostAllocDefault) != cudaSuccess) ctx->h_err = nullptr;
        else ++ctx->allocations;
    }
    bool word_queued = false;
    if (ctx->h_err) {
        *ctx->h_err = 0;
        word_queued = cudaMemcpyAsync(ctx->h_err, ctx->d_err, 4, cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess;
    }
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) ++ctx->sync_epoch;
    if (e == cudaSuccess && ctx->host_pass_done) {  // copies back of a host-buffer pass run on their own stream
        e = cudaEventSynchronize(ctx->host_pass_done);
        ctx->host_pass_done = nullptr;
    }
    stage_reset(ctx);
    if (e != cudaSuccess) return ctx->fail(MLC_ERR_CUDA, "pass failed: %s", cudaGetErrorString(e));
    uint32_t word = 0;
    if (word_queued) word = *ctx->h_err;
    else MLCB_CUDA(ctx, cudaMemcpy(&word, ctx->d_err, 4, cudaMemcpyDeviceToHost));
    if (word) {
        reset_after_device_error(ctx);
        return ctx->fail(MLC_ERR_DEVICE_FLAG, "a kernel of this pass recorded error word 0x%x", word);
    }
    return MLC_OK;
}

}  // extern "C"
