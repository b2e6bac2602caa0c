// Internal definition of the per-GPU context behind the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/mlc_b200.h"

namespace mlcb {

// Pinned-host + device staging area for the small u32 host arrays every call
// carries (page tables, lengths, positions). Regions handed out between two
// resets never overlap, so an async H2D copy can still be in flight while the
// next call fills its own region.
struct StageChunk {
    uint8_t* host = nullptr;
    uint8_t* dev = nullptr;
    size_t cap = 0;
    size_t used = 0;
};

// Caller-provided split-KV scratch (the fixed array of the allocation-free entry point): the last
// kExtCounterBytes of each of its two halves hold the arrival counters of cut units, at an address
// that does not depend on the plan.
static constexpr size_t kExtCounterBytes = 16384;

// Pools a decode launch writes its step's rows into: two for a layer's launch, all layers' for a whole pass.
struct PoolWrites {
    const void* few[2] = {nullptr, nullptr};
    std::vector<const void*> many;
};

// An exchange object (peer_exchange.cu) as the fused attention + exchange kernel sees it.
struct ExchangeView {
    char* peer[16] = {};
    char* local = nullptr;
    uint32_t* seq = nullptr;
    uint32_t* done = nullptr;
    size_t slot_floats = 0, flags_off = 0, max_rows = 0, D = 0;
    size_t ll_off = 0, ll_slot_bytes = 0;   // the stamped slots of the fused attention + exchange kernel
    uint32_t rank = 0, world = 1;
};

struct AttnPlanCache;  // attn_api.cu
struct TensorMapCache; // attn_decode_tma.cu

}  // namespace mlcb

struct mlc_ctx {
    int device = -1;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    bool pass_open = false;
    bool capturing = false;          // between mlc_graph_begin_capture and mlc_graph_end_capture
    uint64_t launches_at_capture = 0;
    int sm_count = 0;
    int force_general = 0;
    uint32_t wait_limit = 0;        // polls before a flag wait gives up; 0 = the kernel's default (about a second)
    int last_attention_kernel = 0;  // 0 none yet, 1 general, 2 TMA / tensor-core
    uint64_t launches = 0;
    uint64_t sync_epoch = 1;        // counts full synchronisations of the stream (mlc_pass_flush): work enqueued in an earlier epoch is done
    uint64_t allocations = 0;       // device and pinned-host allocations made through this context
    uint64_t decode_launches = 0;   // selects the workspace copy of the split-KV kernel
    mlcb::PoolWrites recent_writes[2];   // pools written by the last two decode launches on this context
    void* pass_args = nullptr;           // parameter block of the whole-pass decode launch (attn_decode_tma.cu)
    uint64_t ext_launches = 0;      // same for launches on caller-provided (fixed) scratch
    uint32_t* ext_counter_block[2] = {nullptr, nullptr};  // arrival counters inside that scratch, once used
    std::string last_error;
    std::unordered_map<const void*, size_t> allocs;
    std::unordered_map<std::string, std::pair<void*, size_t>> cached;
    std::vector<mlcb::StageChunk> stage;
    uint32_t* d_err = nullptr;  // device error word
    uint32_t* h_err = nullptr;  // pinned copy, filled by an async copy in front of the flush's synchronisation
    // split-KV workspace (partials + arrival counters), grown on demand
    void* d_work = nullptr;
    size_t work_bytes = 0;
    uint32_t* d_counters = nullptr;
    size_t n_counters = 0;
    size_t decode_smem_set[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};  // dynamic-smem opt-in already applied, per kernel variant
    bool prefill_smem_set = false;             // same, for the chunked-prefill kernel
    // copy streams and events of the host-buffer decode pass (created on first use)
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
    std::vector<cudaEvent_t> pass_events;
    cudaEvent_t host_pass_done = nullptr;   // last copy back of the most recent host-buffer pass, while not yet waited for
    // optional per-warp phase stamps of the last decode launch (env MLC_B200_TRACE=1)
    unsigned long long* d_trace = nullptr;
    size_t trace_words = 0;
    uint32_t trace_ctas = 0;
    uint32_t trace_parity = 0;  // which half of d_trace the most recent launch wrote
    mlcb::AttnPlanCache* plan_cache = nullptr;
    mlcb::TensorMapCache* tmap_cache = nullptr;
    void* tmap_encode_fn = nullptr;  // cuTensorMapEncodeTiled, resolved through the runtime

    int fail(int status, const char* fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof(buf), fmt, ap);
        va_end(ap);
        last_error = buf;
        return status;
    }
};

namespace mlcb {

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

#define MLCB_CUDA(ctx, expr)                                                              \
    do {                                                                                  \
        cudaError_t _e = (expr);                                                          \
        if (_e != cudaSuccess)                                                            \
            return (ctx)->fail(MLC_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// Copies `bytes` of host memory into the staging area and enqueues the H2D copy
// on the context's stream; returns the device address (256-byte aligned) or null.
void* stage_to_device(mlc_ctx* ctx, const void* host, size_t bytes);
// Reserves a staging region and returns both addresses; the caller fills `*host`
// and then calls stage_commit for the same region.
bool stage_reserve(mlc_ctx* ctx, size_t bytes, void** host, void** dev);
bool stage_commit(mlc_ctx* ctx, void* host, void* dev, size_t bytes);
void stage_reset(mlc_ctx* ctx);
// After a kernel reported an error word: clears the word and re-zeroes the split-KV arrival
// counters, which a launch that gave up may have left half counted. The stream is idle here.
void reset_after_device_error(mlc_ctx* ctx);
// Grows the split-KV workspace / counters (synchronises when it has to reallocate).
int ensure_workspace(mlc_ctx* ctx, size_t bytes, size_t counters);
// Number of pages a pool pointer can hold given the caller's claim (0 = unknown)
// and the context's own allocation registry.
size_t resolve_capacity(const mlc_ctx* ctx, const void* pool, size_t claimed, size_t page_bytes);
void destroy_plan_cache(mlc_ctx* ctx);
void destroy_tmap_cache(mlc_ctx* ctx);
void destroy_pass_args(mlc_ctx* ctx);
}  // namespace mlcb
struct mlc_exchange;
namespace mlcb {
bool exchange_describe(const mlc_exchange* ex, ExchangeView* v);

}  // namespace mlcb
