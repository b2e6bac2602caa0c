// Planned decode attention that allocates nothing: its split-KV scratch is a
// fixed array compiled into the library.
//
// No counterpart in the reference (its kernel never splits a sequence, so it has no
// scratch at all). This entry point exists for callers that must not allocate
// device memory at call time - a serving loop that has handed the whole GPU to its
// own memory pool, so that a later cudaMalloc would fail or fragment it; or a
// latency-critical decode loop that cannot afford the device-wide synchronisation
// cudaMalloc / cudaFree imply. The regular entry points grow a per-context
// workspace on demand; this one never does.
#include "attn_internal.hpp"

namespace mlcb {

// 8 MiB per GPU, held from library load until exit by every GPU that loads the library.
// Used as two 4 MiB halves by alternate launches (see launch_attention_decode_tma).
static constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// Device addresses of the array, one per device ordinal. In host code the array's
// name is only a handle for cudaGetSymbolAddress, never a device pointer.
static constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices] = {};

static int static_scratch_address(mlc_ctx* ctx, void** out) {
    const int dev = ctx->device;
    if (dev < 0 || dev >= kMaxDevices) return ctx->fail(MLC_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!g_scratch_addr[dev]) {
        // once per device, with that device current (the caller holds a DeviceGuard)
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
        if (e != cudaSuccess || !p)
            return ctx->fail(MLC_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return MLC_OK;
}

}  // namespace mlcb

using namespace mlcb;

extern "C" {

size_t mlc_static_scratch_bytes(void) { return kStaticScratchBytes; }

int mlc_encode_paged_flash_attention_planned_static(mlc_ctx* ctx, const mlc_attn_plan* plan, const void* q,
                                                    const void* k_pages, const void* v_pages, void* o,
                                                    float scale, int q_dtype, int o_dtype) {
    if (!ctx || !plan) return MLC_ERR_INVALID_ARG;
    if (!ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    DeviceGuard guard(ctx->device);
    if (int ust = mlcb::use_plan(ctx, plan); ust != MLC_OK) return ust;
    void* scratch = nullptr;
    int st = static_scratch_address(ctx, &scratch);
    if (st != MLC_OK) return st;
    AttnArgs a;
    a.q = q; a.k_pages = k_pages; a.v_pages = v_pages; a.o = o;
    a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = o_dtype;
    a.ext_work = scratch;
    a.ext_work_bytes = kStaticScratchBytes;
    return launch_attention_with_plan(ctx, a, plan);
}

}  // extern "C"
