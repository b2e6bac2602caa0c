// Paged KV writers and readers (pure byte movement, bit-exact).
//
// CUDA counterparts of the reference's MSL kernels
//   scatter_kv_paged_batched_f16   compiler/runtime/metal_runtime.mm:405-424
//   scatter_kv_paged_f16 / _f32    compiler/runtime/metal_runtime.mm:468-512
//   gather_kv_pages_f16 / _f32     compiler/runtime/metal_runtime.mm:328-370
// and of their host wrappers (metal_runtime.mm:7168-7294, 7647-7721, 7828-7906).
//
// The reference moves one 2- or 4-byte element per thread with 32-bit index
// arithmetic. Here every thread moves one 16-byte vector when the row geometry
// allows it (head_dim * dtype_bytes a multiple of 16 and 16-byte aligned
// buffers - true for every shape the pools are used with) and offsets are
// 64-bit; an element-wise kernel covers everything else. Page ids and slots are
// checked on the host when the pool capacity is known and again in the kernel,
// which records an error word and skips the access instead of faulting.
#include "attn_internal.hpp"

namespace mlcb {

template <typename Vec>
__global__ void scatter_rows_batched_kernel(const Vec* __restrict__ k_src, Vec* __restrict__ k_pool,
                                            const Vec* __restrict__ v_src, Vec* __restrict__ v_pool,
                                            const uint32_t* __restrict__ page_ids,
                                            const uint32_t* __restrict__ slots,
                                            uint32_t vec_per_row,      // KVH*D*2 / sizeof(Vec)
                                            uint32_t page_size, uint32_t batch, uint32_t capacity,
                                            uint32_t* __restrict__ err) {
    const Vec* src = blockIdx.y == 0 ? k_src : v_src;
    Vec* pool = blockIdx.y == 0 ? k_pool : v_pool;
    uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t total = batch * vec_per_row;
    if (gid >= total) return;
    uint32_t req = gid / vec_per_row;
    uint32_t v = gid - req * vec_per_row;
    uint32_t page = page_ids[req], slot = slots[req];
    if (page >= capacity) { atomicOr(err, MLC_DEVERR_BAD_PAGE); return; }
    if (slot >= page_size) { atomicOr(err, MLC_DEVERR_BAD_SLOT); return; }
    size_t dst = (static_cast<size_t>(page) * page_size + slot) * vec_per_row + v;
    pool[dst] = src[gid];
}

// Multi-token scatter (to_pool = true) or gather (to_pool = false) of one
// request. Contiguous side: [KVH, tokens, D]; vec_per_head = D*dtype/sizeof(Vec).
template <typename Vec, bool to_pool>
__global__ void paged_tokens_kernel(Vec* __restrict__ pool, Vec* __restrict__ flat,
                                    const uint32_t* __restrict__ page_table, uint32_t vec_per_head,
                                    uint32_t kv_heads, uint32_t page_size, uint32_t tokens,
                                    uint32_t start_slot, uint32_t capacity,
                                    uint32_t* __restrict__ err) {
    size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    size_t total = static_cast<size_t>(kv_heads) * tokens * vec_per_head;
    if (gid >= total) return;
    uint32_t v = gid % vec_per_head;
    size_t tmp = gid / vec_per_head;
    uint32_t token = tmp % tokens;
    uint32_t kv = tmp / tokens;
    uint32_t abs_slot = start_slot + token;
    uint32_t page = page_table[abs_slot / page_size];
    uint32_t slot = abs_slot % page_size;
    if (page >= capacity) { atomicOr(err, MLC_DEVERR_BAD_PAGE); return; }
    size_t p = ((static_cast<size_t>(page) * page_size + slot) * kv_heads + kv) * vec_per_head + v;
    if (to_pool) pool[p] = flat[gid];
    else flat[gid] = pool[p];
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int launch_scatter_rows_device_tables(mlc_ctx* ctx, void* k_pool, void* v_pool, const uint32_t* d_ids,
                                      const uint32_t* d_slots, size_t P, size_t KVH, size_t D,
                                      size_t batch, const void* k_src, const void* v_src, size_t capacity) {
    const size_t row_bytes = KVH * D * 2;
    const uint32_t cap32 = capacity ? static_cast<uint32_t>(capacity) : 0xFFFFFFFFu;
    bool vec = row_bytes % 16 == 0 && aligned16(k_pool) && aligned16(k_src) &&
               (!v_pool || (aligned16(v_pool) && aligned16(v_src)));
    dim3 grid(1, v_pool ? 2 : 1);
    const int threads = 256;
    if (vec) {
        uint32_t vpr = static_cast<uint32_t>(row_bytes / 16);
        grid.x = static_cast<unsigned>((batch * vpr + threads - 1) / threads);
        scatter_rows_batched_kernel<uint4><<<grid, threads, 0, ctx->stream>>>(
            static_cast<const uint4*>(k_src), static_cast<uint4*>(k_pool),
            static_cast<const uint4*>(v_src), static_cast<uint4*>(v_pool), d_ids, d_slots, vpr,
            static_cast<uint32_t>(P), static_cast<uint32_t>(batch), cap32, ctx->d_err);
    } else {
        uint32_t vpr = static_cast<uint32_t>(row_bytes / 2);
        grid.x = static_cast<unsigned>((batch * vpr + threads - 1) / threads);
        scatter_rows_batched_kernel<uint16_t><<<grid, threads, 0, ctx->stream>>>(
            static_cast<const uint16_t*>(k_src), static_cast<uint16_t*>(k_pool),
            static_cast<const uint16_t*>(v_src), static_cast<uint16_t*>(v_pool), d_ids, d_slots, vpr,
            static_cast<uint32_t>(P), static_cast<uint32_t>(batch), cap32, ctx->d_err);
    }
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    return MLC_OK;
}

static int scatter_batched_impl(mlc_ctx* ctx, bool sync, void* k_pool, void* v_pool,
                                const uint32_t* page_ids, const uint32_t* slots, size_t P,
                                size_t KVH, size_t D, size_t batch, const void* k_src,
                                const void* v_src, size_t capacity_pages) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    // metal_runtime.mm:7241-7243 (sync form); the encode form has no checks in the
    // reference beyond the open pass, the same rules are applied to both here.
    if (!k_pool || !k_src || !page_ids || !slots) return ctx->fail(MLC_ERR_INVALID_ARG, "null argument");
    if ((v_pool == nullptr) != (v_src == nullptr)) return ctx->fail(MLC_ERR_INVALID_ARG, "V pool/src mismatch");
    if (batch == 0 || KVH == 0 || D == 0 || P == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (!sync && !ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (batch * KVH * D >= (size_t(1) << 32)) return ctx->fail(MLC_ERR_UNSUPPORTED, "batch too large");
    if (ctx->capturing)
        return ctx->fail(MLC_ERR_UNSUPPORTED, "host page ids inside a graph capture: use the planned scatter");
    DeviceGuard guard(ctx->device);
    size_t row_bytes = KVH * D * 2;
    size_t cap = resolve_capacity(ctx, k_pool, capacity_pages, P * row_bytes);
    for (size_t r = 0; r < batch; ++r) {
        if (cap && page_ids[r] >= cap)
            return ctx->fail(MLC_ERR_BOUNDS, "page_ids[%zu]=%u >= capacity %zu", r, page_ids[r], cap);
        if (slots[r] >= P)
            return ctx->fail(MLC_ERR_BOUNDS, "slots_in_page[%zu]=%u >= page size %zu", r, slots[r], P);
    }
    // one staging region: ids then slots
    void *h = nullptr, *d = nullptr;
    if (!stage_reserve(ctx, batch * 8, &h, &d)) return MLC_ERR_OOM;
    memcpy(h, page_ids, batch * 4);
    memcpy(static_cast<char*>(h) + batch * 4, slots, batch * 4);
    if (!stage_commit(ctx, h, d, batch * 8)) return MLC_ERR_CUDA;
    const uint32_t* d_ids = static_cast<const uint32_t*>(d);
    const uint32_t* d_slots = d_ids + batch;

    int st = launch_scatter_rows_device_tables(ctx, k_pool, v_pool, d_ids, d_slots, P, KVH, D, batch, k_src,
                                               v_src, cap);
    if (st != MLC_OK) return st;
    if (sync) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (!ctx->pass_open) stage_reset(ctx);
        if (e != cudaSuccess) return ctx->fail(MLC_ERR_CUDA, "scatter failed: %s", cudaGetErrorString(e));
    }
    return MLC_OK;
}

template <bool to_pool>
static int paged_tokens_impl(mlc_ctx* ctx, void* pool, const uint32_t* page_table, size_t n_pt,
                             size_t P, size_t KVH, size_t D, size_t tokens, size_t start_slot,
                             void* flat, size_t dtype_bytes, size_t capacity_pages) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    // metal_runtime.mm:7838-7850 (scatter) and 7656-7667 (gather)
    if (!pool || !flat || !page_table) return ctx->fail(MLC_ERR_INVALID_ARG, "null argument");
    if (P == 0 || KVH == 0 || D == 0 || tokens == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (dtype_bytes != 2 && dtype_bytes != 4) return ctx->fail(MLC_ERR_INVALID_ARG, "dtype_bytes must be 2 or 4");
    if (start_slot >= P) return ctx->fail(MLC_ERR_INVALID_ARG, "start_slot >= page size");
    size_t pages_needed = (start_slot + tokens + P - 1) / P;
    if (n_pt < pages_needed) return ctx->fail(MLC_ERR_INVALID_ARG, "page table covers %zu pages, %zu needed", n_pt, pages_needed);
    if (start_slot + tokens >= (size_t(1) << 32)) return ctx->fail(MLC_ERR_UNSUPPORTED, "too many tokens");
    DeviceGuard guard(ctx->device);
    size_t cap = resolve_capacity(ctx, pool, capacity_pages, P * KVH * D * dtype_bytes);
    if (cap)
        for (size_t i = 0; i < pages_needed; ++i)
            if (page_table[i] >= cap)
                return ctx->fail(MLC_ERR_BOUNDS, "page_table[%zu]=%u >= capacity %zu", i, page_table[i], cap);
    uint32_t cap32 = cap ? static_cast<uint32_t>(cap) : 0xFFFFFFFFu;
    const uint32_t* d_pt = static_cast<const uint32_t*>(stage_to_device(ctx, page_table, pages_needed * 4));
    if (!d_pt) return MLC_ERR_OOM;
    size_t head_bytes = D * dtype_bytes;
    const int threads = 256;
    bool vec = head_bytes % 16 == 0 && aligned16(pool) && aligned16(flat);
    if (vec) {
        uint32_t vph = static_cast<uint32_t>(head_bytes / 16);
        size_t total = KVH * tokens * vph;
        paged_tokens_kernel<uint4, to_pool><<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, ctx->stream>>>(
            static_cast<uint4*>(pool), static_cast<uint4*>(flat), d_pt, vph, static_cast<uint32_t>(KVH),
            static_cast<uint32_t>(P), static_cast<uint32_t>(tokens), static_cast<uint32_t>(start_slot), cap32, ctx->d_err);
    } else if (dtype_bytes == 4) {
        size_t total = KVH * tokens * D;
        paged_tokens_kernel<uint32_t, to_pool><<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, ctx->stream>>>(
            static_cast<uint32_t*>(pool), static_cast<uint32_t*>(flat), d_pt, static_cast<uint32_t>(D), static_cast<uint32_t>(KVH),
            static_cast<uint32_t>(P), static_cast<uint32_t>(tokens), static_cast<uint32_t>(start_slot), cap32, ctx->d_err);
    } else {
        size_t total = KVH * tokens * D;
        paged_tokens_kernel<uint16_t, to_pool><<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, ctx->stream>>>(
            static_cast<uint16_t*>(pool), static_cast<uint16_t*>(flat), d_pt, static_cast<uint32_t>(D), static_cast<uint32_t>(KVH),
            static_cast<uint32_t>(P), static_cast<uint32_t>(tokens), static_cast<uint32_t>(start_slot), cap32, ctx->d_err);
    }
    ++ctx->launches;
    MLCB_CUDA(ctx, cudaGetLastError());
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (!ctx->pass_open) stage_reset(ctx);
    if (e != cudaSuccess) return ctx->fail(MLC_ERR_CUDA, "paged copy failed: %s", cudaGetErrorString(e));
    return MLC_OK;
}

}  // namespace mlcb

using namespace mlcb;

extern "C" {

int mlc_run_scatter_kv_paged_batched_f16(mlc_ctx* ctx, void* page_storage, const uint32_t* page_ids,
                                         const uint32_t* slots_in_page, size_t page_size_tokens,
                                         size_t n_kv_heads, size_t head_dim, size_t batch,
                                         const void* src, size_t capacity_pages) {
    return scatter_batched_impl(ctx, true, page_storage, nullptr, page_ids, slots_in_page,
                                page_size_tokens, n_kv_heads, head_dim, batch, src, nullptr,
                                capacity_pages);
}

int mlc_encode_scatter_kv_paged_batched_f16(mlc_ctx* ctx, void* page_storage,
                                            const uint32_t* page_ids, const uint32_t* slots_in_page,
                                            size_t page_size_tokens, size_t n_kv_heads,
                                            size_t head_dim, size_t batch, const void* src,
                                            size_t capacity_pages) {
    return scatter_batched_impl(ctx, false, page_storage, nullptr, page_ids, slots_in_page,
                                page_size_tokens, n_kv_heads, head_dim, batch, src, nullptr,
                                capacity_pages);
}

int mlc_encode_scatter_kv_pair_paged_batched_f16(mlc_ctx* ctx, void* k_page_storage,
                                                 void* v_page_storage, const uint32_t* page_ids,
                                                 const uint32_t* slots_in_page,
                                                 size_t page_size_tokens, size_t n_kv_heads,
                                                 size_t head_dim, size_t batch, const void* k_src,
                                                 const void* v_src, size_t capacity_pages) {
    if (ctx && (!v_page_storage || !v_src)) return ctx->fail(MLC_ERR_INVALID_ARG, "null argument");
    return scatter_batched_impl(ctx, false, k_page_storage, v_page_storage, page_ids, slots_in_page,
                                page_size_tokens, n_kv_heads, head_dim, batch, k_src, v_src,
                                capacity_pages);
}

int mlc_run_scatter_kv_paged(mlc_ctx* ctx, void* page_storage, const uint32_t* page_table,
                             size_t n_page_table, size_t page_size_tokens, size_t n_kv_heads,
                             size_t head_dim, size_t tokens, size_t start_slot, const void* src,
                             size_t dtype_bytes, size_t capacity_pages) {
    return paged_tokens_impl<true>(ctx, page_storage, page_table, n_page_table, page_size_tokens,
                                   n_kv_heads, head_dim, tokens, start_slot,
                                   const_cast<void*>(src), dtype_bytes, capacity_pages);
}

int mlc_run_gather_kv_pages(mlc_ctx* ctx, const void* page_storage, const uint32_t* page_table,
                            size_t n_page_table, size_t page_size_tokens, size_t n_kv_heads,
                            size_t head_dim, size_t num_tokens, void* dst, size_t dtype_bytes,
                            size_t capacity_pages) {
    return paged_tokens_impl<false>(ctx, const_cast<void*>(page_storage), page_table, n_page_table,
                                    page_size_tokens, n_kv_heads, head_dim, num_tokens, 0, dst,
                                    dtype_bytes, capacity_pages);
}

}  // extern "C"
