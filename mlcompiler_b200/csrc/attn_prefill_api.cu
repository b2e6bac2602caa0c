// Entry points of chunked (multi-token) causal paged attention.
//
// The reference runs a paged prefill as q_len single-token decode passes
// (compiler/runtime/batched_executor.cpp:450-467); query i of request r sits at position
// q_start[r] + i and attends to kv_pos <= q_start[r] + i (mask rule metal_runtime.mm:2286),
// which is also what its CPU backend computes for seq_len > 1
// (compiler/runtime/operator_backend.cpp:906-968). These entry points compute all query
// tokens of all requests in one launch. The new tokens' K/V rows must already be in the
// pages (scatter first), as in the reference's order scatter -> attention
// (compiler/runtime/batched_walker.cpp:299-331).
#include <cstring>
#include <vector>

#include "attn_internal.hpp"

using namespace mlcb;

namespace {

int prefill_impl(mlc_ctx* ctx, bool sync, const void* q, const void* k_pages, const void* v_pages, void* o,
                 const uint32_t* pt_flat, size_t n_flat, const uint32_t* pt_off, const uint32_t* seq_lens,
                 const uint32_t* q_start, const uint32_t* q_len, size_t batch, size_t H, size_t KVH, size_t D,
                 size_t P, float scale, int q_dtype, int o_dtype, size_t capacity_pages) {
    if (!ctx) return MLC_ERR_INVALID_ARG;
    if (!q || !k_pages || !v_pages || !o) return ctx->fail(MLC_ERR_INVALID_ARG, "null buffer");
    if (!pt_off || !seq_lens || !q_start || !q_len || (!pt_flat && n_flat)) return ctx->fail(MLC_ERR_INVALID_ARG, "null table");
    if (batch == 0 || H == 0 || D == 0 || P == 0) return ctx->fail(MLC_ERR_INVALID_ARG, "zero dimension");
    if (KVH == 0 || H % KVH != 0) return ctx->fail(MLC_ERR_INVALID_ARG, "num_heads must be a multiple of kv_heads");
    if (D > 256) return ctx->fail(MLC_ERR_UNSUPPORTED, "head_dim > 256");
    if ((q_dtype != MLC_F16 && q_dtype != MLC_F32) || (o_dtype != MLC_F16 && o_dtype != MLC_F32))
        return ctx->fail(MLC_ERR_INVALID_ARG, "q / o dtype must be MLC_F16 or MLC_F32");
    if (!sync && !ctx->pass_open) return ctx->fail(MLC_ERR_NO_OPEN_PASS, "encode without an open pass");
    if (ctx->capturing) return ctx->fail(MLC_ERR_UNSUPPORTED, "host tables inside a graph capture");
    if (n_flat < pt_off[batch]) return ctx->fail(MLC_ERR_INVALID_ARG, "page_tables_flat shorter than the last offset");
    const size_t capacity = resolve_capacity(ctx, k_pages, capacity_pages, P * KVH * D * 2);
    size_t total_q = 0, max_q = 0;
    for (size_t r = 0; r < batch; ++r) {
        if (pt_off[r + 1] < pt_off[r]) return ctx->fail(MLC_ERR_BOUNDS, "page_table_offsets not monotone at %zu", r);
        const uint64_t room = static_cast<uint64_t>(pt_off[r + 1] - pt_off[r]) * P;
        if (seq_lens[r] > room)
            return ctx->fail(MLC_ERR_BOUNDS, "seq_lens[%zu]=%u exceeds its %u pages", r, seq_lens[r], pt_off[r + 1] - pt_off[r]);
        if (static_cast<uint64_t>(q_start[r]) + q_len[r] > seq_lens[r])
            return ctx->fail(MLC_ERR_BOUNDS, "q_start[%zu] + q_len[%zu] = %llu exceeds seq_lens = %u", r, r,
                             static_cast<unsigned long long>(q_start[r]) + q_len[r], seq_lens[r]);
        total_q += q_len[r];
        if (q_len[r] > max_q) max_q = q_len[r];
    }
    if (total_q == 0) return MLC_OK;
    if (total_q * H >= (size_t(1) << 31)) return ctx->fail(MLC_ERR_UNSUPPORTED, "query tokens * heads too large");
    if (capacity)
        for (size_t i = 0; i < pt_off[batch]; ++i)
            if (pt_flat[i] >= capacity)
                return ctx->fail(MLC_ERR_BOUNDS, "page_tables_flat[%zu]=%u >= capacity %zu", i, pt_flat[i], capacity);
    DeviceGuard guard(ctx->device);
    if (scale == 0.f) scale = 1.0f / std::sqrt(static_cast<float>(D));

    const size_t nf = pt_off[batch];
    const bool tc = q_dtype == MLC_F16 && o_dtype == MLC_F16 && prefill_tcgen05_supported(H, KVH, D, P, capacity) &&
                    (reinterpret_cast<uintptr_t>(q) % 16 == 0) && (reinterpret_cast<uintptr_t>(o) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(k_pages) % 128 == 0) && (reinterpret_cast<uintptr_t>(v_pages) % 128 == 0) &&
                    scale > 0.f && !ctx->force_general;  // the kernel orders raw scores: needs scale > 0
    int st;
    if (tc) {
        // one staging region: pt_flat | pt_off | seq_lens | q_start | q_len | q_row0
        const size_t words = nf + (batch + 1) + 4 * batch;
        void *h = nullptr, *d = nullptr;
        if (!stage_reserve(ctx, words * 4, &h, &d)) return ctx->fail(MLC_ERR_OOM, "staging area exhausted");
        uint32_t* w = static_cast<uint32_t*>(h);
        if (nf) std::memcpy(w, pt_flat, nf * 4);
        std::memcpy(w + nf, pt_off, (batch + 1) * 4);
        std::memcpy(w + nf + batch + 1, seq_lens, batch * 4);
        std::memcpy(w + nf + 2 * batch + 1, q_start, batch * 4);
        std::memcpy(w + nf + 3 * batch + 1, q_len, batch * 4);
        uint32_t row = 0;
        for (size_t r = 0; r < batch; ++r) {
            w[nf + 4 * batch + 1 + r] = row;
            row += q_len[r];
        }
        if (!stage_commit(ctx, h, d, words * 4)) return ctx->fail(MLC_ERR_CUDA, "table upload failed");
        const uint32_t* dw = static_cast<const uint32_t*>(d);
        st = launch_prefill_tcgen05(ctx, q, k_pages, v_pages, o, dw, dw + nf, dw + nf + batch + 1, dw + nf + 2 * batch + 1,
                                    dw + nf + 3 * batch + 1, dw + nf + 4 * batch + 1, batch, total_q, max_q, H, KVH,
                                    capacity, scale);
        if (st == MLC_OK) ctx->last_attention_kernel = 3;
    } else {
        // Any other shape / dtype: every query token becomes one row of the any-shape decode
        // kernel, sharing its request's page table and attending to q_start + i + 1 tokens.
        const size_t words = nf + 2 * total_q;
        void *h = nullptr, *d = nullptr;
        if (!stage_reserve(ctx, words * 4, &h, &d)) return ctx->fail(MLC_ERR_OOM, "staging area exhausted");
        uint32_t* w = static_cast<uint32_t*>(h);
        if (nf) std::memcpy(w, pt_flat, nf * 4);
        size_t t = 0;
        for (size_t r = 0; r < batch; ++r)
            for (uint32_t i = 0; i < q_len[r]; ++i, ++t) {
                w[nf + t] = pt_off[r];
                const uint32_t see = q_start[r] + i + 1;
                w[nf + total_q + t] = see < seq_lens[r] ? see : seq_lens[r];
            }
        if (!stage_commit(ctx, h, d, words * 4)) return ctx->fail(MLC_ERR_CUDA, "table upload failed");
        const uint32_t* dw = static_cast<const uint32_t*>(d);
        AttnArgs a;
        a.q = q; a.k_pages = k_pages; a.v_pages = v_pages; a.o = o;
        a.batch = total_q; a.H = H; a.KVH = KVH; a.D = D; a.P = P;
        a.capacity = capacity; a.scale = scale; a.q_dtype = q_dtype; a.o_dtype = o_dtype;
        st = launch_attention_general(ctx, a, dw, dw + nf, dw + nf + total_q);
        if (st == MLC_OK) ctx->last_attention_kernel = 1;
    }
    if (st != MLC_OK) return st;
    if (sync) {
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (!ctx->pass_open) stage_reset(ctx);
        if (e != cudaSuccess) return ctx->fail(MLC_ERR_CUDA, "prefill attention failed: %s", cudaGetErrorString(e));
        uint32_t word = 0;
        MLCB_CUDA(ctx, cudaMemcpy(&word, ctx->d_err, 4, cudaMemcpyDeviceToHost));
        if (word) {
            reset_after_device_error(ctx);
            return ctx->fail(MLC_ERR_DEVICE_FLAG, "prefill attention recorded error word 0x%x", word);
        }
    }
    return MLC_OK;
}

}  // namespace

extern "C" {

int mlc_run_paged_prefill_attention(mlc_ctx* ctx, const void* q, const void* k_pages, const void* v_pages, void* o,
                                    const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                                    const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                                    const uint32_t* q_start, const uint32_t* q_len, size_t batch, size_t num_heads,
                                    size_t kv_heads, size_t head_dim, size_t page_size, float scale, int q_dtype,
                                    int o_dtype, size_t capacity_pages) {
    return prefill_impl(ctx, true, q, k_pages, v_pages, o, page_tables_flat, n_page_tables_flat, page_table_offsets,
                        seq_lens, q_start, q_len, batch, num_heads, kv_heads, head_dim, page_size, scale, q_dtype,
                        o_dtype, capacity_pages);
}

int mlc_encode_paged_prefill_attention(mlc_ctx* ctx, const void* q, const void* k_pages, const void* v_pages, void* o,
                                       const uint32_t* page_tables_flat, size_t n_page_tables_flat,
                                       const uint32_t* page_table_offsets, const uint32_t* seq_lens,
                                       const uint32_t* q_start, const uint32_t* q_len, size_t batch, size_t num_heads,
                                       size_t kv_heads, size_t head_dim, size_t page_size, float scale, int q_dtype,
                                       int o_dtype, size_t capacity_pages) {
    return prefill_impl(ctx, false, q, k_pages, v_pages, o, page_tables_flat, n_page_tables_flat, page_table_offsets,
                        seq_lens, q_start, q_len, batch, num_heads, kv_heads, head_dim, page_size, scale, q_dtype,
                        o_dtype, capacity_pages);
}

}  // extern "C"
