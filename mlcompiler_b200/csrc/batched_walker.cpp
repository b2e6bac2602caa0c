// See batched_walker.hpp.
#include "batched_walker.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include "attn_internal.hpp"
#include "ctx.hpp"

namespace mlcb {
namespace runtime {

BatchedWalker::~BatchedWalker() {
    if (logits_pinned_) cudaFreeHost(logits_pinned_);
    if (tokens_pinned_) cudaFreeHost(tokens_pinned_);
}

// NVTX range for the lifetime of the object: a pass, and inside a model pass every layer, show up by name in a
// timeline tool (where the reference prints its MLC_BATCHED_PROFILE table, batched_walker.cpp:100-125). Without a
// tool attached the calls do nothing.
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

// MLC_B200_WALKER_TRACE=1 in the environment: one line per model pass on stderr with the host time of its phases.
static bool walker_trace() {
    static const bool on = [] {
        const char* e = std::getenv("MLC_B200_WALKER_TRACE");
        return e && e[0] == '1';
    }();
    return on;
}
static double now_us() {
    return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

BatchedDecodeOutput BatchedWalker::step(const std::vector<RequestSlot>& slots, const LogitsSink* sink,
                                        std::vector<uint64_t>* greedy) {
    BatchedDecodeOutput out;
    if (slots.empty()) return out;
    NvtxRange pass_range("mlc decode pass");
    const double t_start = walker_trace() ? now_us() : 0.0;
    PagedAttentionExecutor& ex = exec_;
    mlc_ctx* ctx = ex.ctx_;
    PagedKVStorage* storage = ex.storage_;
    const size_t N = slots.size();
    const uint32_t H = ex.H_, KVH = ex.KVH_, D = ex.D_, P = storage->page_size_tokens();
    auto fail_all = [&]() {
        out.per_request.clear();
        for (const auto& s : slots) {
            BatchedDecodeOutput::PerRequest p;
            p.request_id = s.request_id;
            out.per_request.push_back(std::move(p));
        }
        return out;
    };

    // One new token per request: extend the page tables. If the pool runs out, every slot of
    // the pass is reported failed and the requests extended so far keep their extension,
    // exactly as in the reference (batched_walker.cpp:127-149).
    std::vector<PagedAttentionExecutor::PerRequest*> reqs(N, nullptr);
    std::vector<uint32_t> page_ids(N), slot_ids(N);
    for (size_t r = 0; r < N; ++r) {
        reqs[r] = &ex.ensure_request(slots[r].request_id);
        if (!reqs[r]->page_state) {
            reqs[r]->page_state.reset(new RequestKVState());
            reqs[r]->page_state->request_id = slots[r].request_id;
            reqs[r]->page_state->page_size_tokens = ex.page_size_tokens_;
        }
        auto loc = reqs[r]->page_state->extend_one_token(*ex.pool_);
        if (!loc) return fail_all();
        page_ids[r] = loc->first;
        slot_ids[r] = loc->second;
    }

    // Tables of the pass, built once (the reference rebuilds them per layer, 316-325):
    // seq_lens count the new token, q_pos is the new token's own position.
    std::vector<uint32_t> pt_flat, pt_off(N + 1, 0), seq_lens(N), q_pos(N);
    for (size_t r = 0; r < N; ++r) {
        pt_off[r] = static_cast<uint32_t>(pt_flat.size());
        const auto& table = reqs[r]->page_state->page_table;
        pt_flat.insert(pt_flat.end(), table.begin(), table.end());
        seq_lens[r] = static_cast<uint32_t>(reqs[r]->page_state->total_tokens());
        q_pos[r] = static_cast<uint32_t>(slots[r].sequence_position);
    }
    pt_off[N] = static_cast<uint32_t>(pt_flat.size());

    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    const size_t cap = storage->capacity_pages();
    const bool fused = ex.order_ == PagedAttentionExecutor::CallOrder::Fused;
    // Two plans that live as long as the executor, used by alternate passes and refreshed in place with the
    // pass's tables: after the first two passes a decode pass allocates nothing (while the batch does not
    // outgrow the plans' buffers), where creating and destroying a plan per pass cost a cudaMalloc /
    // cudaFree pair and pinned allocations every time.
    mlc_attn_plan* plan = nullptr;
    if (fused) {
        mlc_attn_plan*& slot = ex.plans_[ex.passes_++ & 1u];
        const int st = slot ? mlc_attn_plan_update(ctx, slot, pt_flat.data(), pt_flat.size(), pt_off.data(), seq_lens.data(),
                                                   q_pos.data(), page_ids.data(), slot_ids.data(), N)
                            : mlc_attn_plan_create(ctx, pt_flat.data(), pt_flat.size(), pt_off.data(), seq_lens.data(),
                                                   q_pos.data(), page_ids.data(), slot_ids.data(), N, H, KVH, D, P, 1, cap,
                                                   &slot);
        if (st != MLC_OK) return fail_all();
        plan = slot;
    }

    if (ex.model_) {
        // The whole walker step on the device; logits [N, vocab] come back (batched_walker.cpp:461-475).
        // A caller's buffer in page-locked memory takes the rows straight from the device; anything else goes
        // through this walker's page-locked landing area (a copy into pageable memory is several times slower).
        const size_t vocab = ex.model_->vocab_size;
        bool direct = false;
        if (sink && sink->dst && sink->stride >= vocab) {
            cudaPointerAttributes attr{};
            direct = cudaPointerGetAttributes(&attr, sink->dst) == cudaSuccess && attr.type == cudaMemoryTypeHost;
            cudaGetLastError();   // a pointer the runtime does not know is not an error here
        }
        if (greedy && tokens_pinned_count_ < N) {
            if (tokens_pinned_) cudaFreeHost(tokens_pinned_);
            tokens_pinned_ = nullptr;
            tokens_pinned_count_ = 0;
            DeviceGuard guard(ctx->device);
            if (cudaHostAlloc(reinterpret_cast<void**>(&tokens_pinned_), std::max<size_t>(N, 64) * sizeof(uint32_t),
                              cudaHostAllocDefault) != cudaSuccess)
                return fail_all();
            tokens_pinned_count_ = std::max<size_t>(N, 64);
            ++ctx->allocations;
        }
        if (!greedy && !direct && logits_pinned_floats_ < N * vocab) {
            if (logits_pinned_) cudaFreeHost(logits_pinned_);
            logits_pinned_ = nullptr;
            logits_pinned_floats_ = 0;
            DeviceGuard guard(ctx->device);
            if (cudaHostAlloc(reinterpret_cast<void**>(&logits_pinned_), N * vocab * sizeof(float), cudaHostAllocDefault) !=
                cudaSuccess)
                return fail_all();
            logits_pinned_floats_ = N * vocab;
            ++ctx->allocations;
        }
        const double t_plan = walker_trace() ? now_us() : 0.0;
        bool ok = mlc_pass_begin(ctx) == MLC_OK;
        ok = ok && encode_model_pass(slots, plan, page_ids, slot_ids, pt_flat, pt_off, seq_lens, q_pos,
                                     direct ? sink->dst : logits_pinned_, direct ? sink->stride : vocab, 0,
                                     true,   // a decode pass writes one row per request, at the plan's (page, slot)
                                     greedy ? tokens_pinned_ : nullptr);
        const double t_enc = walker_trace() ? now_us() : 0.0;
        ok = (mlc_pass_flush(ctx) == MLC_OK) && ok;   // the logits are on the host when this returns
        const double t_flush = walker_trace() ? now_us() : 0.0;
        if (!ok) return fail_all();
        if (greedy) {
            greedy->assign(tokens_pinned_, tokens_pinned_ + N);
        } else if (!direct && sink && sink->dst && sink->stride >= vocab) {
            for (size_t r = 0; r < N; ++r)
                std::memcpy(sink->dst + r * sink->stride, logits_pinned_ + r * vocab, vocab * sizeof(float));
        }
        const bool to_sink = sink && sink->dst && sink->stride >= vocab;
        out.per_request.reserve(N);
        for (size_t r = 0; r < N; ++r) {
            BatchedDecodeOutput::PerRequest p;
            p.request_id = slots[r].request_id;
            p.success = true;
            if (!to_sink && !greedy) p.logits.assign(logits_pinned_ + r * vocab, logits_pinned_ + (r + 1) * vocab);
            reqs[r]->next_position = slots[r].sequence_position + 1;
            out.per_request.push_back(std::move(p));
        }
        if (walker_trace())
            std::fprintf(stderr, "[walker] tables+plan %.0f us | encode %.0f | flush + logits %.0f | rows %.0f | total %.0f\n",
                         t_plan - t_start, t_enc - t_plan, t_flush - t_enc, now_us() - t_flush, now_us() - t_start);
        return out;
    }

    // Name-keyed persistent device buffers, as the reference's walker keeps (163-180).
    const size_t q_bytes = N * H * D * sizeof(float), kv_bytes = N * KVH * D * sizeof(uint16_t);
    void* buf_q = mlc_cached_buffer(ctx, "walker_q", q_bytes * ex.L_);
    void* buf_k = mlc_cached_buffer(ctx, "walker_kv_f16_k", kv_bytes * ex.L_);
    void* buf_v = mlc_cached_buffer(ctx, "walker_kv_f16_v", kv_bytes * ex.L_);
    void* buf_o = mlc_cached_buffer(ctx, "walker_attn_mix", q_bytes * ex.L_);   // one output block per layer
    if (!buf_q || !buf_k || !buf_v || !buf_o) return fail_all();

    q_host_.resize(N * H * D * ex.L_);
    k_host_.resize(N * KVH * D * ex.L_);
    v_host_.resize(N * KVH * D * ex.L_);
    for (uint32_t layer = 0; layer < ex.L_; ++layer)
        ex.source_->fill(layer, slots, H, KVH, D, q_host_.data() + static_cast<size_t>(layer) * N * H * D,
                         k_host_.data() + static_cast<size_t>(layer) * N * KVH * D,
                         v_host_.data() + static_cast<size_t>(layer) * N * KVH * D);
    if (mlc_upload(ctx, buf_q, q_host_.data(), q_bytes * ex.L_, 0) != MLC_OK ||
        mlc_upload(ctx, buf_k, k_host_.data(), kv_bytes * ex.L_, 0) != MLC_OK ||
        mlc_upload(ctx, buf_v, v_host_.data(), kv_bytes * ex.L_, 0) != MLC_OK)
        return fail_all();


    bool ok = mlc_pass_begin(ctx) == MLC_OK;
    if (ok && fused) {
        // Every layer's Q and new rows are on the device already (this walker has no model between the
        // attention layers), so the pass goes to the library as one call - one launch when the plan allows.
        std::vector<const void*> qv(ex.L_), knv(ex.L_), vnv(ex.L_);
        std::vector<void*> kpv(ex.L_), vpv(ex.L_), ov(ex.L_);
        for (uint32_t layer = 0; layer < ex.L_; ++layer) {
            qv[layer] = static_cast<const char*>(buf_q) + static_cast<size_t>(layer) * q_bytes;
            knv[layer] = static_cast<const char*>(buf_k) + static_cast<size_t>(layer) * kv_bytes;
            vnv[layer] = static_cast<const char*>(buf_v) + static_cast<size_t>(layer) * kv_bytes;
            kpv[layer] = storage->k_buffer(layer);
            vpv[layer] = storage->v_buffer(layer);
            ov[layer] = static_cast<char*>(buf_o) + static_cast<size_t>(layer) * q_bytes;
        }
        ok = mlc_encode_paged_decode_pass_planned(ctx, plan, ex.L_, qv.data(), knv.data(), vnv.data(), kpv.data(),
                                                  vpv.data(), ov.data(), scale, MLC_F32, MLC_F32) == MLC_OK;
    }
    for (uint32_t layer = 0; ok && !fused && layer < ex.L_; ++layer) {
        const char* q_l = static_cast<const char*>(buf_q) + static_cast<size_t>(layer) * q_bytes;
        const char* k_l = static_cast<const char*>(buf_k) + static_cast<size_t>(layer) * kv_bytes;
        const char* v_l = static_cast<const char*>(buf_v) + static_cast<size_t>(layer) * kv_bytes;
        void* kp = storage->k_buffer(layer);
        void* vp = storage->v_buffer(layer);
        void* o_l = static_cast<char*>(buf_o) + static_cast<size_t>(layer) * q_bytes;
        {
            // the reference's call order (batched_walker.cpp:299-331)
            ok = mlc_encode_scatter_kv_paged_batched_f16(ctx, kp, page_ids.data(), slot_ids.data(), P, KVH, D, N,
                                                         k_l, cap) == MLC_OK &&
                 mlc_encode_scatter_kv_paged_batched_f16(ctx, vp, page_ids.data(), slot_ids.data(), P, KVH, D, N,
                                                         v_l, cap) == MLC_OK &&
                 mlc_encode_paged_flash_attention(ctx, q_l, kp, vp, o_l, pt_flat.data(), pt_flat.size(),
                                                  pt_off.data(), seq_lens.data(), q_pos.data(), N, H, KVH, D, P, 1,
                                                  scale, MLC_F32, MLC_F32, cap) == MLC_OK;
        }
    }
    ok = (mlc_pass_flush(ctx) == MLC_OK) && ok;
    if (!ok) return fail_all();

    // what the reference downloads as logits [N, vocab] (461-475) is the last layer's
    // attention output [N, H*D] here
    o_host_.resize(N * H * D);
    if (mlc_download(ctx, buf_o, o_host_.data(), q_bytes, static_cast<size_t>(ex.L_ - 1) * q_bytes) != MLC_OK) return fail_all();
    out.per_request.reserve(N);
    for (size_t r = 0; r < N; ++r) {
        BatchedDecodeOutput::PerRequest p;
        p.request_id = slots[r].request_id;
        p.success = true;
        p.logits.assign(o_host_.begin() + static_cast<std::ptrdiff_t>(r * H * D),
                        o_host_.begin() + static_cast<std::ptrdiff_t>((r + 1) * H * D));
        reqs[r]->next_position = slots[r].sequence_position + 1;
        out.per_request.push_back(std::move(p));
    }
    return out;
}

// One decode pass of the model, layer by layer as the reference's walker encodes it
// (batched_walker.cpp:183-458). In the reference's call order every op is its own launch, 13 per layer:
// RMSNorm, QKV mat-vec, split + rotary + cast, scatter K, scatter V, attention, output mat-vec, add, RMSNorm,
// gate | up mat-vec, split + SiLU * up, down mat-vec, add. The fused order makes the same step with 8:
// the rotary kernel writes the K / V rows into the pools itself, the output and down projections add the
// residual in their epilogue, and the down projection computes SiLU(gate) * up as it loads its input.
bool BatchedWalker::encode_model_pass(const std::vector<RequestSlot>& slots, mlc_attn_plan* plan,
                                      const std::vector<uint32_t>& page_ids, const std::vector<uint32_t>& slot_ids,
                                      const std::vector<uint32_t>& pt_flat, const std::vector<uint32_t>& pt_off,
                                      const std::vector<uint32_t>& seq_lens, const std::vector<uint32_t>& q_pos,
                                      float* logits_host, size_t logits_stride, size_t head_first,
                                      bool rows_per_request_only, uint32_t* greedy_host) {
    PagedAttentionExecutor& ex = exec_;
    mlc_ctx* ctx = ex.ctx_;
    PagedKVStorage* storage = ex.storage_;
    const ModelWeights& m = *ex.model_;
    const size_t N = slots.size();
    const uint32_t H = ex.H_, KVH = ex.KVH_, D = ex.D_, P = storage->page_size_tokens();
    const size_t hidden = m.hidden_size, inner = m.ffn_inner, vocab = m.vocab_size;
    const size_t q_rows = static_cast<size_t>(H) * D, k_rows = static_cast<size_t>(KVH) * D, qkv_rows = q_rows + 2 * k_rows;
    const size_t row_h = hidden / 32 * 18, row_i = inner / 32 * 18;   // Q4_0 row sizes
    const size_t cap = storage->capacity_pages();
    const bool fused = ex.order_ == PagedAttentionExecutor::CallOrder::Fused && plan;
    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    const float eps = m.rms_epsilon;

    auto scratch = [&](const char* name, size_t bytes) { return mlc_cached_buffer(ctx, name, bytes); };
    const size_t fb = sizeof(float);
    void* residual = scratch("w_residual", N * hidden * fb);
    void* norm_o = scratch("w_norm_out", N * hidden * fb);
    void* qkv = scratch("w_qkv", N * qkv_rows * fb);
    void* q = scratch("w_q", N * q_rows * fb);
    void* attn_mix = scratch("w_attn_mix", N * hidden * fb);
    void* resid1 = scratch("w_resid1", N * hidden * fb);
    void* gate_up = scratch("w_gate_up", N * 2 * inner * fb);
    void* final_n = scratch("w_final_norm", N * hidden * fb);
    void* logits = scratch("w_logits", N * vocab * fb);
    void* tokens = scratch("w_tokens", N * sizeof(uint32_t));
    const size_t pairs = m.rotary_dim / 2;
    void* cos_t = scratch("w_rope_cos", std::max<size_t>(1, N * pairs) * fb);
    void* sin_t = scratch("w_rope_sin", std::max<size_t>(1, N * pairs) * fb);
    if (!residual || !norm_o || !qkv || !q || !attn_mix || !resid1 || !gate_up || !final_n || !logits || !tokens ||
        !cos_t || !sin_t)
        return false;
    // buffers only the reference's call order needs
    void *k32 = nullptr, *v32 = nullptr, *k16 = nullptr, *v16 = nullptr, *attn_out = nullptr, *ffn_mix = nullptr,
         *ffn_down = nullptr;
    if (!fused) {
        k32 = scratch("w_k", N * k_rows * fb);
        v32 = scratch("w_v", N * k_rows * fb);
        k16 = scratch("w_kv_f16_k", N * k_rows * 2);
        v16 = scratch("w_kv_f16_v", N * k_rows * 2);
        attn_out = scratch("w_attn_out", N * hidden * fb);
        ffn_mix = scratch("w_ffn_mix", N * inner * fb);
        ffn_down = scratch("w_ffn_down", N * hidden * fb);
        if (!k32 || !v32 || !k16 || !v16 || !attn_out || !ffn_mix || !ffn_down) return false;
    }

    // token ids and the pass's rotary tables (position-only: one upload serves every layer, 215-236)
    tok_host_.resize(N);
    for (size_t r = 0; r < N; ++r) {
        if (slots[r].input_token >= vocab) return false;
        tok_host_[r] = static_cast<uint32_t>(slots[r].input_token);
    }
    if (mlc_upload(ctx, tokens, tok_host_.data(), N * sizeof(uint32_t), 0) != MLC_OK) return false;
    if (pairs) {
        cos_host_.resize(N * pairs);
        sin_host_.resize(N * pairs);
        for (size_t r = 0; r < N; ++r)
            mlc_compute_rotary_coefficients(slots[r].sequence_position, m.rotary_dim, m.rope_base, m.rope_scale,
                                            cos_host_.data() + r * pairs, sin_host_.data() + r * pairs);
        if (mlc_upload(ctx, cos_t, cos_host_.data(), N * pairs * fb, 0) != MLC_OK ||
            mlc_upload(ctx, sin_t, sin_host_.data(), N * pairs * fb, 0) != MLC_OK)
            return false;
    }

    bool ok = mlc_encode_embedding_q4_0(ctx, m.token_embd, row_h, tokens, N, hidden, vocab, residual) == MLC_OK;
    char range_name[32];
    for (uint32_t L = 0; ok && L < ex.L_; ++L) {
        std::snprintf(range_name, sizeof(range_name), "mlc layer %u", L);
        NvtxRange layer_range(range_name);
        const LayerWeights& w = m.layers[L];
        void* kp = storage->k_buffer(L);
        void* vp = storage->v_buffer(L);
        // fused order: the norms write the mat-vec's operand format directly (the mat-vec then converts nothing)
        // fused order, head_dim a multiple of 4: the QKV projection rotates, casts and writes Q and the K / V page rows
        // itself; otherwise the projection leaves fp32 rows for the split / rotary / page-write kernel
        const bool qkv_epilogue = fused && D % 4 == 0;
        ok = fused ? mlc_encode_rms_norm_batched_packed(ctx, residual, w.attn_norm, eps, N, hidden, nullptr, norm_o) == MLC_OK &&
                         (qkv_epilogue
                              ? mlc_encode_matmul_qkv_rope_scatter_planned(ctx, plan, 0, w.attn_qkv, norm_o, hidden, 2, hidden, row_h,
                                                                           q, kp, vp, cos_t, sin_t, m.rotary_dim)
                              : mlc_encode_matmul_quant_fused(ctx, 0, w.attn_qkv, norm_o, hidden, 2, nullptr, N, qkv_rows, hidden,
                                                              row_h, qkv)) == MLC_OK
                   : mlc_encode_rms_norm_batched(ctx, residual, w.attn_norm, eps, N, hidden, norm_o, nullptr) == MLC_OK &&
                         mlc_encode_matmul_q4_0_batched(ctx, w.attn_qkv, norm_o, N, qkv_rows, hidden, row_h, qkv) == MLC_OK;
        if (!ok) break;
        if (fused) {
            ok = (qkv_epilogue || mlc_encode_qkv_split_rope_scatter_planned(ctx, plan, qkv, q, MLC_F16, kp, vp, cos_t, sin_t,
                                                                            qkv_rows, m.rotary_dim) == MLC_OK) &&
                 (rows_per_request_only
                      ? encode_attention_planned_after_row_write(ctx, plan, q, kp, vp, attn_mix, scale, MLC_F16, MLC_F32)
                      : mlc_encode_paged_flash_attention_planned(ctx, plan, q, kp, vp, attn_mix, scale, MLC_F16, MLC_F32)) == MLC_OK &&
                 mlc_encode_matmul_quant_fused(ctx, 0, w.attn_output, attn_mix, hidden, 0, residual, N, hidden, hidden,
                                               row_h, resid1) == MLC_OK &&
                 mlc_encode_rms_norm_batched_packed(ctx, resid1, w.ffn_norm, eps, N, hidden, nullptr, norm_o) == MLC_OK &&
                 // SiLU(gate) * up leaves the gate | up kernel as operand words [N, inner] (in the gate_up scratch)
                 mlc_encode_matmul_gate_up_silu_packed(ctx, 0, w.ffn_gate_up, norm_o, hidden, 2, N, inner, hidden, row_h,
                                                       gate_up) == MLC_OK &&
                 mlc_encode_matmul_quant_fused(ctx, 0, w.ffn_down, gate_up, inner, 2, resid1, N, hidden, inner, row_i,
                                               residual) == MLC_OK;
        } else {
            ok = mlc_encode_qkv_split_rope_cast(ctx, qkv, q, k32, v32, k16, v16, cos_t, sin_t, N, H, KVH, D, qkv_rows,
                                                q_rows, k_rows, k_rows, m.rotary_dim) == MLC_OK &&
                 mlc_encode_scatter_kv_paged_batched_f16(ctx, kp, page_ids.data(), slot_ids.data(), P, KVH, D, N, k16,
                                                         cap) == MLC_OK &&
                 mlc_encode_scatter_kv_paged_batched_f16(ctx, vp, page_ids.data(), slot_ids.data(), P, KVH, D, N, v16,
                                                         cap) == MLC_OK &&
                 mlc_encode_paged_flash_attention(ctx, q, kp, vp, attn_mix, pt_flat.data(), pt_flat.size(), pt_off.data(),
                                                  seq_lens.data(), q_pos.data(), N, H, KVH, D, P, 1, scale, MLC_F32,
                                                  MLC_F32, cap) == MLC_OK &&
                 mlc_encode_matmul_q4_0_batched(ctx, w.attn_output, attn_mix, N, hidden, hidden, row_h, attn_out) == MLC_OK &&
                 mlc_encode_add_batched(ctx, residual, attn_out, resid1, N * hidden) == MLC_OK &&
                 mlc_encode_rms_norm_batched(ctx, resid1, w.ffn_norm, eps, N, hidden, norm_o, nullptr) == MLC_OK &&
                 mlc_encode_matmul_q4_0_batched(ctx, w.ffn_gate_up, norm_o, N, 2 * inner, hidden, row_h, gate_up) == MLC_OK &&
                 mlc_encode_gate_up_split_silu_mul(ctx, gate_up, nullptr, nullptr, ffn_mix, N, inner, 2 * inner) == MLC_OK &&
                 mlc_encode_matmul_q4_0_batched(ctx, w.ffn_down, ffn_mix, N, hidden, inner, row_i, ffn_down) == MLC_OK &&
                 mlc_encode_add_batched(ctx, resid1, ffn_down, residual, N * hidden) == MLC_OK;
        }
    }
    NvtxRange head_range("mlc final norm + lm_head");
    const size_t head_stride = m.lm_head_quant == 1 ? hidden / 256 * 210 : row_h;
    const int head_quant = m.lm_head_quant == 1 ? 1 : 0;
    if (!ok) return false;
    // Only rows [head_first, N) get logits (a prompt chunk wants its last token's, or none at all)
    if (head_first >= N) return true;
    const size_t head_n = N - head_first;
    const float* head_in = static_cast<const float*>(residual) + head_first * hidden;
    if ((fused ? mlc_encode_rms_norm_batched_packed(ctx, head_in, m.output_norm, eps, head_n, hidden, nullptr, final_n)
               : mlc_encode_rms_norm_batched(ctx, head_in, m.output_norm, eps, head_n, hidden, final_n, nullptr)) != MLC_OK)
        return false;
    // The lm_head runs as groups of vocabulary rows (one group in the reference's call order): a group's logits
    // [N, rows of the group] start for the host - page-locked rows, on the copy-back stream - while the next
    // group is computed, so all but the last group's share of the copy is off the step's critical path.
    // mlc_pass_flush waits for the last copy.
    const size_t groups = fused ? 4 : 1;
    const size_t group_rows = ((vocab + groups - 1) / groups + 63) / 64 * 64;
    DeviceGuard guard(ctx->device);
    if (!ctx->d2h_stream && cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking) != cudaSuccess) return false;
    while (ctx->pass_events.size() < groups + 1) {
        cudaEvent_t e;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return false;
        ctx->pass_events.push_back(e);
    }
    size_t g = 0;
    for (size_t r0 = 0; r0 < vocab; r0 += group_rows, ++g) {
        const size_t nr = std::min(group_rows, vocab - r0);
        float* out_g = static_cast<float*>(logits) + head_n * r0;
        const uint8_t* w_g = static_cast<const uint8_t*>(m.lm_head) + r0 * head_stride;
        const int st = fused ? mlc_encode_matmul_quant_fused(ctx, head_quant, w_g, final_n, hidden, 2, nullptr, head_n, nr, hidden,
                                                             head_stride, out_g)
                       : head_quant == 1 ? mlc_encode_matmul_q6k_batched(ctx, w_g, final_n, head_n, nr, hidden, head_stride, out_g)
                                         : mlc_encode_matmul_q4_0_batched(ctx, w_g, final_n, head_n, nr, hidden, head_stride, out_g);
        if (st != MLC_OK) return false;
        if (greedy_host) continue;   // the logits stay on the device
        if (cudaEventRecord(ctx->pass_events[g], ctx->stream) != cudaSuccess ||
            cudaStreamWaitEvent(ctx->d2h_stream, ctx->pass_events[g], 0) != cudaSuccess ||
            cudaMemcpy2DAsync(logits_host + r0, logits_stride * sizeof(float), out_g, nr * sizeof(float), nr * sizeof(float), head_n,
                              cudaMemcpyDeviceToHost, ctx->d2h_stream) != cudaSuccess)
            return false;
    }
    if (greedy_host) {
        // greedy sampling on the device: one token id per request comes back instead of the logits
        void* ids = scratch("w_argmax", head_n * sizeof(uint32_t));
        return ids && mlc_encode_argmax_rows(ctx, logits, head_n, vocab, group_rows, ids) == MLC_OK &&
               cudaMemcpyAsync(greedy_host, ids, head_n * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess;
    }
    if (cudaEventRecord(ctx->pass_events[groups], ctx->d2h_stream) != cudaSuccess) return false;
    ctx->host_pass_done = ctx->pass_events[groups];
    return true;
}


std::vector<float> BatchedWalker::prefill_model(uint32_t request_id, const std::vector<uint64_t>& tokens, size_t cursor) {
    PagedAttentionExecutor& ex = exec_;
    mlc_ctx* ctx = ex.ctx_;
    PagedKVStorage* storage = ex.storage_;
    if (tokens.empty() || !storage || !ex.pool_ || !ex.model_) return {};
    const uint32_t H = ex.H_, KVH = ex.KVH_, D = ex.D_, P = storage->page_size_tokens();
    const size_t vocab = ex.model_->vocab_size, cap = storage->capacity_pages();
    constexpr size_t kChunk = 32;   // tokens per pass: the mat-vec kernels' best batch

    PagedAttentionExecutor::PerRequest& req = ex.ensure_request(request_id);
    if (!req.page_state) {
        req.page_state.reset(new RequestKVState());
        req.page_state->request_id = request_id;
        req.page_state->page_size_tokens = ex.page_size_tokens_;
    }
    if (logits_pinned_floats_ < vocab) {
        if (logits_pinned_) cudaFreeHost(logits_pinned_);
        logits_pinned_ = nullptr;
        logits_pinned_floats_ = 0;
        DeviceGuard guard(ctx->device);
        if (cudaHostAlloc(reinterpret_cast<void**>(&logits_pinned_), vocab * sizeof(float), cudaHostAllocDefault) != cudaSuccess)
            return {};
        logits_pinned_floats_ = vocab;
        ++ctx->allocations;
    }
    for (size_t done = 0; done < tokens.size(); done += kChunk) {
        const size_t n = std::min(kChunk, tokens.size() - done);
        // The chunk's tokens stand in the pass like n requests that share one page table: token i sees the
        // context up to and including itself (its row and the rows of the chunk's earlier tokens are written
        // before any attention of the layer runs). A pool that runs out fails the prefill; the pages taken so
        // far stay with the request until it is released, as in the token loop.
        std::vector<uint32_t> page_ids(n), slot_ids(n), seq_lens(n), q_pos(n), pt_off(n + 1, 0), pt_flat;
        std::vector<RequestSlot> slots(n);
        for (size_t i = 0; i < n; ++i) {
            auto loc = req.page_state->extend_one_token(*ex.pool_);
            if (!loc) return {};
            page_ids[i] = loc->first;
            slot_ids[i] = loc->second;
            slots[i] = RequestSlot{request_id, tokens[done + i], cursor + done + i};
        }
        const std::vector<uint32_t>& table = req.page_state->page_table;
        for (size_t i = 0; i < n; ++i) {
            q_pos[i] = static_cast<uint32_t>(cursor + done + i);
            seq_lens[i] = q_pos[i] + 1;
            const size_t pages = (seq_lens[i] + P - 1) / P;
            if (pages > table.size()) return {};   // the cursor does not continue the request's context
            pt_off[i] = static_cast<uint32_t>(pt_flat.size());
            pt_flat.insert(pt_flat.end(), table.begin(), table.begin() + pages);
        }
        pt_off[n] = static_cast<uint32_t>(pt_flat.size());
        mlc_attn_plan*& slot = ex.plans_[ex.passes_++ & 1u];
        const int st = slot ? mlc_attn_plan_update(ctx, slot, pt_flat.data(), pt_flat.size(), pt_off.data(), seq_lens.data(),
                                                   q_pos.data(), page_ids.data(), slot_ids.data(), n)
                            : mlc_attn_plan_create(ctx, pt_flat.data(), pt_flat.size(), pt_off.data(), seq_lens.data(),
                                                   q_pos.data(), page_ids.data(), slot_ids.data(), n, H, KVH, D, P, 1, cap,
                                                   &slot);
        if (st != MLC_OK) return {};
        const bool last = done + n == tokens.size();
        bool ok = mlc_pass_begin(ctx) == MLC_OK;
        ok = ok && encode_model_pass(slots, slot, page_ids, slot_ids, pt_flat, pt_off, seq_lens, q_pos, logits_pinned_, vocab,
                                     last ? n - 1 : n, false, nullptr);   // a chunk's rows are context of the chunk's later tokens
        ok = (mlc_pass_flush(ctx) == MLC_OK) && ok;
        if (!ok) return {};
    }
    req.next_position = cursor + tokens.size();
    return std::vector<float>(logits_pinned_, logits_pinned_ + vocab);
}

std::vector<float> BatchedWalker::prefill(uint32_t request_id, const std::vector<uint64_t>& tokens, size_t cursor) {
    PagedAttentionExecutor& ex = exec_;
    mlc_ctx* ctx = ex.ctx_;
    PagedKVStorage* storage = ex.storage_;
    const size_t n = tokens.size();
    if (n == 0 || !storage || !ex.pool_) return {};
    const uint32_t H = ex.H_, KVH = ex.KVH_, D = ex.D_, P = storage->page_size_tokens();

    PagedAttentionExecutor::PerRequest& req = ex.ensure_request(request_id);
    if (!req.page_state) {
        req.page_state.reset(new RequestKVState());
        req.page_state->request_id = request_id;
        req.page_state->page_size_tokens = ex.page_size_tokens_;
    }
    // one (page, slot) per token of the chunk; a pool that runs out fails the prefill and the
    // pages taken so far stay with the request until it is released, as in the token loop
    std::vector<uint32_t> page_ids(n), slot_ids(n);
    std::vector<RequestSlot> slots(n);
    for (size_t i = 0; i < n; ++i) {
        auto loc = req.page_state->extend_one_token(*ex.pool_);
        if (!loc) return {};
        page_ids[i] = loc->first;
        slot_ids[i] = loc->second;
        slots[i] = RequestSlot{request_id, tokens[i], cursor + i};
    }
    const std::vector<uint32_t>& table = req.page_state->page_table;
    const uint32_t pt_off[2] = {0u, static_cast<uint32_t>(table.size())};
    const uint32_t seq_len = static_cast<uint32_t>(req.page_state->total_tokens());
    const uint32_t q_start = static_cast<uint32_t>(cursor), q_len = static_cast<uint32_t>(n);
    if (static_cast<uint64_t>(q_start) + q_len != seq_len) return {};  // the chunk must end the sequence

    const size_t q_elems = n * H * D, kv_elems = n * KVH * D;
    void* buf_q = mlc_cached_buffer(ctx, "walker_prefill_q_f16", q_elems * 2);
    void* buf_k = mlc_cached_buffer(ctx, "walker_prefill_k_f16", kv_elems * 2);
    void* buf_v = mlc_cached_buffer(ctx, "walker_prefill_v_f16", kv_elems * 2);
    void* buf_o = mlc_cached_buffer(ctx, "walker_prefill_o_f16", q_elems * 2);
    if (!buf_q || !buf_k || !buf_v || !buf_o) return {};
    q_host_.resize(q_elems);
    q16_host_.resize(q_elems);
    k_host_.resize(kv_elems);
    v_host_.resize(kv_elems);

    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    const size_t cap = storage->capacity_pages();
    for (uint32_t layer = 0; layer < ex.L_; ++layer) {
        ex.source_->fill(layer, slots, H, KVH, D, q_host_.data(), k_host_.data(), v_host_.data());
        for (size_t i = 0; i < q_elems; ++i) {  // the decode kernel makes the same cast when it loads fp32 Q
            const __half_raw h = __float2half_rn(q_host_[i]);
            q16_host_[i] = h.x;
        }
        if (mlc_upload(ctx, buf_q, q16_host_.data(), q_elems * 2, 0) != MLC_OK ||
            mlc_upload(ctx, buf_k, k_host_.data(), kv_elems * 2, 0) != MLC_OK ||
            mlc_upload(ctx, buf_v, v_host_.data(), kv_elems * 2, 0) != MLC_OK)
            return {};
        void* kp = storage->k_buffer(layer);
        void* vp = storage->v_buffer(layer);
        bool ok = mlc_pass_begin(ctx) == MLC_OK;
        ok = ok && mlc_encode_scatter_kv_pair_paged_batched_f16(ctx, kp, vp, page_ids.data(), slot_ids.data(), P, KVH,
                                                                D, n, buf_k, buf_v, cap) == MLC_OK;
        ok = ok && mlc_encode_paged_prefill_attention(ctx, buf_q, kp, vp, buf_o, table.data(), table.size(), pt_off,
                                                      &seq_len, &q_start, &q_len, 1, H, KVH, D, P, scale, MLC_F16,
                                                      MLC_F16, cap) == MLC_OK;
        ok = (mlc_pass_flush(ctx) == MLC_OK) && ok;
        if (!ok) return {};
    }
    // the last token's row of the last layer
    o16_host_.resize(static_cast<size_t>(H) * D);
    if (mlc_download(ctx, buf_o, o16_host_.data(), o16_host_.size() * 2, (n - 1) * static_cast<size_t>(H) * D * 2) != MLC_OK)
        return {};
    std::vector<float> last(o16_host_.size());
    for (size_t i = 0; i < last.size(); ++i) {
        __half_raw h;
        h.x = o16_host_[i];
        last[i] = __half2float(__half(h));
    }
    req.next_position = cursor + n;
    return last;
}

}  // namespace runtime
}  // namespace mlcb
