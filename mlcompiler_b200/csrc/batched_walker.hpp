// One batched decode pass over all layers for N requests: the paged-attention section of
// the reference's BatchedWalker::step (compiler/runtime/batched_walker.cpp:81-479; page
// extension 127-149, scatter + table build + attention 299-331).
#pragma once

#include <vector>

#include "batched_executor.hpp"

namespace mlcb {
namespace runtime {

class BatchedWalker {
public:
    explicit BatchedWalker(PagedAttentionExecutor& exec) : exec_(exec) {}
    ~BatchedWalker();
    // Where a model pass may put its logits instead of into per-request vectors: row r at dst + r * stride floats.
    struct LogitsSink {
        float* dst = nullptr;
        size_t stride = 0;
    };
    // greedy (model attached only): the pass ends with the argmax of every request's logits on the device and
    // *greedy receives one token id per request; no logits come back.
    BatchedDecodeOutput step(const std::vector<RequestSlot>& slots, const LogitsSink* sink = nullptr,
                             std::vector<uint64_t>* greedy = nullptr);
    // All tokens of a prompt chunk in one pass per layer: the chunk's K/V rows are scattered,
    // then chunked causal attention runs over the request's pages. Returns the last token's
    // attention output of the last layer, or {} on failure. The reference reaches the same
    // state with one decode pass per token (batched_executor.cpp:450-467).
    std::vector<float> prefill(uint32_t request_id, const std::vector<uint64_t>& tokens, size_t cursor);
    // The same with a model attached: the prompt goes through the whole step 32 tokens per pass - a chunk's tokens
    // stand in the batch like requests that share one page table - and only the last token's logits are computed
    // and returned ({} on failure). The reference feeds a prompt one token per pass (batched_executor.cpp:450-467).
    std::vector<float> prefill_model(uint32_t request_id, const std::vector<uint64_t>& tokens, size_t cursor);

private:
    // The layers of a pass with a model attached: encodes embedding .. lm_head onto the open pass and the copies of
    // the logits of rows [head_first, N) into page-locked host rows `logits_stride` floats apart.
    // rows_per_request_only: every entry of the batch is a request of its own (a decode pass), so the only rows a
    // layer's QKV projection writes are the newest token's of each entry and attention may fetch everything else early.
    bool encode_model_pass(const std::vector<RequestSlot>& slots, mlc_attn_plan* plan, const std::vector<uint32_t>& page_ids,
                           const std::vector<uint32_t>& slot_ids, const std::vector<uint32_t>& pt_flat,
                           const std::vector<uint32_t>& pt_off, const std::vector<uint32_t>& seq_lens,
                           const std::vector<uint32_t>& q_pos, float* logits_host, size_t logits_stride, size_t head_first,
                           bool rows_per_request_only, uint32_t* greedy_host);

    PagedAttentionExecutor& exec_;
    std::vector<float> cos_host_, sin_host_;
    std::vector<uint32_t> tok_host_;
    float* logits_pinned_ = nullptr;   // page-locked landing area of the logits download, grown on demand
    size_t logits_pinned_floats_ = 0;
    uint32_t* tokens_pinned_ = nullptr;   // page-locked landing area of the greedy token ids
    size_t tokens_pinned_count_ = 0;
    // host staging, reused across passes
    std::vector<float> q_host_;
    std::vector<uint16_t> k_host_, v_host_;
    std::vector<float> o_host_;
    std::vector<uint16_t> q16_host_, o16_host_;
};

}  // namespace runtime
}  // namespace mlcb
