// Executor interface the scheduler drives, and the paged-attention executor behind it.
//
// RequestSlot / BatchedDecodeOutput / IBatchedExecutor carry the reference's names and
// meaning (compiler/runtime/batched_executor.hpp:33-57). PagedAttentionExecutor is the
// part of the reference's BatchedExecutor that belongs to the paged-attention path
// (batched_executor.hpp:59-141, batched_executor.cpp:29-65, 96-103, 445-467): per-request
// page state, pool / storage attachment, page release, decode routed to the batched
// walker, prefill as a loop of single-token decode passes. The model around attention
// (embeddings, mat-vecs, norms, logits) is out of this repository's scope: Q and the new
// K/V rows of every layer come from an IQkvSource, and what the reference returns as
// logits is here the attention output of the last layer.
#pragma once

#include <cstdint>
#include <memory>
#include <unordered_map>
#include <vector>

#include <string>

#include "paged_kv.hpp"

struct mlc_ctx;
struct mlc_attn_plan;

namespace mlcb {
namespace gguf {
class File;
}
namespace runtime {

struct RequestSlot {
    uint32_t request_id = 0;
    uint64_t input_token = 0;
    size_t sequence_position = 0;
};

struct BatchedDecodeOutput {
    struct PerRequest {
        uint32_t request_id = 0;
        bool success = false;
        std::vector<float> logits;  // empty on failure
    };
    std::vector<PerRequest> per_request;
};

class IBatchedExecutor {
public:
    virtual ~IBatchedExecutor() = default;
    virtual BatchedDecodeOutput run_decode(const std::vector<RequestSlot>& slots) = 0;
    // Optional (no counterpart in the reference, whose scheduler takes the argmax of the logits itself,
    // scheduler.cpp:101-118): the same pass ending in greedy sampling inside the executor. On success tokens[i] is
    // the index of the first maximum of slot i's logits and the function returns true; an executor that cannot do
    // this returns false without having run anything, and the caller falls back to run_decode.
    virtual bool run_decode_greedy(const std::vector<RequestSlot>& slots, std::vector<uint64_t>& tokens) {
        (void)slots;
        (void)tokens;
        return false;
    }
    virtual std::vector<float> run_prefill(uint32_t request_id, const std::vector<uint64_t>& tokens) = 0;
    virtual void release_request(uint32_t request_id) = 0;
};

// Supplies, for one layer of one pass, what the projections before attention would:
// q fp32 [N, H, D] and the new K / V rows as fp16 bits [N, KVH, D], on the host.
class IQkvSource {
public:
    virtual ~IQkvSource() = default;
    virtual void fill(uint32_t layer, const std::vector<RequestSlot>& slots, uint32_t H, uint32_t KVH, uint32_t D,
                      float* q, uint16_t* k_new, uint16_t* v_new) = 0;
};

// Deterministic stand-in: every element is a hash of (seed, request, token, position,
// layer, tensor, index) mapped onto the grid {-1024..1023}/1024, which fp16 holds exactly.
class HashQkvSource : public IQkvSource {
public:
    explicit HashQkvSource(uint64_t seed) : seed_(seed) {}
    void fill(uint32_t layer, const std::vector<RequestSlot>& slots, uint32_t H, uint32_t KVH, uint32_t D,
              float* q, uint16_t* k_new, uint16_t* v_new) override;
    static float value(uint64_t seed, uint32_t request, uint64_t token, uint64_t position, uint32_t layer,
                       uint32_t tensor, uint32_t index);

private:
    uint64_t seed_;
};

// Device-resident weights of a Llama-style decoder in the reference's GGUF tensor roles
// (batched_walker.cpp:248-458): per layer attn_norm, fused attn_qkv, attn_output, ffn_norm, fused
// ffn gate | up, ffn_down (mat-vec weights Q4_0), then output_norm and the lm_head (Q6_K or Q4_0);
// token_embd is a Q4_0 table. Rows are tightly packed (row stride = the format's row size).
struct LayerWeights {
    const float* attn_norm = nullptr;
    const uint8_t* attn_qkv = nullptr;
    const uint8_t* attn_output = nullptr;
    const float* ffn_norm = nullptr;
    const uint8_t* ffn_gate_up = nullptr;
    const uint8_t* ffn_down = nullptr;
};

struct ModelWeights {
    uint32_t hidden_size = 0, ffn_inner = 0, vocab_size = 0, rotary_dim = 0;
    float rope_base = 10000.0f, rope_scale = 1.0f, rms_epsilon = 1e-5f;
    int lm_head_quant = 1;   // 0 = Q4_0, 1 = Q6_K
    const uint8_t* token_embd = nullptr;
    const float* output_norm = nullptr;
    const uint8_t* lm_head = nullptr;
    std::vector<LayerWeights> layers;
};

class BatchedWalker;

class PagedAttentionExecutor : public IBatchedExecutor {
    friend class BatchedWalker;

public:
    enum class CallOrder {
        Fused,      // one launch per layer: KV row write fused into attention
        Reference,  // the reference walker's order: scatter K, scatter V, attention
    };

    PagedAttentionExecutor(mlc_ctx* ctx, uint32_t num_heads, uint32_t kv_heads, uint32_t head_dim,
                           uint32_t n_layers, std::unique_ptr<IQkvSource> source);
    ~PagedAttentionExecutor() override;

    void attach_page_pool(PagePool* pool, uint32_t page_size_tokens = 64);
    void attach_paged_storage(PagedKVStorage* storage) { storage_ = storage; }
    void set_call_order(CallOrder o) { order_ = o; }
    // With a model attached a decode pass is the whole walker step - embedding, every layer's norms,
    // mat-vecs, rotary, attention and residual adds, final norm and lm_head - and the logits are the model's
    // [vocab_size] per request; a prompt is fed token by token through the decode path in the reference's call
    // order (batched_executor.cpp:450-467), 32 tokens per pass in the fused order. Returns false if the
    // description does not fit the executor.
    bool run_decode_greedy(const std::vector<RequestSlot>& slots, std::vector<uint64_t>& tokens) override;
    bool attach_model(const ModelWeights& model);
    // Reads the model out of a GGUF file (the tensors and metadata keys the reference's walker uses,
    // batched_walker.cpp:183-190, 248-420; kernel_scheduler.cpp:251-258), uploads the weights into one device
    // allocation owned by this executor and attaches them. On failure `error` says what is missing or unfit.
    bool attach_gguf(gguf::File& file, std::string* error);
    bool has_model() const { return model_ != nullptr; }
    // Gives a request that has no pages yet a context of `tokens` tokens whose K/V rows the caller has put
    // (or will put) into the pools itself: pages are reserved and the next position is `tokens`. For
    // restoring a saved context and for benchmarks that start from long contexts. False if the request
    // already has pages or the pool cannot supply them.
    bool assume_context(uint32_t request_id, size_t tokens);
    const RequestKVState* page_state(uint32_t request_id) const;

    BatchedDecodeOutput run_decode(const std::vector<RequestSlot>& slots) override;
    // The same pass with a model attached, the logits written to the caller's rows (row r at logits + r * stride
    // floats, stride >= vocabulary size) instead of into per-request vectors; straight from the device when the
    // buffer is page-locked memory. The returned entries carry request ids and success flags only.
    BatchedDecodeOutput run_decode_into(const std::vector<RequestSlot>& slots, float* logits, size_t stride);
    size_t logits_per_request() const;
    std::vector<float> run_prefill(uint32_t request_id, const std::vector<uint64_t>& tokens) override;
    void release_request(uint32_t request_id) override;
    void reset();

    size_t known_position(uint32_t request_id) const;
    size_t live_request_count() const { return requests_.size(); }
    uint32_t num_heads() const { return H_; }
    uint32_t kv_heads() const { return KVH_; }
    uint32_t head_dim() const { return D_; }
    uint32_t n_layers() const { return L_; }

private:
    struct PerRequest {
        size_t next_position = 0;
        std::unique_ptr<RequestKVState> page_state;
    };
    PerRequest& ensure_request(uint32_t request_id);

    mlc_ctx* ctx_;
    uint32_t H_, KVH_, D_, L_;
    std::unique_ptr<IQkvSource> source_;
    std::unique_ptr<ModelWeights> model_;
    void* model_arena_ = nullptr;   // device memory of a model loaded by attach_gguf
    void release_model_arena();
    std::unordered_map<uint32_t, PerRequest> requests_;
    PagePool* pool_ = nullptr;
    uint32_t page_size_tokens_ = 64;
    PagedKVStorage* storage_ = nullptr;
    CallOrder order_ = CallOrder::Fused;
    std::unique_ptr<BatchedWalker> walker_;
    mlc_attn_plan* plans_[2] = {nullptr, nullptr};   // the walker's two long-lived plans (alternate passes)
    uint64_t passes_ = 0;
};

}  // namespace runtime
}  // namespace mlcb
