// See batched_executor.hpp.
#include "batched_executor.hpp"

#include "batched_walker.hpp"
#include "ctx.hpp"

#include <cstring>

namespace mlcb {
namespace runtime {

static inline uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

float HashQkvSource::value(uint64_t seed, uint32_t request, uint64_t token, uint64_t position, uint32_t layer,
                           uint32_t tensor, uint32_t index) {
    uint64_t h = mix64(seed ^ 0xA24BAED4963EE407ull);
    h = mix64(h ^ request);
    h = mix64(h ^ token);
    h = mix64(h ^ position);
    h = mix64(h ^ ((static_cast<uint64_t>(layer) << 8) | tensor));
    h = mix64(h ^ index);
    const int v = static_cast<int>((h >> 20) & 0x7FFu) - 1024;  // 11 bits: exact in fp16
    return static_cast<float>(v) / 1024.0f;
}

// fp32 -> fp16 bits for values on the {-1024..1023}/1024 grid (exactly representable).
static uint16_t grid_to_half(float f) {
    if (f == 0.0f) return 0;
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    const int32_t exp = static_cast<int32_t>((bits >> 23) & 0xFF) - 127 + 15;  // -10..0 -> 5..15
    const uint32_t man = (bits >> 13) & 0x3FFu;                                // low 13 bits are zero
    return static_cast<uint16_t>(sign | (static_cast<uint32_t>(exp) << 10) | man);
}

void HashQkvSource::fill(uint32_t layer, const std::vector<RequestSlot>& slots, uint32_t H, uint32_t KVH,
                         uint32_t D, float* q, uint16_t* k_new, uint16_t* v_new) {
    for (size_t r = 0; r < slots.size(); ++r) {
        const RequestSlot& s = slots[r];
        for (uint32_t i = 0; i < H * D; ++i)
            q[r * H * D + i] = value(seed_, s.request_id, s.input_token, s.sequence_position, layer, 0, i);
        for (uint32_t i = 0; i < KVH * D; ++i) {
            k_new[r * KVH * D + i] =
                grid_to_half(value(seed_, s.request_id, s.input_token, s.sequence_position, layer, 1, i));
            v_new[r * KVH * D + i] =
                grid_to_half(value(seed_, s.request_id, s.input_token, s.sequence_position, layer, 2, i));
        }
    }
}

PagedAttentionExecutor::PagedAttentionExecutor(mlc_ctx* ctx, uint32_t num_heads, uint32_t kv_heads,
                                               uint32_t head_dim, uint32_t n_layers,
                                               std::unique_ptr<IQkvSource> source)
    : ctx_(ctx), H_(num_heads), KVH_(kv_heads), D_(head_dim), L_(n_layers), source_(std::move(source)),
      walker_(new BatchedWalker(*this)) {}

PagedAttentionExecutor::~PagedAttentionExecutor() {
    for (mlc_attn_plan* p : plans_)
        if (p) mlc_attn_plan_destroy(ctx_, p);
    release_model_arena();
}

void PagedAttentionExecutor::attach_page_pool(PagePool* pool, uint32_t page_size_tokens) {
    pool_ = pool;
    page_size_tokens_ = page_size_tokens > 0 ? page_size_tokens : 64;  // batched_executor.cpp:47-50
}

const RequestKVState* PagedAttentionExecutor::page_state(uint32_t request_id) const {
    auto it = requests_.find(request_id);
    return it == requests_.end() ? nullptr : it->second.page_state.get();
}

size_t PagedAttentionExecutor::known_position(uint32_t request_id) const {
    auto it = requests_.find(request_id);
    return it == requests_.end() ? 0 : it->second.next_position;
}

PagedAttentionExecutor::PerRequest& PagedAttentionExecutor::ensure_request(uint32_t request_id) {
    return requests_[request_id];
}

bool PagedAttentionExecutor::assume_context(uint32_t request_id, size_t tokens) {
    if (!pool_ || tokens == 0) return false;
    PerRequest& req = ensure_request(request_id);
    if (req.page_state && req.page_state->total_tokens() > 0) return false;
    if (!req.page_state) {
        req.page_state.reset(new RequestKVState());
        req.page_state->request_id = request_id;
        req.page_state->page_size_tokens = page_size_tokens_;
    }
    if (!req.page_state->reserve(*pool_, tokens)) return false;
    req.next_position = tokens;
    return true;
}

void PagedAttentionExecutor::release_request(uint32_t request_id) {
    auto it = requests_.find(request_id);
    if (it == requests_.end()) return;
    if (pool_ && it->second.page_state) it->second.page_state->release_all(*pool_);  // batched_executor.cpp:38-45
    requests_.erase(it);
}

void PagedAttentionExecutor::reset() {
    if (pool_)
        for (auto& kv : requests_)
            if (kv.second.page_state) kv.second.page_state->release_all(*pool_);
    requests_.clear();
}

BatchedDecodeOutput PagedAttentionExecutor::run_decode(const std::vector<RequestSlot>& slots) {
    BatchedDecodeOutput out;
    if (slots.empty()) return out;
    if (!storage_ || !pool_) {  // nothing attached: every slot fails (batched_walker.cpp:87-95)
        for (const auto& s : slots) {
            BatchedDecodeOutput::PerRequest p;
            p.request_id = s.request_id;
            out.per_request.push_back(std::move(p));
        }
        return out;
    }
    return walker_->step(slots);
}

BatchedDecodeOutput PagedAttentionExecutor::run_decode_into(const std::vector<RequestSlot>& slots, float* logits, size_t stride) {
    if (slots.empty() || !storage_ || !pool_ || !model_) return run_decode(slots);
    BatchedWalker::LogitsSink sink;
    sink.dst = logits;
    sink.stride = stride;
    return walker_->step(slots, &sink);
}

bool PagedAttentionExecutor::run_decode_greedy(const std::vector<RequestSlot>& slots, std::vector<uint64_t>& tokens) {
    // only the whole model step in the fused order ends in logits on the device
    if (slots.empty() || !storage_ || !pool_ || !model_ || order_ != CallOrder::Fused) return false;
    tokens.clear();
    const BatchedDecodeOutput out = walker_->step(slots, nullptr, &tokens);
    if (tokens.size() != slots.size() || out.per_request.size() != slots.size()) {
        tokens.assign(slots.size(), UINT64_MAX);   // the pass ran and failed (pool exhausted, bad token): every slot failed
        return true;
    }
    for (size_t i = 0; i < slots.size(); ++i)
        if (!out.per_request[i].success) tokens[i] = UINT64_MAX;
    return true;
}

size_t PagedAttentionExecutor::logits_per_request() const {
    return model_ ? model_->vocab_size : static_cast<size_t>(H_) * D_;
}

bool PagedAttentionExecutor::attach_model(const ModelWeights& m) {
    if (m.layers.size() != L_ || !m.hidden_size || !m.ffn_inner || !m.vocab_size) return false;
    if (m.hidden_size != H_ * D_ || m.hidden_size % 256 || m.ffn_inner % 256) return false;
    if (m.rotary_dim > D_ || m.rotary_dim % 2) return false;
    if (!m.token_embd || !m.output_norm || !m.lm_head) return false;
    for (const auto& l : m.layers)
        if (!l.attn_norm || !l.attn_qkv || !l.attn_output || !l.ffn_norm || !l.ffn_gate_up || !l.ffn_down) return false;
    model_.reset(new ModelWeights(m));
    return true;
}

std::vector<float> PagedAttentionExecutor::run_prefill(uint32_t request_id, const std::vector<uint64_t>& tokens) {
    // With paged storage the reference fills the pages token by token through the decode
    // path (batched_executor.cpp:450-467); that loop is kept for the reference call order.
    // The default feeds the whole chunk at once: scatter of its K/V rows, then chunked causal
    // attention (tcgen05 kernel for head_dim 128 / 64-token pages); with a model attached, the whole step
    // for 32 prompt tokens per pass.
    std::vector<float> last;
    if (tokens.empty()) return last;
    size_t cursor = known_position(request_id);
    if (order_ == CallOrder::Fused && storage_ && pool_ && !model_) return walker_->prefill(request_id, tokens, cursor);
    if (order_ == CallOrder::Fused && storage_ && pool_ && model_) return walker_->prefill_model(request_id, tokens, cursor);
    for (uint64_t tok : tokens) {
        std::vector<RequestSlot> slot{{request_id, tok, cursor}};
        BatchedDecodeOutput out = run_decode(slot);
        if (out.per_request.empty() || !out.per_request.front().success) return {};
        last = std::move(out.per_request.front().logits);
        ++cursor;
    }
    return last;
}

}  // namespace runtime
}  // namespace mlcb
