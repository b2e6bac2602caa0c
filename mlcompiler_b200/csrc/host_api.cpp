// C ABI of the host-side objects: page pool, per-request page state, paged KV storage,
// paged-attention executor and scheduler (declared in include/mlc_b200.h).
#include <algorithm>
#include <cstring>
#include <string>
#include <memory>
#include <vector>

#include "../../include/mlc_b200.h"
#include "batched_executor.hpp"
#include "gguf_file.hpp"
#include "tokenizer.hpp"
#include "paged_kv.hpp"
#include "scheduler.hpp"

using namespace mlcb::runtime;

struct mlc_page_pool { PagePool pool; explicit mlc_page_pool(uint32_t c) : pool(c) {} };
struct mlc_kv_state { RequestKVState st; };
struct mlc_kv_storage { std::unique_ptr<PagedKVStorage> s; };

namespace {

// IBatchedExecutor over C callbacks (lets a host language provide the executor; tests use
// it for the mock executor of the reference's scheduler tests).
class CallbackExecutor : public IBatchedExecutor {
public:
    explicit CallbackExecutor(const mlc_executor_callbacks& cb) : cb_(cb) {}
    BatchedDecodeOutput run_decode(const std::vector<RequestSlot>& slots) override {
        std::vector<mlc_request_slot> in(slots.size());
        for (size_t i = 0; i < slots.size(); ++i)
            in[i] = {slots[i].request_id, slots[i].input_token, static_cast<uint64_t>(slots[i].sequence_position)};
        std::vector<mlc_decode_row> rows(slots.size());
        BatchedDecodeOutput out;
        const size_t n = cb_.run_decode ? cb_.run_decode(cb_.user, in.data(), in.size(), rows.data()) : 0;
        for (size_t i = 0; i < n && i < rows.size(); ++i) {
            BatchedDecodeOutput::PerRequest p;
            p.request_id = rows[i].request_id;
            p.success = rows[i].success != 0;
            if (p.success && rows[i].logits && rows[i].n_logits)
                p.logits.assign(rows[i].logits, rows[i].logits + rows[i].n_logits);
            out.per_request.push_back(std::move(p));
        }
        return out;
    }
    std::vector<float> run_prefill(uint32_t request_id, const std::vector<uint64_t>& tokens) override {
        const float* logits = nullptr;
        const size_t n = cb_.run_prefill ? cb_.run_prefill(cb_.user, request_id, tokens.data(), tokens.size(), &logits) : 0;
        return (n && logits) ? std::vector<float>(logits, logits + n) : std::vector<float>();
    }
    void release_request(uint32_t request_id) override {
        if (cb_.release_request) cb_.release_request(cb_.user, request_id);
    }

private:
    mlc_executor_callbacks cb_;
};

}  // namespace

struct mlc_executor {
    std::unique_ptr<IBatchedExecutor> exec;
    PagedAttentionExecutor* paged = nullptr;  // non-null when exec is the built-in one
};

struct mlc_gguf {
    std::unique_ptr<mlcb::gguf::File> file;
    std::string json;   // describe_json(), made on demand
};

struct mlc_tokenizer {
    explicit mlc_tokenizer(const mlcb::gguf::File& f) : tok(f) {}
    mlcb::text::Tokenizer tok;
};

struct mlc_scheduler {
    std::unique_ptr<Scheduler> sched;
    std::vector<Scheduler::Request> drained;
};

extern "C" {

// ---- PagePool ------------------------------------------------------------------------
mlc_page_pool* mlc_page_pool_create(uint32_t capacity) { return new mlc_page_pool(capacity); }
void mlc_page_pool_destroy(mlc_page_pool* p) { delete p; }
int mlc_page_pool_allocate(mlc_page_pool* p, uint32_t* page_id) {
    if (!p || !page_id) return 0;
    auto id = p->pool.allocate();
    if (!id) return 0;
    *page_id = *id;
    return 1;
}
int mlc_page_pool_allocate_n(mlc_page_pool* p, size_t n, uint32_t* out) {
    if (!p || (!out && n)) return 0;
    std::vector<uint32_t> ids;
    if (!p->pool.allocate_n(n, ids)) return 0;
    std::memcpy(out, ids.data(), n * sizeof(uint32_t));
    return 1;
}
int mlc_page_pool_release(mlc_page_pool* p, uint32_t page_id) { return p && p->pool.release(page_id) ? 1 : 0; }
uint32_t mlc_page_pool_capacity(const mlc_page_pool* p) { return p ? p->pool.capacity() : 0; }
size_t mlc_page_pool_in_use(const mlc_page_pool* p) { return p ? p->pool.pages_in_use() : 0; }
size_t mlc_page_pool_free(const mlc_page_pool* p) { return p ? p->pool.pages_free() : 0; }

// ---- RequestKVState ----------------------------------------------------------------------
mlc_kv_state* mlc_kv_state_create(uint32_t request_id, uint32_t page_size_tokens) {
    auto* s = new mlc_kv_state();
    s->st.request_id = request_id;
    s->st.page_size_tokens = page_size_tokens;
    return s;
}
void mlc_kv_state_destroy(mlc_kv_state* s) { delete s; }
int mlc_kv_state_reserve(mlc_kv_state* s, mlc_page_pool* p, size_t target_tokens) {
    return s && p && s->st.reserve(p->pool, target_tokens) ? 1 : 0;
}
int mlc_kv_state_extend_one_token(mlc_kv_state* s, mlc_page_pool* p, uint32_t* page_id, uint32_t* slot) {
    if (!s || !p) return 0;
    auto loc = s->st.extend_one_token(p->pool);
    if (!loc) return 0;
    if (page_id) *page_id = loc->first;
    if (slot) *slot = loc->second;
    return 1;
}
int mlc_kv_state_locate(const mlc_kv_state* s, size_t pos, uint32_t* page_id, uint32_t* slot) {
    if (!s) return 0;
    auto loc = s->st.locate(pos);
    if (!loc) return 0;
    if (page_id) *page_id = loc->first;
    if (slot) *slot = loc->second;
    return 1;
}
void mlc_kv_state_release_all(mlc_kv_state* s, mlc_page_pool* p) {
    if (s && p) s->st.release_all(p->pool);
}
size_t mlc_kv_state_total_tokens(const mlc_kv_state* s) { return s ? s->st.total_tokens() : 0; }
uint32_t mlc_kv_state_tokens_in_last_page(const mlc_kv_state* s) { return s ? s->st.tokens_in_last_page : 0; }
size_t mlc_kv_state_page_table(const mlc_kv_state* s, uint32_t* out, size_t capacity) {
    if (!s) return 0;
    const size_t n = s->st.page_table.size();
    if (out) std::memcpy(out, s->st.page_table.data(), std::min(n, capacity) * sizeof(uint32_t));
    return n;
}

// ---- PagedKVStorage -----------------------------------------------------------------------
mlc_kv_storage* mlc_kv_storage_create(mlc_ctx* ctx, uint32_t capacity_pages, uint32_t n_layers,
                                      uint32_t page_size_tokens, uint32_t n_kv_heads, uint32_t head_dim,
                                      uint32_t dtype_bytes) {
    auto* s = new mlc_kv_storage();
    s->s.reset(new PagedKVStorage(ctx, capacity_pages, n_layers, page_size_tokens, n_kv_heads, head_dim, dtype_bytes));
    return s;
}
void mlc_kv_storage_destroy(mlc_kv_storage* s) { delete s; }
int mlc_kv_storage_initialize(mlc_kv_storage* s) { return s && s->s->initialize() ? 1 : 0; }
void* mlc_kv_storage_k_buffer(const mlc_kv_storage* s, size_t layer) { return s ? s->s->k_buffer(layer) : nullptr; }
void* mlc_kv_storage_v_buffer(const mlc_kv_storage* s, size_t layer) { return s ? s->s->v_buffer(layer) : nullptr; }
size_t mlc_kv_storage_page_bytes(const mlc_kv_storage* s) { return s ? s->s->page_bytes() : 0; }

// ---- executors -------------------------------------------------------------------------------
mlc_executor* mlc_paged_executor_create(mlc_ctx* ctx, uint32_t num_heads, uint32_t kv_heads, uint32_t head_dim,
                                        uint32_t n_layers, uint64_t qkv_seed) {
    if (!ctx || !num_heads || !kv_heads || !head_dim || !n_layers || num_heads % kv_heads) return nullptr;
    auto* e = new mlc_executor();
    auto* paged = new PagedAttentionExecutor(ctx, num_heads, kv_heads, head_dim, n_layers,
                                             std::unique_ptr<IQkvSource>(new HashQkvSource(qkv_seed)));
    e->exec.reset(paged);
    e->paged = paged;
    return e;
}
mlc_executor* mlc_callback_executor_create(const mlc_executor_callbacks* callbacks) {
    if (!callbacks) return nullptr;
    auto* e = new mlc_executor();
    e->exec.reset(new CallbackExecutor(*callbacks));
    return e;
}
void mlc_executor_destroy(mlc_executor* e) { delete e; }
int mlc_executor_attach_page_pool(mlc_executor* e, mlc_page_pool* pool, uint32_t page_size_tokens) {
    if (!e || !e->paged) return MLC_ERR_INVALID_ARG;
    e->paged->attach_page_pool(pool ? &pool->pool : nullptr, page_size_tokens);
    return MLC_OK;
}
int mlc_executor_attach_paged_storage(mlc_executor* e, mlc_kv_storage* storage) {
    if (!e || !e->paged) return MLC_ERR_INVALID_ARG;
    e->paged->attach_paged_storage(storage ? storage->s.get() : nullptr);
    return MLC_OK;
}
int mlc_executor_attach_model(mlc_executor* e, const mlc_model_desc* d) {
    if (!e || !e->paged || !d || !d->layers) return MLC_ERR_INVALID_ARG;
    ModelWeights m;
    m.hidden_size = d->hidden_size;
    m.ffn_inner = d->ffn_inner;
    m.vocab_size = d->vocab_size;
    m.rotary_dim = d->rotary_dim;
    m.rope_base = d->rope_base;
    m.rope_scale = d->rope_scale;
    m.rms_epsilon = d->rms_epsilon > 0.0f ? d->rms_epsilon : 1e-5f;
    m.lm_head_quant = d->lm_head_quant;
    m.token_embd = static_cast<const uint8_t*>(d->token_embd);
    m.output_norm = static_cast<const float*>(d->output_norm);
    m.lm_head = static_cast<const uint8_t*>(d->lm_head);
    m.layers.resize(d->n_layers);
    for (uint32_t i = 0; i < d->n_layers; ++i) {
        const mlc_layer_weights& w = d->layers[i];
        m.layers[i] = {static_cast<const float*>(w.attn_norm), static_cast<const uint8_t*>(w.attn_qkv),
                       static_cast<const uint8_t*>(w.attn_output), static_cast<const float*>(w.ffn_norm),
                       static_cast<const uint8_t*>(w.ffn_gate_up), static_cast<const uint8_t*>(w.ffn_down)};
    }
    return e->paged->attach_model(m) ? MLC_OK : MLC_ERR_INVALID_ARG;
}
// ---- GGUF ----------------------------------------------------------------------------
static void copy_message(const std::string& what, char* error, size_t capacity) {
    if (!error || !capacity) return;
    const size_t n = std::min(what.size(), capacity - 1);
    std::memcpy(error, what.data(), n);
    error[n] = 0;
}
mlc_gguf* mlc_gguf_open(const char* path, char* error, size_t error_capacity) {
    if (error && error_capacity) error[0] = 0;
    if (!path) { copy_message("null path", error, error_capacity); return nullptr; }
    try {
        std::unique_ptr<mlc_gguf> g(new mlc_gguf);
        g->file.reset(new mlcb::gguf::File(path));
        return g.release();
    } catch (const std::exception& e) {
        copy_message(e.what(), error, error_capacity);
        return nullptr;
    }
}
void mlc_gguf_close(mlc_gguf* g) { delete g; }
int mlc_gguf_concatenate_block_weights(mlc_gguf* g, char* error, size_t error_capacity) {
    if (error && error_capacity) error[0] = 0;
    if (!g) return -1;
    try {
        g->json.clear();
        return static_cast<int>(g->file->concatenate_block_weights());
    } catch (const std::exception& e) {
        copy_message(e.what(), error, error_capacity);
        return -1;
    }
}
size_t mlc_gguf_describe(mlc_gguf* g, char* json, size_t capacity) {
    if (!g) return 0;
    try {
        if (g->json.empty()) g->json = g->file->describe_json();
    } catch (const std::exception&) {
        return 0;   // out of memory while building the text
    }
    if (json && capacity) {
        const size_t n = std::min(g->json.size(), capacity - 1);
        std::memcpy(json, g->json.data(), n);
        json[n] = 0;
    }
    return g->json.size() + 1;
}
int64_t mlc_gguf_tensor_data(mlc_gguf* g, const char* name, void* dst, size_t capacity, char* error, size_t error_capacity) {
    if (error && error_capacity) error[0] = 0;
    if (!g || !name) return -1;
    try {
        const mlcb::gguf::TensorInfo* t = g->file->find_tensor(name);
        if (!t) { copy_message(std::string("no tensor named ") + name, error, error_capacity); return -1; }
        const uint8_t* p = g->file->data(*t);
        if (dst) std::memcpy(dst, p, std::min<size_t>(capacity, t->n_bytes));
        return static_cast<int64_t>(t->n_bytes);
    } catch (const std::exception& e) {
        copy_message(e.what(), error, error_capacity);
        return -1;
    }
}
int mlc_executor_attach_gguf(mlc_executor* e, mlc_gguf* g, char* error, size_t error_capacity) {
    if (error && error_capacity) error[0] = 0;
    if (!e || !e->paged || !g) return MLC_ERR_INVALID_ARG;
    std::string what;
    g->json.clear();   // attaching may add the concatenated tensors
    if (e->paged->attach_gguf(*g->file, &what)) return MLC_OK;
    copy_message(what, error, error_capacity);
    return MLC_ERR_INVALID_ARG;
}

// ---- tokenizer -----------------------------------------------------------------------
mlc_tokenizer* mlc_tokenizer_create(mlc_gguf* g) {
    if (!g) return nullptr;
    try {
        return new mlc_tokenizer(*g->file);
    } catch (const std::exception&) {
        return nullptr;
    }
}
void mlc_tokenizer_destroy(mlc_tokenizer* t) { delete t; }
int mlc_tokenizer_info(const mlc_tokenizer* t, size_t* vocab_size, uint64_t* bos, uint64_t* eos, uint64_t* unk) {
    if (!t) return 0;
    if (vocab_size) *vocab_size = t->tok.vocab_size();
    if (bos) *bos = t->tok.bos();
    if (eos) *eos = t->tok.eos();
    if (unk) *unk = t->tok.unk();
    return t->tok.valid() ? 1 : 0;
}
size_t mlc_tokenizer_encode(const mlc_tokenizer* t, const char* text, size_t length, int add_bos, int add_eos, uint64_t* ids,
                            size_t capacity) {
    if (!t || (!text && length)) return 0;
    try {
        const std::vector<uint64_t> out = t->tok.encode(std::string(text ? text : "", length), add_bos != 0, add_eos != 0);
        for (size_t i = 0; ids && i < out.size() && i < capacity; ++i) ids[i] = out[i];
        return out.size();
    } catch (const std::exception&) {
        return 0;
    }
}
size_t mlc_tokenizer_decode(const mlc_tokenizer* t, const uint64_t* ids, size_t n, char* out, size_t capacity) {
    if (!t || (!ids && n)) return 0;
    try {
        const std::string s = t->tok.decode(ids, n);
        if (out) std::memcpy(out, s.data(), std::min(capacity, s.size()));
        return s.size();
    } catch (const std::exception&) {
        return 0;
    }
}
size_t mlc_tokenizer_token_string(const mlc_tokenizer* t, uint64_t id, char* out, size_t capacity) {
    if (!t) return 0;
    const std::string s = t->tok.token_string(id);
    if (out) std::memcpy(out, s.data(), std::min(capacity, s.size()));
    return s.size();
}
int mlc_tokenizer_token_flags(const mlc_tokenizer* t, uint64_t id) {
    if (!t) return 0;
    return (t->tok.is_control(id) ? 1 : 0) | (t->tok.is_eog(id) ? 2 : 0);
}

int mlc_executor_assume_context(mlc_executor* e, uint32_t request_id, size_t tokens) {
    if (!e || !e->paged) return MLC_ERR_INVALID_ARG;
    return e->paged->assume_context(request_id, tokens) ? MLC_OK : MLC_ERR_INVALID_ARG;
}
int mlc_executor_set_call_order(mlc_executor* e, int reference_order) {
    if (!e || !e->paged) return MLC_ERR_INVALID_ARG;
    e->paged->set_call_order(reference_order ? PagedAttentionExecutor::CallOrder::Reference
                                             : PagedAttentionExecutor::CallOrder::Fused);
    return MLC_OK;
}
size_t mlc_executor_run_decode(mlc_executor* e, const mlc_request_slot* slots, size_t n, uint8_t* success,
                               float* logits, size_t logits_stride) {
    if (!e || (!slots && n)) return 0;
    std::vector<RequestSlot> in(n);
    for (size_t i = 0; i < n; ++i)
        in[i] = {slots[i].request_id, slots[i].input_token, static_cast<size_t>(slots[i].sequence_position)};
    // with a model attached the logits go straight into the caller's rows (no per-request vectors in between)
    const bool into = e->paged && e->paged->has_model() && logits && logits_stride >= e->paged->logits_per_request();
    const BatchedDecodeOutput out = into ? e->paged->run_decode_into(in, logits, logits_stride) : e->exec->run_decode(in);
    for (size_t i = 0; i < out.per_request.size() && i < n; ++i) {
        if (success) success[i] = out.per_request[i].success ? 1 : 0;
        if (logits && out.per_request[i].success && !into)
            std::memcpy(logits + i * logits_stride, out.per_request[i].logits.data(),
                        std::min(logits_stride, out.per_request[i].logits.size()) * sizeof(float));
    }
    return out.per_request.size();
}
size_t mlc_executor_run_decode_greedy(mlc_executor* e, const mlc_request_slot* slots, size_t n, uint64_t* tokens) {
    if (!e || (!slots && n) || (!tokens && n)) return 0;
    std::vector<RequestSlot> in(n);
    for (size_t i = 0; i < n; ++i)
        in[i] = {slots[i].request_id, slots[i].input_token, static_cast<size_t>(slots[i].sequence_position)};
    std::vector<uint64_t> out;
    if (!e->exec->run_decode_greedy(in, out) || out.size() != n) return 0;
    std::memcpy(tokens, out.data(), n * sizeof(uint64_t));
    return n;
}
size_t mlc_executor_run_prefill(mlc_executor* e, uint32_t request_id, const uint64_t* tokens, size_t n,
                                float* logits, size_t capacity) {
    if (!e) return 0;
    const std::vector<float> out = e->exec->run_prefill(request_id, std::vector<uint64_t>(tokens, tokens + n));
    if (logits) std::memcpy(logits, out.data(), std::min(capacity, out.size()) * sizeof(float));
    return out.size();
}
void mlc_executor_release_request(mlc_executor* e, uint32_t request_id) {
    if (e) e->exec->release_request(request_id);
}
size_t mlc_executor_live_request_count(const mlc_executor* e) { return e && e->paged ? e->paged->live_request_count() : 0; }
size_t mlc_executor_known_position(const mlc_executor* e, uint32_t request_id) {
    return e && e->paged ? e->paged->known_position(request_id) : 0;
}
size_t mlc_executor_page_table(const mlc_executor* e, uint32_t request_id, uint32_t* out, size_t capacity,
                               size_t* total_tokens) {
    if (!e || !e->paged) return 0;
    const RequestKVState* st = e->paged->page_state(request_id);
    if (!st) return 0;
    if (total_tokens) *total_tokens = st->total_tokens();
    if (out) std::memcpy(out, st->page_table.data(), std::min(capacity, st->page_table.size()) * sizeof(uint32_t));
    return st->page_table.size();
}
float mlc_hash_qkv_value(uint64_t seed, uint32_t request, uint64_t token, uint64_t position, uint32_t layer,
                         uint32_t tensor, uint32_t index) {
    return HashQkvSource::value(seed, request, token, position, layer, tensor, index);
}

// ---- Scheduler -------------------------------------------------------------------------------
mlc_scheduler* mlc_scheduler_create(mlc_executor* e, size_t max_batch_size) {
    if (!e) return nullptr;
    auto* s = new mlc_scheduler();
    s->sched.reset(new Scheduler(e->exec.get(), max_batch_size));
    return s;
}
void mlc_scheduler_destroy(mlc_scheduler* s) { delete s; }
uint32_t mlc_scheduler_add_request(mlc_scheduler* s, const uint64_t* prompt_tokens, size_t n, size_t max_new_tokens,
                                   int64_t eos_token_id) {
    if (!s) return 0;
    GenerationParams p;
    p.max_new_tokens = max_new_tokens;
    p.eos_token_id = eos_token_id;
    return s->sched->add_request(std::vector<uint64_t>(prompt_tokens, prompt_tokens + n), p);
}
void mlc_scheduler_set_token_callback(mlc_scheduler* s, mlc_token_callback cb, void* user) {
    if (!s) return;
    if (cb) s->sched->set_token_callback([cb, user](uint32_t id, uint64_t tok) { cb(user, id, tok); });
    else s->sched->set_token_callback(nullptr);
}
void mlc_scheduler_set_prefill_chunk_tokens(mlc_scheduler* s, size_t tokens) {
    if (s) s->sched->set_prefill_chunk_tokens(tokens);
}
size_t mlc_scheduler_prefill_calls(const mlc_scheduler* s) { return s ? s->sched->stats().total_prefill_calls : 0; }
int mlc_scheduler_tick(mlc_scheduler* s) { return s && s->sched->tick() ? 1 : 0; }
size_t mlc_scheduler_run_until_idle(mlc_scheduler* s) { return s ? s->sched->run_until_idle() : 0; }
int mlc_scheduler_empty(const mlc_scheduler* s) { return !s || s->sched->empty() ? 1 : 0; }
size_t mlc_scheduler_queued_count(const mlc_scheduler* s) { return s ? s->sched->queued_count() : 0; }
size_t mlc_scheduler_active_count(const mlc_scheduler* s) { return s ? s->sched->active_count() : 0; }
size_t mlc_scheduler_completed_count(const mlc_scheduler* s) { return s ? s->sched->completed_count() : 0; }
void mlc_scheduler_stats(const mlc_scheduler* s, size_t* requests_completed, size_t* decode_steps,
                         size_t* tokens_generated) {
    if (!s) return;
    const SchedulerStats& st = s->sched->stats();
    if (requests_completed) *requests_completed = st.total_requests_completed;
    if (decode_steps) *decode_steps = st.total_decode_steps;
    if (tokens_generated) *tokens_generated = st.total_tokens_generated;
}
size_t mlc_scheduler_drain_completed(mlc_scheduler* s) {
    if (!s) return 0;
    s->drained = s->sched->drain_completed();
    return s->drained.size();
}
int mlc_scheduler_drained_request(const mlc_scheduler* s, size_t index, uint32_t* id, int* state,
                                  size_t* n_generated, uint64_t* generated, size_t capacity) {
    if (!s || index >= s->drained.size()) return 0;
    const Scheduler::Request& r = s->drained[index];
    if (id) *id = r.id;
    if (state) *state = static_cast<int>(r.state);
    if (n_generated) *n_generated = r.generated_tokens.size();
    if (generated)
        std::memcpy(generated, r.generated_tokens.data(), std::min(capacity, r.generated_tokens.size()) * sizeof(uint64_t));
    return 1;
}

}  // extern "C"
