// Harness around MLcompiler's own executor-CPU attention path.
//
// TEST INFRASTRUCTURE ONLY: linked into oracle/_ref/libref_attention.so by
// build_ref.py together with the reference's unmodified sources. The product
// library never links or loads this file.
//
// The harness builds the graph the reference's own unit test builds
// (tests/test_runtime.cpp:1659-1719): one CPU `Attention` node with inputs
// q / k_in / v_in, state tensors kv_k / kv_v of shape {KVH, ctx, D} and output
// attn_out. The state tensors carry metadata role="kv_cache", which makes
// ExecutionContext::ensureStateTensor store their rows as fp16
// (compiler/runtime/execution_context.cpp:132-176). ModelConfig.rotary_dim
// stays 0, so RunAttentionCPU applies no RoPE
// (compiler/runtime/attention_cpu.cpp:352-363).
//
// One step = setSequencePosition(pos), set q/k_in/v_in, ExecutionExecutor::run()
// -> CpuExecutionBackend::execute (operator_backend.cpp:887) -> RunAttentionCPU
// (attention_cpu.cpp:272): the new K/V row is written at `pos` through the
// reference's fp16 row writer, then every head attends over [0, pos].

#include "frontends/gguf_loader.hpp"
#include "runtime/attention_cpu.hpp"
#include "runtime/execution_context.hpp"
#include "runtime/execution_executor.hpp"
#include "runtime/execution_graph.hpp"
#include "runtime/operator_backend.hpp"
#include "runtime/quant_utils.hpp"
#include "runtime/quantization.hpp"
#include "runtime/session.hpp"
#include "runtime/tokenizer.hpp"
#include "runtime/float_convert.hpp"
#include "runtime/paged_kv.hpp"
#include "runtime/scheduler.hpp"

#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <fstream>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace {

using namespace mlc::runtime;

// Smallest file Session accepts: GGUF magic, version 1, one F32 [3,2] tensor.
std::string writeTinyGGUF() {
    static std::atomic<int> counter{0};
    std::string path = "/tmp/mlc_b200_oracle_" + std::to_string(getpid()) + "_" +
                       std::to_string(counter++) + ".gguf";
    std::ofstream f(path, std::ios::binary);
    auto u32 = [&](uint32_t v) { f.write(reinterpret_cast<const char*>(&v), 4); };
    auto u64 = [&](uint64_t v) { f.write(reinterpret_cast<const char*>(&v), 8); };
    auto str = [&](const std::string& s) { u64(s.size()); f.write(s.data(), s.size()); };
    u32(0x46554747); u32(1); u64(1); u64(0);
    str("linear.weight"); u32(2); u64(2); u32(3); u32(2); u32(0); u64(256);
    f.seekp(256, std::ios::beg);
    float w[6] = {1, 2, 3, 0, 1, 0.5f};
    f.write(reinterpret_cast<const char*>(w), sizeof(w));
    return path;
}

struct RefAttention {
    size_t H, KVH, D, ctx;
    std::string gguf_path;
    std::unique_ptr<Session> session;
    ExecutionGraph graph;
    std::unique_ptr<ExecutionContext> context;
    std::unique_ptr<ExecutionExecutor> executor;

    RefAttention(size_t h, size_t kvh, size_t d, size_t c) : H(h), KVH(kvh), D(d), ctx(c) {
        gguf_path = writeTinyGGUF();
        session = std::make_unique<Session>(gguf_path);
        graph.addTensor("q", {static_cast<int64_t>(H * D)}, mlc::ir::DataType::F32);
        graph.addTensor("k_in", {static_cast<int64_t>(KVH * D)}, mlc::ir::DataType::F32);
        graph.addTensor("v_in", {static_cast<int64_t>(KVH * D)}, mlc::ir::DataType::F32);
        std::vector<int64_t> cache_shape{static_cast<int64_t>(KVH), static_cast<int64_t>(ctx),
                                         static_cast<int64_t>(D)};
        for (const char* name : {"kv_k", "kv_v"}) {
            auto& t = graph.addTensor(name, cache_shape, mlc::ir::DataType::F32);
            t.is_state = true;
            t.metadata["role"] = "kv_cache";
        }
        graph.addTensor("attn_out", {static_cast<int64_t>(H * D)}, mlc::ir::DataType::F32);
        auto& attn = graph.addNode("attention", ExecOpType::Attention, {"q", "k_in", "v_in"},
                                   {"attn_out", "kv_k", "kv_v"}, BackendKind::CPU);
        attn.attributes["heads"] = static_cast<float>(H);
        attn.attributes["kv_heads"] = static_cast<float>(KVH);
        attn.attributes["head_dim"] = static_cast<float>(D);
        attn.annotations["kv_cache_k"] = "kv_k";
        attn.annotations["kv_cache_v"] = "kv_v";
        context = std::make_unique<ExecutionContext>(*session, &graph);
        executor = std::make_unique<ExecutionExecutor>(graph, nullptr, context.get());
    }
    ~RefAttention() { ::unlink(gguf_path.c_str()); }
};

}  // namespace

extern "C" {

void* ref_attn_create(size_t heads, size_t kv_heads, size_t head_dim, size_t context_length) {
    try {
        return new RefAttention(heads, kv_heads, head_dim, context_length);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ref_attn_create: %s\n", e.what());
        return nullptr;
    }
}

void ref_attn_destroy(void* h) { delete static_cast<RefAttention*>(h); }

// Storage dtype the reference chose for the cache rows (1 == GGML F16 expected).
int ref_attn_cache_dtype(void* h) {
    auto* r = static_cast<RefAttention*>(h);
    TensorStorage* s = r->context->tensorStorage("kv_k");
    return s ? static_cast<int>(s->dtype) : -1;
}

// Pre-load `n` history rows, given token-major as fp32 [n][KVH][D], through the
// reference's own row writer (quantizeRowFrom, quant_utils.cpp:120-131), into the
// reference cache layout [KVH][ctx][D].
int ref_attn_load_history(void* h, const float* k_hist, const float* v_hist, size_t n) {
    auto* r = static_cast<RefAttention*>(h);
    TensorStorage* ks = r->context->tensorStorage("kv_k");
    TensorStorage* vs = r->context->tensorStorage("kv_v");
    if (!ks || !vs || n > r->ctx) return -1;
    for (size_t t = 0; t < n; ++t) {
        for (size_t kv = 0; kv < r->KVH; ++kv) {
            size_t row = kv * r->ctx + t;
            const float* ksrc = k_hist + (t * r->KVH + kv) * r->D;
            const float* vsrc = v_hist + (t * r->KVH + kv) * r->D;
            quantizeRowFrom(ksrc, ks->dtype, r->D, ks->quant_version,
                            ks->raw_data.data() + row * ks->row_stride_bytes);
            quantizeRowFrom(vsrc, vs->dtype, r->D, vs->quant_version,
                            vs->raw_data.data() + row * vs->row_stride_bytes);
        }
    }
    return 0;
}

// One decode step through ExecutionExecutor::run(). q fp32 [H*D]; k_new / v_new
// fp32 [KVH*D] are written at `position`; out fp32 [H*D].
int ref_attn_decode(void* h, size_t position, const float* q, const float* k_new,
                    const float* v_new, float* out) {
    auto* r = static_cast<RefAttention*>(h);
    r->context->setSequencePosition(position);
    r->context->setTensor("q", std::vector<float>(q, q + r->H * r->D));
    r->context->setTensor("k_in", std::vector<float>(k_new, k_new + r->KVH * r->D));
    r->context->setTensor("v_in", std::vector<float>(v_new, v_new + r->KVH * r->D));
    auto res = r->executor->run();
    if (!res.success) return -1;
    const auto* o = r->context->getTensor("attn_out");
    if (!o || o->size() != r->H * r->D) return -2;
    std::memcpy(out, o->data(), o->size() * sizeof(float));
    return 0;
}

// Same step, calling RunAttentionCPU directly (no graph walk) - used for timing.
int ref_attn_decode_direct(void* h, size_t position, const float* q, const float* k_new,
                           const float* v_new, float* out) {
    auto* r = static_cast<RefAttention*>(h);
    r->context->setSequencePosition(position);
    std::vector<float> qv(q, q + r->H * r->D), kv(k_new, k_new + r->KVH * r->D),
        vv(v_new, v_new + r->KVH * r->D);
    auto res = RunAttentionCPU(r->graph.nodes().front(), r->context.get(), qv, kv, vv);
    if (!res.success) return -1;
    const auto* o = r->context->getTensor("attn_out");
    if (!o || o->size() != r->H * r->D) return -2;
    std::memcpy(out, o->data(), o->size() * sizeof(float));
    return 0;
}

// Raw fp16 bits of one cache row (kv_head, position) of K (which=0) or V (which=1).
int ref_attn_read_cache_row(void* h, int which, size_t kv_head, size_t position, uint16_t* dst) {
    auto* r = static_cast<RefAttention*>(h);
    TensorStorage* s = r->context->tensorStorage(which == 0 ? "kv_k" : "kv_v");
    if (!s || s->row_stride_bytes != r->D * 2) return -1;
    size_t row = kv_head * r->ctx + position;
    std::memcpy(dst, s->raw_data.data() + row * s->row_stride_bytes, r->D * 2);
    return 0;
}

// fp16 <-> fp32 through the reference's scalar converters (float_convert.hpp:14-76).
float ref_fp16_to_float(uint16_t h) { return fp16ToFloat(h); }
uint16_t ref_float_to_fp16(float v) { return floatToFp16(v); }

// ---- PagePool / RequestKVState (compiler/runtime/paged_kv.cpp:10-81) ----------
void* ref_pool_create(uint32_t capacity) { return new PagePool(capacity); }
void ref_pool_destroy(void* p) { delete static_cast<PagePool*>(p); }
int ref_pool_allocate(void* p, uint32_t* id) {
    auto r = static_cast<PagePool*>(p)->allocate();
    if (!r) return 0;
    *id = *r;
    return 1;
}
void ref_pool_release(void* p, uint32_t id) { static_cast<PagePool*>(p)->release(id); }
size_t ref_pool_in_use(void* p) { return static_cast<PagePool*>(p)->pages_in_use(); }
size_t ref_pool_free(void* p) { return static_cast<PagePool*>(p)->pages_free(); }

void* ref_kvstate_create(uint32_t page_size) {
    auto* s = new RequestKVState();
    s->page_size_tokens = page_size;
    return s;
}
void ref_kvstate_destroy(void* s) { delete static_cast<RequestKVState*>(s); }
int ref_kvstate_extend(void* s, void* pool, uint32_t* page, uint32_t* slot) {
    auto r = static_cast<RequestKVState*>(s)->extend_one_token(*static_cast<PagePool*>(pool));
    if (!r) return 0;
    *page = r->first;
    *slot = r->second;
    return 1;
}
int ref_kvstate_reserve(void* s, void* pool, size_t tokens) {
    return static_cast<RequestKVState*>(s)->reserve(*static_cast<PagePool*>(pool), tokens) ? 1 : 0;
}
size_t ref_kvstate_pages(void* s, uint32_t* out, size_t cap) {
    auto* st = static_cast<RequestKVState*>(s);
    for (size_t i = 0; i < st->page_table.size() && i < cap; ++i) out[i] = st->page_table[i];
    return st->page_table.size();
}
size_t ref_kvstate_total(void* s) { return static_cast<RequestKVState*>(s)->total_tokens(); }
void ref_kvstate_release(void* s, void* pool) {
    static_cast<RequestKVState*>(s)->release_all(*static_cast<PagePool*>(pool));
}

// computeRotaryCoefficients / applyRotaryEmbedding (compiler/runtime/quantization.cpp:773-823),
// the reference's own CPU code for the rotation batched_rope performs on the GPU.
size_t ref_compute_rotary(size_t position, size_t rotary_dim, float freq_base, float freq_scale,
                          float* cos_out, float* sin_out) {
    std::vector<float> c, s;
    computeRotaryCoefficients(position, rotary_dim, freq_base, freq_scale, c, s);
    for (size_t i = 0; i < c.size(); ++i) {
        cos_out[i] = c[i];
        sin_out[i] = s[i];
    }
    return c.size();
}
void ref_apply_rotary(float* data, const float* cos_in, const float* sin_in, size_t pairs, size_t head_dim,
                      size_t rotary_dim) {
    std::vector<float> c(cos_in, cos_in + pairs), s(sin_in, sin_in + pairs);
    applyRotaryEmbedding(data, c, s, head_dim, rotary_dim);
}


// ---- the other ops of the batched walker's step (compiler/runtime/batched_walker.cpp:248-297, 333-458),
// through the reference's own CPU code: quantised rows through quantization.cpp's row functions, RMSNorm /
// SiLU-mul / Add through CpuExecutionBackend nodes of a one-node graph (operator_backend.cpp:574-643, 645-886,
// 1144-1200).
void ref_dequant_q4_0(const uint8_t* src, size_t cols, float* dst) { dequantizeRowQ4_0(src, cols, 2, dst); }
float ref_dot_q4_0(const uint8_t* src, size_t cols, const float* vec) { return dotProductRowQ4_0(src, cols, 2, vec); }
size_t ref_row_size_q4_0(size_t cols) { return q4_0RowSize(cols, 2); }
void ref_dequant_q6_k(const uint8_t* src, size_t cols, float* dst) { dequantizeRowQ6_K(src, cols, dst); }
float ref_dot_q6_k(const uint8_t* src, size_t cols, const float* vec) { return dotProductRowQ6_K(src, cols, vec); }
size_t ref_row_size_q6_k(size_t cols) { return q6_kRowSize(cols); }

// One CPU node over fp32 vectors. kind 0: Norm (RMS) with `weight` (n floats, served from a one-tensor GGUF as
// the model parameter "norm.weight"); kind 1: FeedForward in its gate / up input form (SiLU(a) * b);
// kind 2: Add (a + b). Returns 0 on success.
int ref_elementwise_node(int kind, const float* a, const float* b_or_weight, size_t n, float* out) {
    static std::atomic<int> counter{0};
    std::string path = "/tmp/mlc_b200_oracle_ops_" + std::to_string(getpid()) + "_" + std::to_string(counter++) + ".gguf";
    try {
        {
            std::ofstream f(path, std::ios::binary);
            auto u32 = [&](uint32_t v) { f.write(reinterpret_cast<const char*>(&v), 4); };
            auto u64 = [&](uint64_t v) { f.write(reinterpret_cast<const char*>(&v), 8); };
            auto str = [&](const std::string& s) { u64(s.size()); f.write(s.data(), s.size()); };
            u32(0x46554747); u32(1); u64(1); u64(0);
            str("norm.weight"); u32(2); u64(2); u32(static_cast<uint32_t>(n)); u32(1); u32(0); u64(256);
            f.seekp(256, std::ios::beg);
            std::vector<float> w(n, 1.0f);
            if (kind == 0) w.assign(b_or_weight, b_or_weight + n);
            f.write(reinterpret_cast<const char*>(w.data()), static_cast<std::streamsize>(n * sizeof(float)));
        }
        Session session(path);
        ExecutionGraph graph;
        const std::vector<int64_t> shape{static_cast<int64_t>(n)};
        graph.addTensor("a", shape, mlc::ir::DataType::F32);
        graph.addTensor("b", shape, mlc::ir::DataType::F32);
        graph.addTensor("y", shape, mlc::ir::DataType::F32);
        if (kind == 0) {
            auto& node = graph.addNode("norm", ExecOpType::Norm, {"a"}, {"y"}, BackendKind::CPU);
            node.annotations["weight"] = "norm.weight";
        } else if (kind == 1) {
            graph.addNode("ffn", ExecOpType::FeedForward, {"a", "b"}, {"y"}, BackendKind::CPU);
        } else {
            graph.addNode("add", ExecOpType::Add, {"a", "b"}, {"y"}, BackendKind::CPU);
        }
        ExecutionContext context(session, &graph);
        context.setTensor("a", std::vector<float>(a, a + n));
        if (kind != 0) context.setTensor("b", std::vector<float>(b_or_weight, b_or_weight + n));
        ExecutionExecutor executor(graph, nullptr, &context);
        auto res = executor.run();
        ::unlink(path.c_str());
        if (!res.success) return -1;
        const auto* y = context.getTensor("y");
        if (!y || y->size() != n) return -2;
        std::memcpy(out, y->data(), n * sizeof(float));
        return 0;
    } catch (const std::exception& e) {
        ::unlink(path.c_str());
        std::fprintf(stderr, "ref_elementwise_node: %s\n", e.what());
        return -3;
    }
}

// ---- the reference's GGUF loader (compiler/frontends/gguf_loader.cpp), dumped in the product's format ----------
namespace {
using mlc::frontend::GGUFLoader;
using mlc::frontend::GGUFValue;
using mlc::frontend::GGUFValueType;

const char* ref_type_name(GGUFValueType t) {
    switch (t) {
        case GGUFValueType::UINT8: return "UINT8";
        case GGUFValueType::INT8: return "INT8";
        case GGUFValueType::UINT16: return "UINT16";
        case GGUFValueType::INT16: return "INT16";
        case GGUFValueType::UINT32: return "UINT32";
        case GGUFValueType::INT32: return "INT32";
        case GGUFValueType::INT64: return "INT64";
        case GGUFValueType::UINT64: return "UINT64";
        case GGUFValueType::FLOAT32: return "FLOAT32";
        case GGUFValueType::FLOAT64: return "FLOAT64";
        case GGUFValueType::BOOL: return "BOOL";
        case GGUFValueType::STRING: return "STRING";
        case GGUFValueType::ARRAY: return "ARRAY";
        case GGUFValueType::RAW: return "RAW";
        default: return "?";
    }
}
void ref_json_string(std::string& out, const std::string& s) {
    out += '"';
    for (unsigned char ch : s) {
        if (ch == '"' || ch == '\\') { out += '\\'; out += static_cast<char>(ch); }
        else if (ch < 0x20) { char b[8]; std::snprintf(b, sizeof(b), "\\u%04x", ch); out += b; }
        else out += static_cast<char>(ch);
    }
    out += '"';
}
void ref_json_float(std::string& out, double f, bool single) {
    if (f != f) { out += "\"nan\""; return; }
    if (f - f != 0.0) { out += f > 0 ? "\"inf\"" : "\"-inf\""; return; }
    char b[40];
    std::snprintf(b, sizeof(b), single ? "%.9g" : "%.17g", f);
    out += b;
}
void ref_json_value(std::string& out, const GGUFValue& v) {
    switch (v.type) {
        case GGUFValueType::UINT8: out += std::to_string(std::get<uint8_t>(v.data)); break;
        case GGUFValueType::INT8: out += std::to_string(std::get<int8_t>(v.data)); break;
        case GGUFValueType::UINT16: out += std::to_string(std::get<uint16_t>(v.data)); break;
        case GGUFValueType::INT16: out += std::to_string(std::get<int16_t>(v.data)); break;
        case GGUFValueType::UINT32: out += std::to_string(std::get<uint32_t>(v.data)); break;
        case GGUFValueType::INT32: out += std::to_string(std::get<int32_t>(v.data)); break;
        case GGUFValueType::UINT64: out += std::to_string(std::get<uint64_t>(v.data)); break;
        case GGUFValueType::INT64: out += std::to_string(std::get<int64_t>(v.data)); break;
        case GGUFValueType::FLOAT32: ref_json_float(out, std::get<float>(v.data), true); break;
        case GGUFValueType::FLOAT64: ref_json_float(out, std::get<double>(v.data), false); break;
        case GGUFValueType::BOOL: out += std::get<bool>(v.data) ? "true" : "false"; break;
        case GGUFValueType::STRING: ref_json_string(out, std::get<std::string>(v.data)); break;
        case GGUFValueType::RAW: {
            out += '"';
            for (uint8_t ch : std::get<std::vector<uint8_t>>(v.data)) { char b[4]; std::snprintf(b, sizeof(b), "%02x", ch); out += b; }
            out += '"';
            break;
        }
        case GGUFValueType::ARRAY: {
            out += '[';
            const auto& arr = std::get<std::vector<GGUFValue>>(v.data);
            for (size_t i = 0; i < arr.size(); ++i) {
                if (i) out += ',';
                ref_json_value(out, arr[i]);
            }
            out += ']';
            break;
        }
        default: out += "null";
    }
}
}  // namespace

// Returns the bytes needed (with terminator), 0 if the loader threw; its message then goes to `json`.
size_t ref_gguf_describe(const char* path, int concatenate, char* json, size_t capacity) {
    std::string out;
    size_t ok = 1;
    try {
        GGUFLoader loader(path);
        loader.load();
        if (concatenate) loader.concatenateBlockWeights();
        std::map<std::string, const GGUFValue*> kv;
        for (const auto& e : loader.kvMetadata()) kv[e.first] = &e.second;
        std::map<std::string, const mlc::frontend::GGUFTensorInfo*> tensors;
        for (const auto& e : loader.tensors()) tensors[e.first] = &e.second;
        out = "{\"version\":" + std::to_string(loader.header().version) + ",\"n_tensors\":" + std::to_string(loader.header().n_tensors) +
              ",\"n_kv\":" + std::to_string(loader.header().n_kv) + ",\"quantization_version\":" + std::to_string(loader.quantizationVersion()) +
              ",\"kv\":{";
        bool first = true;
        for (const auto& e : kv) {
            if (!first) out += ',';
            first = false;
            ref_json_string(out, e.first);
            out += std::string(":{\"type\":\"") + ref_type_name(e.second->type) + "\"";
            if (e.second->type == GGUFValueType::ARRAY) {
                const auto& arr = std::get<std::vector<GGUFValue>>(e.second->data);
                // the loader keeps no element type for an empty array
                out += std::string(",\"elem_type\":\"") + (arr.empty() ? "?" : ref_type_name(arr[0].type)) + "\"";
            }
            out += ",\"value\":";
            ref_json_value(out, *e.second);
            out += '}';
        }
        out += "},\"tensors\":{";
        first = true;
        for (const auto& e : tensors) {
            if (!first) out += ',';
            first = false;
            ref_json_string(out, e.first);
            out += ":{\"shape\":[";
            for (size_t i = 0; i < e.second->shape.size(); ++i) {
                if (i) out += ',';
                out += std::to_string(e.second->shape[i]);
            }
            out += "],\"dtype\":" + std::to_string(e.second->dtype) + ",\"offset\":" +
                   (e.second->offset == UINT64_MAX ? std::string("-1") : std::to_string(e.second->offset)) +
                   ",\"n_bytes\":" + std::to_string(e.second->n_bytes) + "}";
        }
        out += "}}";
    } catch (const std::exception& e) {
        out = e.what();
        ok = 0;
    }
    if (json && capacity) {
        const size_t n = std::min(out.size(), capacity - 1);
        std::memcpy(json, out.data(), n);
        json[n] = 0;
    }
    return ok ? out.size() + 1 : 0;
}

// GGUFLoader::loadTensorData; returns n_bytes, -1 if the tensor is unknown or the loader threw.
long long ref_gguf_tensor(const char* path, const char* name, int concatenate, unsigned char* dst, size_t capacity) {
    try {
        GGUFLoader loader(path);
        loader.load();
        if (concatenate) loader.concatenateBlockWeights();
        auto it = loader.tensors().find(name);
        if (it == loader.tensors().end()) return -1;
        const std::vector<uint8_t> bytes = loader.loadTensorData(it->second);
        if (dst) std::memcpy(dst, bytes.data(), std::min(capacity, bytes.size()));
        return static_cast<long long>(bytes.size());
    } catch (const std::exception&) {
        return -1;
    }
}

// ---- the reference's tokenizer (compiler/runtime/tokenizer.cpp, its own BPE / unigram / greedy code) ----------
struct RefTokenizer {
    std::unique_ptr<mlc::frontend::GGUFLoader> loader;
    std::unique_ptr<mlc::runtime::Tokenizer> tok;
};
void* ref_tokenizer_create(const char* gguf_path) {
    try {
        auto t = std::make_unique<RefTokenizer>();
        t->loader = std::make_unique<mlc::frontend::GGUFLoader>(gguf_path);
        t->loader->load();
        t->tok = std::make_unique<mlc::runtime::Tokenizer>(*t->loader);
        return t.release();
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ref_tokenizer_create: %s\n", e.what());
        return nullptr;
    }
}
void ref_tokenizer_destroy(void* h) { delete static_cast<RefTokenizer*>(h); }
// valid, vocabulary size, bos, eos, unk (UINT64_MAX when unset)
void ref_tokenizer_info(void* h, unsigned long long* out5) {
    const auto& t = *static_cast<RefTokenizer*>(h)->tok;
    out5[0] = t.valid() ? 1 : 0;
    out5[1] = t.vocabSize();
    out5[2] = t.bosId();
    out5[3] = t.eosId();
    out5[4] = t.unkId();
}
size_t ref_tokenizer_encode(void* h, const char* text, size_t len, int add_bos, int add_eos, unsigned long long* ids,
                            size_t capacity) {
    mlc::runtime::TokenizerConfig cfg;
    cfg.add_bos = add_bos != 0;
    cfg.add_eos = add_eos != 0;
    const auto out = static_cast<RefTokenizer*>(h)->tok->encode(std::string(text, len), cfg);
    for (size_t i = 0; i < out.size() && i < capacity; ++i) ids[i] = out[i];
    return out.size();
}
size_t ref_tokenizer_decode(void* h, const unsigned long long* ids, size_t n, char* out, size_t capacity) {
    std::vector<uint64_t> v(ids, ids + n);
    const std::string s = static_cast<RefTokenizer*>(h)->tok->decode(v);
    if (out) std::memcpy(out, s.data(), std::min(capacity, s.size()));
    return s.size();
}
size_t ref_tokenizer_token_string(void* h, unsigned long long id, char* out, size_t capacity) {
    const std::string s = static_cast<RefTokenizer*>(h)->tok->tokenString(id);
    if (out) std::memcpy(out, s.data(), std::min(capacity, s.size()));
    return s.size();
}
int ref_tokenizer_flags(void* h, unsigned long long id) {
    const auto& t = *static_cast<RefTokenizer*>(h)->tok;
    return (t.isControlToken(id) ? 1 : 0) | (t.isEogToken(id) ? 2 : 0);
}

}  // extern "C"
