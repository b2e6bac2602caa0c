// A decoder's weights out of a GGUF file into device memory, in the roles the batched walker reads them in.
// Tensor names and metadata keys are the reference's: token_embd.weight, blk.N.{attn_norm, attn_qkv, attn_output,
// ffn_norm, ffn_gate_up, ffn_down}.weight, output_norm.weight (batched_walker.cpp:183-190, 248-420), the fused
// attn_qkv / ffn_gate_up built by concatenation when the file stores q, k, v and gate, up apart
// (gguf_loader.cpp:877-943); llama.* keys with the fallbacks of kernel_scheduler.cpp:251-258.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

#include "batched_executor.hpp"
#include "ctx.hpp"
#include "gguf_file.hpp"

namespace mlcb {
namespace runtime {

namespace {

struct Wanted {
    const gguf::TensorInfo* info;
    std::function<void(const uint8_t*)> set;   // hands the device pointer to the model description
    size_t arena_offset;
};

constexpr size_t kArenaAlign = 256;
constexpr size_t kStageBytes = size_t(16) << 20;   // two page-locked staging halves of this size

}  // namespace

void PagedAttentionExecutor::release_model_arena() {
    if (!model_arena_) return;
    DeviceGuard guard(ctx_->device);
    cudaFree(model_arena_);
    model_arena_ = nullptr;
}

bool PagedAttentionExecutor::attach_gguf(gguf::File& file, std::string* error) {
    auto fail = [&](const std::string& what) {
        if (error) *error = what;
        return false;
    };
    try {
        file.concatenate_block_weights();
        auto meta_u = [&](std::initializer_list<const char*> keys, uint64_t fallback) {
            const gguf::Value* v = file.find_kv(keys);
            return v ? v->as_u64(fallback) : fallback;
        };
        auto meta_f = [&](std::initializer_list<const char*> keys, double fallback) {
            const gguf::Value* v = file.find_kv(keys);
            return v ? v->as_double(fallback) : fallback;
        };
        ModelWeights m;
        const uint64_t layers = meta_u({"llama.block_count", "llama.layers", "block_count", "n_layer", "num_hidden_layers"}, 0);
        const uint64_t heads = meta_u({"llama.attention.head_count", "attention.head_count", "num_attention_heads"}, 0);
        const uint64_t kv_heads = meta_u({"llama.attention.head_count_kv", "attention.head_count_kv"}, heads);
        m.hidden_size = static_cast<uint32_t>(meta_u({"llama.embedding_length", "llama.n_embd", "embedding_length", "n_embd"}, 0));
        if (layers != L_) return fail("the file has " + std::to_string(layers) + " blocks, the executor " + std::to_string(L_) + " layers");
        if (heads != H_ || kv_heads != KVH_)
            return fail("the file has " + std::to_string(heads) + " / " + std::to_string(kv_heads) + " heads, the executor " +
                        std::to_string(H_) + " / " + std::to_string(KVH_));
        if (m.hidden_size != H_ * D_) return fail("embedding_length does not equal head_count * head_dim of the executor");
        m.rotary_dim = static_cast<uint32_t>(meta_u({"llama.rope.dimension_count", "rope.dimension_count"}, D_));
        m.rope_base = static_cast<float>(meta_f({"llama.rope.freq_base", "rope.freq_base"}, 10000.0));
        m.rope_scale = static_cast<float>(meta_f({"llama.rope.freq_scale", "rope.freq_scale"}, 1.0));
        m.rms_epsilon = static_cast<float>(meta_f({"llama.attention.layer_norm_rms_epsilon", "attention.layer_norm_rms_epsilon"}, 1e-5));
        m.layers.resize(L_);

        std::vector<Wanted> wanted;
        size_t arena_bytes = 0;
        std::string missing;
        auto want = [&](const std::string& name, uint32_t dtype_a, uint32_t dtype_b, uint64_t cols, uint64_t rows, std::function<void(const uint8_t*)> set) {
            const gguf::TensorInfo* t = file.find_tensor(name);
            if (!t) { missing = name + " missing"; return false; }
            if (t->dtype != dtype_a && t->dtype != dtype_b) { missing = name + ": ggml type " + std::to_string(t->dtype) + " not supported in this role"; return false; }
            const uint64_t t_cols = t->shape.empty() ? 0 : t->shape[0], t_rows = t->shape.size() > 1 ? t->shape[1] : 1;
            if (t_cols != cols || (rows && t_rows != rows) || t->shape.size() > 2) { missing = name + ": unexpected shape"; return false; }
            file.data(*t);   // throws here, before anything is allocated, if the bytes are not in the file
            wanted.push_back({t, std::move(set), arena_bytes});
            arena_bytes += (static_cast<size_t>(t->n_bytes) + kArenaAlign - 1) / kArenaAlign * kArenaAlign;
            return true;
        };
        const uint64_t hidden = m.hidden_size, qkv_rows = static_cast<uint64_t>(H_ + 2 * KVH_) * D_;
        const gguf::TensorInfo* embd = file.find_tensor("token_embd.weight");
        if (!embd || embd->shape.size() != 2) return fail("token_embd.weight missing");
        m.vocab_size = static_cast<uint32_t>(embd->shape[1]);
        const gguf::TensorInfo* down0 = file.find_tensor("blk.0.ffn_down.weight");
        m.ffn_inner = static_cast<uint32_t>(meta_u({"llama.feed_forward_length", "feed_forward_length"},
                                                    down0 && !down0->shape.empty() ? down0->shape[0] : 0));
        const uint64_t inner = m.ffn_inner;
        bool ok = want("token_embd.weight", gguf::kGgmlQ4_0, gguf::kGgmlQ4_0, hidden, m.vocab_size, [&m](const uint8_t* d) { m.token_embd = d; }) &&
                  want("output_norm.weight", gguf::kGgmlF32, gguf::kGgmlF32, hidden, 0, [&m](const uint8_t* d) { m.output_norm = reinterpret_cast<const float*>(d); });
        // a file without output.weight shares the embedding table (tied weights)
        const gguf::TensorInfo* head = file.find_tensor("output.weight");
        if (ok && head) {
            ok = want("output.weight", gguf::kGgmlQ6_K, gguf::kGgmlQ4_0, hidden, m.vocab_size, [&m](const uint8_t* d) { m.lm_head = d; });
            m.lm_head_quant = head->dtype == gguf::kGgmlQ6_K ? 1 : 0;
        }
        for (uint32_t l = 0; ok && l < L_; ++l) {
            const std::string p = "blk." + std::to_string(l) + ".";
            LayerWeights* w = &m.layers[l];   // the callbacks run after this loop: they keep the pointer, not a reference to it
            ok = want(p + "attn_norm.weight", gguf::kGgmlF32, gguf::kGgmlF32, hidden, 0, [w](const uint8_t* d) { w->attn_norm = reinterpret_cast<const float*>(d); }) &&
                 want(p + "attn_qkv.weight", gguf::kGgmlQ4_0, gguf::kGgmlQ4_0, hidden, qkv_rows, [w](const uint8_t* d) { w->attn_qkv = d; }) &&
                 want(p + "attn_output.weight", gguf::kGgmlQ4_0, gguf::kGgmlQ4_0, hidden, hidden, [w](const uint8_t* d) { w->attn_output = d; }) &&
                 want(p + "ffn_norm.weight", gguf::kGgmlF32, gguf::kGgmlF32, hidden, 0, [w](const uint8_t* d) { w->ffn_norm = reinterpret_cast<const float*>(d); }) &&
                 want(p + "ffn_gate_up.weight", gguf::kGgmlQ4_0, gguf::kGgmlQ4_0, hidden, 2 * inner, [w](const uint8_t* d) { w->ffn_gate_up = d; }) &&
                 want(p + "ffn_down.weight", gguf::kGgmlQ4_0, gguf::kGgmlQ4_0, inner, hidden, [w](const uint8_t* d) { w->ffn_down = d; });
        }
        if (!ok) return fail(missing);

        // One device allocation for the model; the file streams through two page-locked staging halves so that
        // the copy of one piece runs while the next is read from the mapping.
        DeviceGuard guard(ctx_->device);
        void* arena = nullptr;
        if (cudaMalloc(&arena, std::max<size_t>(arena_bytes, kArenaAlign)) != cudaSuccess) {
            cudaGetLastError();
            return fail("cudaMalloc of " + std::to_string(arena_bytes) + " bytes for the weights failed");
        }
        ++ctx_->allocations;
        uint8_t* stage = nullptr;
        cudaEvent_t done[2] = {nullptr, nullptr};
        bool cuda_ok = cudaHostAlloc(reinterpret_cast<void**>(&stage), 2 * kStageBytes, cudaHostAllocDefault) == cudaSuccess &&
                       cudaEventCreateWithFlags(&done[0], cudaEventDisableTiming) == cudaSuccess &&
                       cudaEventCreateWithFlags(&done[1], cudaEventDisableTiming) == cudaSuccess;
        unsigned half = 0;
        bool used[2] = {false, false};
        for (size_t i = 0; cuda_ok && i < wanted.size(); ++i) {
            const uint8_t* src = file.data(*wanted[i].info);   // throws if the bytes are not in the file
            uint8_t* dst = static_cast<uint8_t*>(arena) + wanted[i].arena_offset;
            for (size_t off = 0; cuda_ok && off < wanted[i].info->n_bytes; off += kStageBytes, half ^= 1u) {
                const size_t n = std::min<size_t>(kStageBytes, wanted[i].info->n_bytes - off);
                if (used[half]) cuda_ok = cudaEventSynchronize(done[half]) == cudaSuccess;
                std::memcpy(stage + half * kStageBytes, src + off, n);
                cuda_ok = cuda_ok && cudaMemcpyAsync(dst + off, stage + half * kStageBytes, n, cudaMemcpyHostToDevice, ctx_->stream) == cudaSuccess &&
                          cudaEventRecord(done[half], ctx_->stream) == cudaSuccess;
                used[half] = true;
            }
            wanted[i].set(dst);
        }
        cuda_ok = cuda_ok && cudaStreamSynchronize(ctx_->stream) == cudaSuccess;
        if (stage) cudaFreeHost(stage);
        for (cudaEvent_t e : done)
            if (e) cudaEventDestroy(e);
        if (!cuda_ok) {
            cudaGetLastError();
            cudaFree(arena);
            return fail("copying the weights to the device failed");
        }
        if (!m.lm_head) {   // tied: the Q4_0 embedding rows serve as the lm_head
            m.lm_head = m.token_embd;
            m.lm_head_quant = 0;
        }
        if (!attach_model(m)) {
            cudaFree(arena);
            return fail("the model does not fit the executor (hidden and ffn sizes must be multiples of 256, rotary_dim even and <= head_dim)");
        }
        release_model_arena();
        model_arena_ = arena;
        return true;
    } catch (const std::exception& e) {
        return fail(e.what());
    }
}

}  // namespace runtime
}  // namespace mlcb
