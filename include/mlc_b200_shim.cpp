// MetalExecutor on libmlc_b200.so: the MLcompiler-side binding of this library.
//
// MLcompiler has no plugin or FFI layer; its batched walker calls member functions of the
// singleton mlc::runtime::MetalExecutor (compiler/runtime/metal_runtime.hpp:23-711). This file
// defines that class's paged-attention members - same signatures, same bool returns, same
// argument rules - on top of the C ABI in mlc_b200.h, so that callers written against the
// reference header (BatchedWalker::step, PagedKVStorage, the paged-KV tests) compile and link
// unchanged. It is compiled against the reference's own header:
//
//   g++ -std=c++17 -I<MLcompiler> -I<MLcompiler>/compiler -I<this repo>/include -c mlc_b200_shim.cpp
//   and link with mlcompiler_b200/libmlc_b200.so
//
// Also defined: the other encode* ops of the walker's decode step (batched RMSNorm, Q4_0 / Q6_K batched
// mat-vec, add, SiLU * up). Members outside that step (single-vector mat-vecs, MPS attention, layer norm ...)
// are not defined here; a build that keeps using them links its own definitions of those.
//
// MLC_B200_SHIM_DEVICE (environment, default 0) selects the CUDA device of the singleton.
#include <cstdint>
#include <cstdlib>
#include <string>
#include <unordered_set>

#include "runtime/metal_runtime.hpp"

#include "mlc_b200.h"

namespace mlc {
namespace runtime {

struct MetalExecutor::Impl {
    mlc_ctx* ctx = nullptr;
};

MetalExecutor::MetalExecutor() : impl_(new Impl) {
    const char* dev = std::getenv("MLC_B200_SHIM_DEVICE");
    if (mlc_ctx_create(dev && *dev ? std::atoi(dev) : 0, /*stream=*/nullptr, &impl_->ctx) != MLC_OK) impl_->ctx = nullptr;
}

MetalExecutor::~MetalExecutor() {
    if (impl_ && impl_->ctx) mlc_ctx_destroy(impl_->ctx);
}

MetalExecutor& MetalExecutor::Instance() {
    static MetalExecutor instance;
    return instance;
}

bool MetalExecutor::isAvailable() const { return impl_->ctx && mlc_ctx_available(impl_->ctx) != 0; }

// ---- pass bracketing (metal_runtime.hpp:181-192): one CUDA stream instead of one command buffer
bool MetalExecutor::beginForwardPassCB() const { return impl_->ctx && mlc_pass_begin(impl_->ctx) == MLC_OK; }
bool MetalExecutor::hasForwardPassCB() const { return impl_->ctx && mlc_pass_is_open(impl_->ctx) != 0; }
bool MetalExecutor::flushForwardPassCB() const { return impl_->ctx && mlc_pass_flush(impl_->ctx) == MLC_OK; }
// A Metal command buffer that was never committed can be dropped; work already enqueued on a CUDA
// stream cannot, so discarding a pass waits for it and ignores the outcome.
void MetalExecutor::discardForwardPassCB() const {
    if (impl_->ctx) mlc_pass_flush(impl_->ctx);
}

// ---- buffers (metal_runtime.hpp:693-703)
void* MetalExecutor::allocateScratchBuffer(size_t bytes) const { return impl_->ctx ? mlc_alloc(impl_->ctx, bytes) : nullptr; }
void MetalExecutor::releaseScratchBuffer(void* buffer) const {
    if (impl_->ctx) mlc_free(impl_->ctx, buffer);
}
void MetalExecutor::uploadToBuffer(void* buffer, const void* src, size_t bytes, size_t dst_offset) const {
    if (impl_->ctx) mlc_upload(impl_->ctx, buffer, src, bytes, dst_offset);
}
void MetalExecutor::downloadFromBuffer(const void* buffer, void* dst, size_t bytes, size_t src_offset) const {
    if (impl_->ctx) mlc_download(impl_->ctx, buffer, dst, bytes, src_offset);
}
void* MetalExecutor::getOrAllocCachedBuffer(const char* name, size_t bytes) const {
    return impl_->ctx ? mlc_cached_buffer(impl_->ctx, name, bytes) : nullptr;
}

// ---- KV writers and reader (metal_runtime.hpp:526-533, 619-626, 666-687)
bool MetalExecutor::encodeScatterKVPagedBatched(void* page_storage_buffer, const std::vector<uint32_t>& page_ids,
                                                const std::vector<uint32_t>& slots_in_page, size_t page_size_tokens,
                                                size_t n_kv_heads, size_t head_dim, size_t batch,
                                                const void* src_buffer) const {
    if (!impl_->ctx || page_ids.size() != batch || slots_in_page.size() != batch) return false;
    return mlc_encode_scatter_kv_paged_batched_f16(impl_->ctx, page_storage_buffer, page_ids.data(), slots_in_page.data(),
                                                   page_size_tokens, n_kv_heads, head_dim, batch, src_buffer,
                                                   /*capacity_pages=*/0) == MLC_OK;
}

bool MetalExecutor::scatterKVPagedBatched(void* page_storage_buffer, const std::vector<uint32_t>& page_ids,
                                          const std::vector<uint32_t>& slots_in_page, size_t page_size_tokens,
                                          size_t n_kv_heads, size_t head_dim, size_t batch, const void* src_buffer) const {
    if (!impl_->ctx || page_ids.size() != batch || slots_in_page.size() != batch) return false;   // metal_runtime.mm:7241-7243
    return mlc_run_scatter_kv_paged_batched_f16(impl_->ctx, page_storage_buffer, page_ids.data(), slots_in_page.data(),
                                                page_size_tokens, n_kv_heads, head_dim, batch, src_buffer,
                                                /*capacity_pages=*/0) == MLC_OK;
}

bool MetalExecutor::scatterKVPaged(void* page_storage_buffer, const std::vector<uint32_t>& page_table,
                                   size_t page_size_tokens, size_t n_kv_heads, size_t head_dim, size_t tokens,
                                   size_t start_slot, const void* src_buffer, size_t dtype_bytes) const {
    if (!impl_->ctx) return false;
    return mlc_run_scatter_kv_paged(impl_->ctx, page_storage_buffer, page_table.data(), page_table.size(), page_size_tokens,
                                    n_kv_heads, head_dim, tokens, start_slot, src_buffer, dtype_bytes,
                                    /*capacity_pages=*/0) == MLC_OK;
}

bool MetalExecutor::gatherKVPages(void* page_storage_buffer, const std::vector<uint32_t>& page_table,
                                  size_t page_size_tokens, size_t n_kv_heads, size_t head_dim, size_t num_tokens,
                                  void* dst_buffer, size_t dtype_bytes) const {
    if (!impl_->ctx) return false;
    return mlc_run_gather_kv_pages(impl_->ctx, page_storage_buffer, page_table.data(), page_table.size(), page_size_tokens,
                                   n_kv_heads, head_dim, num_tokens, dst_buffer, dtype_bytes,
                                   /*capacity_pages=*/0) == MLC_OK;
}

// ---- paged flash attention (metal_runtime.hpp:510-523, 645-658): fp32 Q and O as in the reference,
// scale 1/sqrt(head_dim) (metal_runtime.mm:7133) chosen by passing 0
static bool table_sizes_ok(const std::vector<uint32_t>& page_tables_flat, const std::vector<uint32_t>& page_table_offsets,
                           const std::vector<uint32_t>& seq_lens, const std::vector<uint32_t>& q_positions, size_t batch) {
    // metal_runtime.mm:7746-7749
    return page_table_offsets.size() == batch + 1 && seq_lens.size() == batch && q_positions.size() == batch &&
           page_tables_flat.size() >= page_table_offsets.back();
}

bool MetalExecutor::encodePagedFlashAttention(void* q_buf, void* k_pages_buf, void* v_pages_buf, void* o_buf,
                                              const std::vector<uint32_t>& page_tables_flat,
                                              const std::vector<uint32_t>& page_table_offsets,
                                              const std::vector<uint32_t>& seq_lens,
                                              const std::vector<uint32_t>& q_positions, size_t batch, size_t num_heads,
                                              size_t kv_heads, size_t head_dim, size_t page_size_tokens,
                                              bool apply_causal) const {
    if (!impl_->ctx || !table_sizes_ok(page_tables_flat, page_table_offsets, seq_lens, q_positions, batch)) return false;
    return mlc_encode_paged_flash_attention(impl_->ctx, q_buf, k_pages_buf, v_pages_buf, o_buf, page_tables_flat.data(),
                                            page_tables_flat.size(), page_table_offsets.data(), seq_lens.data(),
                                            q_positions.data(), batch, num_heads, kv_heads, head_dim, page_size_tokens,
                                            apply_causal ? 1 : 0, /*scale=*/0.f, MLC_F32, MLC_F32,
                                            /*capacity_pages=*/0) == MLC_OK;
}

bool MetalExecutor::runPagedFlashAttention(void* q_buffer, void* k_pages_buffer, void* v_pages_buffer, void* o_buffer,
                                           const std::vector<uint32_t>& page_tables_flat,
                                           const std::vector<uint32_t>& page_table_offsets,
                                           const std::vector<uint32_t>& seq_lens,
                                           const std::vector<uint32_t>& q_positions, size_t batch, size_t num_heads,
                                           size_t kv_heads, size_t head_dim, size_t page_size_tokens,
                                           bool apply_causal) const {
    if (!impl_->ctx || batch == 0 ||
        !table_sizes_ok(page_tables_flat, page_table_offsets, seq_lens, q_positions, batch)) return false;
    return mlc_run_paged_flash_attention(impl_->ctx, q_buffer, k_pages_buffer, v_pages_buffer, o_buffer,
                                         page_tables_flat.data(), page_tables_flat.size(), page_table_offsets.data(),
                                         seq_lens.data(), q_positions.data(), batch, num_heads, kv_heads, head_dim,
                                         page_size_tokens, apply_causal ? 1 : 0, /*scale=*/0.f, MLC_F32, MLC_F32,
                                         /*capacity_pages=*/0) == MLC_OK;
}

// ---- the step in front of the scatter (metal_runtime.hpp:540-547): one launch for the reference's seven dispatches
bool MetalExecutor::encodeQkvSplitRopeCast(void* qkv_buf, void* q_buf, void* k_buf, void* v_buf, void* k_f16_buf,
                                           void* v_f16_buf, void* cos_buf, void* sin_buf, size_t batch, size_t num_heads,
                                           size_t kv_heads, size_t head_dim, size_t qkv_rows, size_t q_rows,
                                           size_t k_rows, size_t v_rows, size_t rotary_dim) const {
    if (!impl_->ctx) return false;
    return mlc_encode_qkv_split_rope_cast(impl_->ctx, qkv_buf, q_buf, k_buf, v_buf, k_f16_buf, v_f16_buf, cos_buf, sin_buf,
                                          batch, num_heads, kv_heads, head_dim, qkv_rows, q_rows, k_rows, v_rows,
                                          rotary_dim) == MLC_OK;
}

// ---- the walker step's other ops (metal_runtime.hpp:474-506, 549-552)
// The reference keeps every weight it has seen in a device buffer keyed by the tensor's name and fills it
// on first use; the same here, on the library's name-keyed buffer cache.
static const void* cached_weight(mlc_ctx* ctx, const std::string& name, const void* host, size_t bytes) {
    static std::unordered_set<std::string> uploaded;
    void* dev = mlc_cached_buffer(ctx, name.c_str(), (bytes + 15) / 16 * 16);
    if (dev && uploaded.insert(name).second && mlc_upload(ctx, dev, host, bytes, 0) != MLC_OK) {
        uploaded.erase(name);
        return nullptr;
    }
    return dev;
}

bool MetalExecutor::encodeRmsNormBatched(void* in_buf, const std::vector<float>& weight, float epsilon, size_t batch,
                                         size_t length, void* out_buf) const {
    if (!impl_->ctx || weight.size() < length) return false;
    // norm weights carry no name in this call: key the cache on the host vector's address and length
    const std::string key = "rms_w@" + std::to_string(reinterpret_cast<uintptr_t>(weight.data())) + ":" + std::to_string(length);
    const void* w = cached_weight(impl_->ctx, key, weight.data(), length * sizeof(float));
    return w && mlc_encode_rms_norm_batched(impl_->ctx, in_buf, w, epsilon, batch, length, out_buf, nullptr) == MLC_OK;
}

bool MetalExecutor::encodeMatMulQ4_0Batched(const std::string& weight_name, const std::vector<uint8_t>& weights, void* in_buf,
                                            size_t batch, size_t rows, size_t cols, size_t row_stride,
                                            uint32_t /*quant_version*/, void* out_buf) const {
    if (!impl_->ctx || weights.size() < rows * row_stride) return false;
    const void* w = cached_weight(impl_->ctx, weight_name, weights.data(), rows * row_stride);
    return w && mlc_encode_matmul_q4_0_batched(impl_->ctx, w, in_buf, batch, rows, cols, row_stride, out_buf) == MLC_OK;
}

bool MetalExecutor::encodeMatMulQ6KBatched(const std::string& weight_name, const std::vector<uint8_t>& weights, void* in_buf,
                                           size_t batch, size_t rows, size_t cols, size_t row_stride, void* out_buf) const {
    if (!impl_->ctx || weights.size() < rows * row_stride) return false;
    const void* w = cached_weight(impl_->ctx, weight_name, weights.data(), rows * row_stride);
    return w && mlc_encode_matmul_q6k_batched(impl_->ctx, w, in_buf, batch, rows, cols, row_stride, out_buf) == MLC_OK;
}

bool MetalExecutor::encodeAddBatched(void* a_buf, void* b_buf, void* out_buf, size_t total_elements) const {
    return impl_->ctx && mlc_encode_add_batched(impl_->ctx, a_buf, b_buf, out_buf, total_elements) == MLC_OK;
}

bool MetalExecutor::encodeSiluMulBatched(void* gate_buf, void* up_buf, void* out_buf, size_t total_elements) const {
    return impl_->ctx && mlc_encode_silu_mul_batched(impl_->ctx, gate_buf, up_buf, out_buf, total_elements) == MLC_OK;
}

bool MetalExecutor::encodeGateUpSplitSiluMul(void* gate_up_buf, void* gate_buf, void* up_buf, void* out_buf, size_t batch,
                                             size_t ffn_inner, size_t ffn_gate_up_rows) const {
    return impl_->ctx && mlc_encode_gate_up_split_silu_mul(impl_->ctx, gate_up_buf, gate_buf, up_buf, out_buf, batch,
                                                           ffn_inner, ffn_gate_up_rows) == MLC_OK;
}

}  // namespace runtime
}  // namespace mlc
