// See paged_kv.hpp. Behaviour follows compiler/runtime/paged_kv.cpp:10-127.
#include "paged_kv.hpp"

#include <cuda_runtime.h>

#include "ctx.hpp"

namespace mlcb {
namespace runtime {

PagePool::PagePool(uint32_t capacity) : capacity_(capacity) {
    stack_.resize(capacity);
    // id 0 ends on top, so a fresh pool allocates in ascending order (paged_kv.cpp:10-17)
    for (uint32_t i = 0; i < capacity; ++i) stack_[i] = capacity - 1 - i;
}

std::optional<uint32_t> PagePool::allocate() {
    if (stack_.empty()) return std::nullopt;
    const uint32_t id = stack_.back();
    stack_.pop_back();
    ++in_use_;
    return id;
}

bool PagePool::allocate_n(size_t n, std::vector<uint32_t>& out) {
    if (n > stack_.size()) return false;
    out.insert(out.end(), stack_.rbegin(), stack_.rbegin() + static_cast<std::ptrdiff_t>(n));
    stack_.resize(stack_.size() - n);
    in_use_ += n;
    return true;
}

bool PagePool::release(uint32_t page_id) {
    if (page_id >= capacity_ || in_use_ == 0) return false;
    stack_.push_back(page_id);
    --in_use_;
    return true;
}

bool RequestKVState::reserve(PagePool& pool, size_t target_tokens) {
    if (page_size_tokens == 0) return false;
    const size_t needed = (target_tokens + page_size_tokens - 1) / page_size_tokens;
    if (needed <= page_table.size()) return true;  // never shrinks
    return pool.allocate_n(needed - page_table.size(), page_table);
}

std::optional<std::pair<uint32_t, uint32_t>> RequestKVState::extend_one_token(PagePool& pool) {
    if (page_size_tokens == 0) return std::nullopt;
    if (page_table.empty() || tokens_in_last_page == page_size_tokens) {
        const auto id = pool.allocate();
        if (!id) return std::nullopt;  // table unchanged
        page_table.push_back(*id);
        tokens_in_last_page = 0;
    }
    return std::make_pair(page_table.back(), tokens_in_last_page++);
}

std::optional<std::pair<uint32_t, uint32_t>> RequestKVState::locate(size_t pos) const {
    if (page_size_tokens == 0 || pos >= total_tokens()) return std::nullopt;
    return std::make_pair(page_table[pos / page_size_tokens], static_cast<uint32_t>(pos % page_size_tokens));
}

void RequestKVState::release_all(PagePool& pool) {
    for (uint32_t id : page_table) pool.release(id);
    page_table.clear();
    tokens_in_last_page = 0;
}

PagedKVStorage::PagedKVStorage(mlc_ctx* ctx, uint32_t capacity_pages, uint32_t n_layers,
                               uint32_t page_size_tokens, uint32_t n_kv_heads, uint32_t head_dim,
                               uint32_t dtype_bytes)
    : ctx_(ctx), capacity_pages_(capacity_pages), n_layers_(n_layers), page_size_tokens_(page_size_tokens),
      n_kv_heads_(n_kv_heads), head_dim_(head_dim), dtype_bytes_(dtype_bytes),
      k_(n_layers, nullptr), v_(n_layers, nullptr) {}

PagedKVStorage::~PagedKVStorage() {
    if (!ctx_) return;
    for (void* b : k_) if (b) mlc_free(ctx_, b);
    for (void* b : v_) if (b) mlc_free(ctx_, b);
}

bool PagedKVStorage::initialize() {
    if (!ctx_ || !mlc_ctx_available(ctx_)) return false;
    const size_t bytes = static_cast<size_t>(capacity_pages_) * page_bytes();
    if (bytes == 0) return false;
    DeviceGuard guard(ctx_->device);
    for (uint32_t layer = 0; layer < n_layers_; ++layer) {
        if (!k_[layer]) k_[layer] = mlc_alloc(ctx_, bytes);
        if (!v_[layer]) v_[layer] = mlc_alloc(ctx_, bytes);
        if (!k_[layer] || !v_[layer]) return false;
        // unread slots stay zero, like the reference's zero upload (paged_kv.cpp:112-117)
        if (cudaMemsetAsync(k_[layer], 0, bytes, ctx_->stream) != cudaSuccess) return false;
        if (cudaMemsetAsync(v_[layer], 0, bytes, ctx_->stream) != cudaSuccess) return false;
    }
    return cudaStreamSynchronize(ctx_->stream) == cudaSuccess;
}

}  // namespace runtime
}  // namespace mlcb
