// Logical page allocation, per-request page tables and per-layer paged K/V storage.
//
// Same public surface as the reference's compiler/runtime/paged_kv.hpp:28-145
// (PagePool, RequestKVState, PagedKVStorage); the storage is backed by the CUDA
// context instead of Metal buffers. Single-threaded by contract, like the
// reference (paged_kv.hpp:25-27).
#pragma once

#include <cstddef>
#include <cstdint>
#include <optional>
#include <utility>
#include <vector>

struct mlc_ctx;

namespace mlcb {
namespace runtime {

// Fixed-capacity allocator of page ids. A fresh pool hands out 0, 1, 2, ...; a released
// id is the next one handed out again (LIFO). Page id 0 is valid; exhaustion is
// reported through std::optional / bool (paged_kv.hpp:28-53).
class PagePool {
public:
    explicit PagePool(uint32_t capacity);
    std::optional<uint32_t> allocate();
    // All or nothing: appends n ids to `out`, or leaves pool and `out` untouched.
    bool allocate_n(size_t n, std::vector<uint32_t>& out);
    // Returns false (and changes nothing) for an id outside the pool or with nothing in use;
    // the reference asserts in debug builds and is undefined in release builds.
    bool release(uint32_t page_id);
    uint32_t capacity() const { return capacity_; }
    size_t pages_in_use() const { return in_use_; }
    size_t pages_free() const { return stack_.size(); }

private:
    uint32_t capacity_;
    std::vector<uint32_t> stack_;  // top of the stack = next id handed out
    size_t in_use_ = 0;
};

// One request's ordered page list and fill level (paged_kv.hpp:65-97). The page ids are
// layer-agnostic: the same list indexes every layer's K and V pool.
struct RequestKVState {
    uint32_t request_id = 0;
    uint32_t page_size_tokens = 64;
    std::vector<uint32_t> page_table;
    uint32_t tokens_in_last_page = 0;

    size_t total_tokens() const {
        return page_table.empty() ? 0
                                  : (page_table.size() - 1) * static_cast<size_t>(page_size_tokens) + tokens_in_last_page;
    }
    bool reserve(PagePool& pool, size_t target_tokens);
    std::optional<std::pair<uint32_t, uint32_t>> extend_one_token(PagePool& pool);
    std::optional<std::pair<uint32_t, uint32_t>> locate(size_t pos) const;
    void release_all(PagePool& pool);
};

// Per-layer bulk K and V pools of capacity_pages * page_bytes each, zero-initialised
// (paged_kv.hpp:109-145, paged_kv.cpp:83-127). Page layout
// [page_size_tokens, n_kv_heads, head_dim] of dtype_bytes-wide elements.
class PagedKVStorage {
public:
    PagedKVStorage(mlc_ctx* ctx, uint32_t capacity_pages, uint32_t n_layers, uint32_t page_size_tokens,
                   uint32_t n_kv_heads, uint32_t head_dim, uint32_t dtype_bytes);
    ~PagedKVStorage();
    PagedKVStorage(const PagedKVStorage&) = delete;
    PagedKVStorage& operator=(const PagedKVStorage&) = delete;

    bool initialize();  // allocates and zero-fills; false when the device has no room
    void* k_buffer(size_t layer) const { return layer < k_.size() ? k_[layer] : nullptr; }
    void* v_buffer(size_t layer) const { return layer < v_.size() ? v_[layer] : nullptr; }
    uint32_t capacity_pages() const { return capacity_pages_; }
    uint32_t page_size_tokens() const { return page_size_tokens_; }
    uint32_t n_layers() const { return n_layers_; }
    uint32_t n_kv_heads() const { return n_kv_heads_; }
    uint32_t head_dim() const { return head_dim_; }
    uint32_t dtype_bytes() const { return dtype_bytes_; }
    size_t page_bytes() const {
        return static_cast<size_t>(page_size_tokens_) * n_kv_heads_ * head_dim_ * dtype_bytes_;
    }

private:
    mlc_ctx* ctx_;
    uint32_t capacity_pages_, n_layers_, page_size_tokens_, n_kv_heads_, head_dim_, dtype_bytes_;
    std::vector<void*> k_, v_;
};

}  // namespace runtime
}  // namespace mlcb
