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
    BatchedDecodeOutput step(const std::vector<RequestSlot>& slots);

private:
    PagedAttentionExecutor& exec_;
    // host staging, reused across passes
    std::vector<float> q_host_;
    std::vector<uint16_t> k_host_, v_host_;
    std::vector<float> o_host_;
};

}  // namespace runtime
}  // namespace mlcb
