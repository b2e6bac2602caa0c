// FIFO continuous-batching scheduler: admit up to max_batch_size, prefill one request per
// tick (whole, or in chunks), one batched decode per tick, greedy arg-max sampling, stop on EOS
// or token budget, reap finished requests and release their pages. Same public surface and
// behaviour as the reference's compiler/runtime/scheduler.hpp:27-104 / scheduler.cpp:10-186; it
// depends on IBatchedExecutor only, so tests drive it with a mock.
#pragma once

#include <cstdint>
#include <deque>
#include <functional>
#include <string>
#include <vector>

#include "batched_executor.hpp"

namespace mlcb {
namespace runtime {

struct GenerationParams {
    size_t max_new_tokens = 100;
    int64_t eos_token_id = -1;  // -1: no EOS check
};

struct SchedulerStats {
    size_t total_requests_completed = 0;
    size_t total_decode_steps = 0;
    size_t total_tokens_generated = 0;
    size_t total_prefill_calls = 0;   // run_prefill calls (one per prompt, or one per chunk)
};

class Scheduler {
public:
    enum class State { Queued, Prefilling, Decoding, Complete, Failed };

    struct Request {
        uint32_t id = 0;
        std::vector<uint64_t> prompt_tokens;
        GenerationParams params;
        State state = State::Queued;
        std::vector<uint64_t> generated_tokens;
        size_t position = 0;      // next sequence position to feed (while prefilling: prompt tokens fed so far)
        uint64_t last_token = 0;  // most recently sampled token
        std::string failure_reason;
    };

    using TokenCallback = std::function<void(uint32_t request_id, uint64_t token)>;
    using CompleteCallback = std::function<void(const Request& req)>;

    explicit Scheduler(IBatchedExecutor* executor, size_t max_batch_size = 8);

    uint32_t add_request(std::vector<uint64_t> prompt_tokens, GenerationParams params);
    void set_token_callback(TokenCallback cb) { token_cb_ = std::move(cb); }
    void set_complete_callback(CompleteCallback cb) { complete_cb_ = std::move(cb); }
    // Chunked admission: a prompt is fed at most `tokens` at a time, one chunk per tick, with the batch's
    // decode pass running every tick in between (0, the default, feeds a prompt whole in one tick like the
    // reference, scheduler.cpp:47-81, where a long prompt holds every decoding request up for its duration).
    void set_prefill_chunk_tokens(size_t tokens) { prefill_chunk_tokens_ = tokens; }
    size_t prefill_chunk_tokens() const { return prefill_chunk_tokens_; }

    size_t run_until_idle();  // returns the number of decode steps it ran
    bool tick();              // admit + prefill one + decode once + reap

    bool empty() const { return queued_.empty() && active_.empty(); }
    size_t queued_count() const { return queued_.size(); }
    size_t active_count() const { return active_.size(); }
    size_t completed_count() const { return completed_.size(); }
    const SchedulerStats& stats() const { return stats_; }
    std::vector<Request> drain_completed();

private:
    void admit_new();
    void prefill_one_active();
    void decode_active();
    void reap_completed();
    // Records a sampled token and decides whether the request goes on.
    void accept_token(Request& req, uint64_t tok);
    static uint64_t argmax(const std::vector<float>& logits);

    IBatchedExecutor* executor_;
    size_t max_batch_size_;
    size_t prefill_chunk_tokens_ = 0;
    std::deque<Request> queued_;
    std::vector<Request> active_;
    std::vector<Request> completed_;
    TokenCallback token_cb_;
    CompleteCallback complete_cb_;
    uint32_t next_id_ = 1;
    SchedulerStats stats_;
};

}  // namespace runtime
}  // namespace mlcb
