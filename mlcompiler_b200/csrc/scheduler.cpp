// See scheduler.hpp. The behaviour is pinned by the reference's scheduler tests
// (tests/test_scheduler.cpp:64-187: one prefill and max_new_tokens - 1 decodes per request, never more
// than max_batch_size active, EOS at the first token means no decode, vacancies refill) and by its tick
// order (compiler/runtime/scheduler.cpp:152-165: admit, prefill, decode, reap). What is added is the
// chunked admission of prompts.
#include "scheduler.hpp"

#include <algorithm>

namespace mlcb {
namespace runtime {

namespace {

bool finished(const Scheduler::Request& r) {
    return r.state == Scheduler::State::Complete || r.state == Scheduler::State::Failed;
}

void fail(Scheduler::Request& r, const char* why) {
    r.state = Scheduler::State::Failed;
    r.failure_reason = why;
}

}  // namespace

Scheduler::Scheduler(IBatchedExecutor* executor, size_t max_batch_size)
    : executor_(executor), max_batch_size_(max_batch_size ? max_batch_size : 1) {}

uint32_t Scheduler::add_request(std::vector<uint64_t> prompt_tokens, GenerationParams params) {
    queued_.emplace_back();
    Request& req = queued_.back();
    req.id = next_id_++;
    req.prompt_tokens = std::move(prompt_tokens);
    req.params = params;
    return req.id;
}

uint64_t Scheduler::argmax(const std::vector<float>& logits) {
    size_t best = 0;
    for (size_t i = 1; i < logits.size(); ++i)
        if (logits[i] > logits[best]) best = i;   // the first maximum wins, like std::max_element
    return best;
}

void Scheduler::accept_token(Request& req, uint64_t tok) {
    req.last_token = tok;
    req.generated_tokens.push_back(tok);
    ++stats_.total_tokens_generated;
    if (token_cb_) token_cb_(req.id, tok);
    const bool hit_eos = req.params.eos_token_id >= 0 && tok == static_cast<uint64_t>(req.params.eos_token_id);
    const bool budget_spent = req.generated_tokens.size() >= req.params.max_new_tokens;
    if (hit_eos || budget_spent) req.state = State::Complete;
}

// FIFO: the oldest waiting requests take the free places of the batch.
void Scheduler::admit_new() {
    const size_t room = max_batch_size_ > active_.size() ? max_batch_size_ - active_.size() : 0;
    const size_t n = std::min(room, queued_.size());
    for (size_t i = 0; i < n; ++i) {
        active_.push_back(std::move(queued_.front()));
        queued_.pop_front();
        Request& req = active_.back();
        req.state = req.prompt_tokens.empty() ? State::Decoding : State::Prefilling;
    }
}

// One request per tick gets prompt tokens, the first one in the batch that still has some: the whole
// prompt (the reference, scheduler.cpp:47-81), or at most prefill_chunk_tokens_ of it, so that the decode
// pass of the other requests is never more than one chunk away. The executor continues a request's
// prefill from the position it has reached (batched_executor.cpp:445-467 starts at known_position).
void Scheduler::prefill_one_active() {
    for (Request& req : active_) {
        if (req.state != State::Prefilling) continue;
        const size_t total = req.prompt_tokens.size();
        const size_t done = req.position;                    // prompt tokens already fed
        const size_t take = prefill_chunk_tokens_ ? std::min(prefill_chunk_tokens_, total - done) : total - done;
        std::vector<float> logits;
        if (done == 0 && take == total) {
            logits = executor_->run_prefill(req.id, req.prompt_tokens);
        } else {
            const std::vector<uint64_t> chunk(req.prompt_tokens.begin() + static_cast<std::ptrdiff_t>(done),
                                              req.prompt_tokens.begin() + static_cast<std::ptrdiff_t>(done + take));
            logits = executor_->run_prefill(req.id, chunk);
        }
        ++stats_.total_prefill_calls;
        if (logits.empty()) {
            fail(req, "prefill failed");
            return;
        }
        req.position = done + take;
        if (req.position == total) {                         // the prompt is in: its last logits give the first token
            req.state = State::Decoding;
            accept_token(req, argmax(logits));
        }
        return;
    }
}

// One batched pass for every request that is decoding and still has budget.
void Scheduler::decode_active() {
    std::vector<RequestSlot> slots;
    std::vector<Request*> who;
    for (Request& req : active_) {
        if (req.state != State::Decoding) continue;
        if (req.generated_tokens.size() >= req.params.max_new_tokens) {
            req.state = State::Complete;
            continue;
        }
        slots.push_back(RequestSlot{req.id, req.last_token, req.position});
        who.push_back(&req);
    }
    if (slots.empty()) return;
    // an executor that samples greedily itself hands back token ids instead of logits
    std::vector<uint64_t> sampled;
    if (executor_->run_decode_greedy(slots, sampled)) {
        ++stats_.total_decode_steps;
        if (sampled.size() != slots.size()) {
            for (Request* req : who) fail(*req, "decode output size mismatch");
            return;
        }
        for (size_t i = 0; i < who.size(); ++i) {
            if (sampled[i] == UINT64_MAX) {
                fail(*who[i], "decode failed");
                continue;
            }
            ++who[i]->position;
            accept_token(*who[i], sampled[i]);
        }
        return;
    }
    const BatchedDecodeOutput out = executor_->run_decode(slots);
    ++stats_.total_decode_steps;
    if (out.per_request.size() != slots.size()) {
        for (Request* req : who) fail(*req, "decode output size mismatch");
        return;
    }
    for (size_t i = 0; i < who.size(); ++i) {
        const BatchedDecodeOutput::PerRequest& res = out.per_request[i];
        if (!res.success || res.logits.empty()) {
            fail(*who[i], "decode failed");
            continue;
        }
        ++who[i]->position;
        accept_token(*who[i], argmax(res.logits));
    }
}

// Finished and failed requests leave the batch in arrival order; their pages go back to the pool.
void Scheduler::reap_completed() {
    std::vector<Request> keep;
    keep.reserve(active_.size());
    for (Request& req : active_) {
        if (!finished(req)) {
            keep.push_back(std::move(req));
            continue;
        }
        if (executor_) executor_->release_request(req.id);
        if (complete_cb_) complete_cb_(req);
        ++stats_.total_requests_completed;
        completed_.push_back(std::move(req));
    }
    active_.swap(keep);
}

bool Scheduler::tick() {
    const size_t active0 = active_.size(), steps0 = stats_.total_decode_steps, prefills0 = stats_.total_prefill_calls,
                 done0 = completed_.size();
    admit_new();
    const bool admitted = active_.size() > active0;
    prefill_one_active();
    decode_active();
    reap_completed();
    const bool progressed = admitted || stats_.total_decode_steps > steps0 || stats_.total_prefill_calls > prefills0 ||
                            completed_.size() > done0;
    return progressed || !empty();
}

size_t Scheduler::run_until_idle() {
    const size_t before = stats_.total_decode_steps;
    while (!empty() && tick()) {
    }
    return stats_.total_decode_steps - before;
}

std::vector<Scheduler::Request> Scheduler::drain_completed() {
    std::vector<Request> out;
    out.swap(completed_);
    return out;
}

}  // namespace runtime
}  // namespace mlcb
