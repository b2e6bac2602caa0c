// See scheduler.hpp. Tick order and stop rules follow compiler/runtime/scheduler.cpp:38-165.
#include "scheduler.hpp"

#include <algorithm>

namespace mlcb {
namespace runtime {

Scheduler::Scheduler(IBatchedExecutor* executor, size_t max_batch_size)
    : executor_(executor), max_batch_size_(max_batch_size ? max_batch_size : 1) {}

uint32_t Scheduler::add_request(std::vector<uint64_t> prompt_tokens, GenerationParams params) {
    Request req;
    req.id = next_id_++;
    req.prompt_tokens = std::move(prompt_tokens);
    req.params = params;
    queued_.push_back(std::move(req));
    return queued_.back().id;
}

uint64_t Scheduler::argmax(const std::vector<float>& logits) {
    return static_cast<uint64_t>(std::max_element(logits.begin(), logits.end()) - logits.begin());
}

void Scheduler::accept_token(Request& req, uint64_t tok) {
    req.last_token = tok;
    req.generated_tokens.push_back(tok);
    ++stats_.total_tokens_generated;
    if (token_cb_) token_cb_(req.id, tok);
    const bool eos = req.params.eos_token_id >= 0 && tok == static_cast<uint64_t>(req.params.eos_token_id);
    if (eos || req.generated_tokens.size() >= req.params.max_new_tokens) req.state = State::Complete;
}

void Scheduler::admit_new() {  // scheduler.cpp:38-45
    while (!queued_.empty() && active_.size() < max_batch_size_) {
        Request req = std::move(queued_.front());
        queued_.pop_front();
        req.state = req.prompt_tokens.empty() ? State::Decoding : State::Prefilling;
        active_.push_back(std::move(req));
    }
}

void Scheduler::prefill_one_active() {  // scheduler.cpp:47-81: at most one request per tick
    auto it = std::find_if(active_.begin(), active_.end(),
                           [](const Request& r) { return r.state == State::Prefilling; });
    if (it == active_.end()) return;
    Request& req = *it;
    if (req.prompt_tokens.empty()) {
        req.state = State::Decoding;
        return;
    }
    const std::vector<float> logits = executor_->run_prefill(req.id, req.prompt_tokens);
    if (logits.empty()) {
        req.state = State::Failed;
        req.failure_reason = "prefill failed";
        return;
    }
    req.position = req.prompt_tokens.size();  // every prompt token has been consumed
    req.state = State::Decoding;
    accept_token(req, argmax(logits));  // the first generated token comes from the prefill
}

void Scheduler::decode_active() {  // scheduler.cpp:83-135
    std::vector<RequestSlot> slots;
    std::vector<size_t> index;
    for (size_t i = 0; i < active_.size(); ++i) {
        Request& req = active_[i];
        if (req.state != State::Decoding) continue;
        if (req.generated_tokens.size() >= req.params.max_new_tokens) {
            req.state = State::Complete;
            continue;
        }
        slots.push_back({req.id, req.last_token, req.position});
        index.push_back(i);
    }
    if (slots.empty()) return;
    const BatchedDecodeOutput out = executor_->run_decode(slots);
    ++stats_.total_decode_steps;
    if (out.per_request.size() != slots.size()) {
        for (size_t i : index) {
            active_[i].state = State::Failed;
            active_[i].failure_reason = "decode output size mismatch";
        }
        return;
    }
    for (size_t k = 0; k < index.size(); ++k) {
        Request& req = active_[index[k]];
        const auto& per = out.per_request[k];
        if (!per.success || per.logits.empty()) {
            req.state = State::Failed;
            req.failure_reason = "decode failed";
            continue;
        }
        ++req.position;
        accept_token(req, argmax(per.logits));
    }
}

void Scheduler::reap_completed() {  // scheduler.cpp:137-150: failed requests are reaped and released too
    auto done = [](const Request& r) { return r.state == State::Complete || r.state == State::Failed; };
    auto split = std::stable_partition(active_.begin(), active_.end(), [&](const Request& r) { return !done(r); });
    for (auto it = split; it != active_.end(); ++it) {
        if (executor_) executor_->release_request(it->id);
        if (complete_cb_) complete_cb_(*it);
        ++stats_.total_requests_completed;
        completed_.push_back(std::move(*it));
    }
    active_.erase(split, active_.end());
}

bool Scheduler::tick() {  // scheduler.cpp:152-165
    const size_t active_before = active_.size();
    admit_new();
    bool any = active_.size() > active_before;
    prefill_one_active();
    const size_t steps_before = stats_.total_decode_steps;
    decode_active();
    any = any || stats_.total_decode_steps > steps_before;
    const size_t completed_before = completed_.size();
    reap_completed();
    any = any || completed_.size() > completed_before;
    return any || !empty();
}

size_t Scheduler::run_until_idle() {
    const size_t before = stats_.total_decode_steps;
    while (!empty())
        if (!tick()) break;
    return stats_.total_decode_steps - before;
}

std::vector<Scheduler::Request> Scheduler::drain_completed() {
    std::vector<Request> out;
    out.swap(completed_);
    return out;
}

}  // namespace runtime
}  // namespace mlcb
