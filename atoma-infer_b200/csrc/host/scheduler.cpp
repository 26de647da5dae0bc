#include "scheduler.hpp"

#include <algorithm>

namespace engine {

int64_t Scheduler::prompt_limit() const {
    // backends/vllm/src/scheduler.rs:2120-2128
    if (cfg_.enable_chunked_prefill) return cfg_.max_model_len;
    return std::min<int64_t>(cfg_.max_model_len, cfg_.max_num_batched_tokens);
}

int Scheduler::add_request(int64_t req, int64_t prompt_len) {
    if (reqs_.count(req)) return kErrDuplicate;
    if (prompt_len <= 0) return kErrArgument;
    Request r{req, prompt_len, 0, next_arrival_++, kWaiting, 0, 0};
    reqs_.emplace(req, r);
    waiting_.push_back(req);
    return kOk;
}

void Scheduler::insert_running(int64_t req) {
    int64_t a = reqs_[req].arrival;
    auto it = running_.begin();
    while (it != running_.end() && reqs_[*it].arrival < a) ++it;
    running_.insert(it, req);
}

void Scheduler::preempt(Request& r, StepPlan& plan) {
    if (cache_->has_request(r.id)) cache_->free_request(r.id);
    r.num_computed = 0;
    r.decoded = 0;
    r.planned = 0;
    r.status = kWaiting;
    plan.preempted.push_back(r.id);
    ++num_preemptions_;
}

bool Scheduler::schedule_running(StepPlan& plan, int& token_budget, bool chunk) {
    std::deque<int64_t> queue(running_.begin(), running_.end());
    std::vector<int64_t> kept, victims;
    while (!queue.empty()) {
        Request& r = reqs_[queue.front()];
        int64_t remaining = r.length - r.num_computed;
        int64_t want = remaining;
        if (chunk) want = std::min<int64_t>(want, token_budget);
        else if (want > token_budget) want = 0;
        if (want <= 0) {  // the budget is spent: the request keeps its place and waits a step
            kept.push_back(r.id);
            queue.pop_front();
            continue;
        }
        bool alive = true;
        for (;;) {
            int can = cache_->can_reserve(r.id, r.num_computed + want);
            if (can == kOk) break;
            if (can == kErrNever) {  // has outgrown the whole cache: it cannot go on
                cache_->free_request(r.id);
                plan.ignored.push_back(r.id);
                alive = false;
                break;
            }
            if (queue.size() > 1) {
                int64_t victim = queue.back();
                queue.pop_back();
                preempt(reqs_[victim], plan);
                victims.push_back(victim);
            } else {
                preempt(r, plan);
                victims.push_back(r.id);
                alive = false;
                break;
            }
        }
        int64_t id = queue.front();
        queue.pop_front();
        if (!alive) {
            if (reqs_[id].status != kWaiting) reqs_.erase(id);
            continue;
        }
        cache_->reserve(r.id, r.num_computed + want);
        r.planned = (int)want;
        plan.entries.push_back(StepEntry{r.id, r.num_computed, (int32_t)want,
                                         (int32_t)(r.num_computed + want == r.length), (int32_t)!r.decoded});
        planned_.push_back(r.id);
        token_budget -= (int)want;
        kept.push_back(r.id);
    }
    running_ = kept;
    // Victims return to the front of the waiting queue in their arrival order.
    std::sort(victims.begin(), victims.end(),
              [&](int64_t a, int64_t b) { return reqs_[a].arrival < reqs_[b].arrival; });
    for (auto it = victims.rbegin(); it != victims.rend(); ++it) waiting_.push_front(*it);
    return !victims.empty();
}

void Scheduler::schedule_waiting(StepPlan& plan, int& token_budget, bool chunk) {
    const int groups = cache_->num_groups();
    // Pages that running requests will still take to finish what they already know
    // of themselves (prompt portions not yet run): not to be given to newcomers.
    std::vector<int64_t> promised(groups, 0);
    for (int64_t id : running_) {
        const Request& r = reqs_[id];
        for (int g = 0; g < groups; ++g) {
            int n = cache_->pages_needed(id, g, r.length);
            if (n > 0) promised[g] += n;
        }
    }
    while (!waiting_.empty()) {
        Request& r = reqs_[waiting_.front()];
        if ((int)running_.size() >= cfg_.max_num_seqs) break;
        if (r.length > prompt_limit()) {
            plan.ignored.push_back(r.id);
            waiting_.pop_front();
            reqs_.erase(plan.ignored.back());
            continue;
        }
        int64_t want = r.length;
        if (chunk) want = std::min<int64_t>(want, token_budget);
        else if (want > token_budget) break;
        if (want <= 0) break;
        bool never = false, later = false;
        for (int g = 0; g < groups; ++g) {
            int n = cache_->pages_needed_new(g, r.length);
            if (n > cache_->num_usable_pages(g)) never = true;
            else if (n + promised[g] > cache_->num_free_pages(g)) later = true;
        }
        if (never) {
            plan.ignored.push_back(r.id);
            waiting_.pop_front();
            reqs_.erase(plan.ignored.back());
            continue;
        }
        if (later || cache_->num_free_slots() == 0) break;  // head of the line blocks the rest
        cache_->add_request(r.id);
        cache_->reserve(r.id, want);
        for (int g = 0; g < groups; ++g) promised[g] += std::max(0, cache_->pages_needed(r.id, g, r.length));
        r.status = kRunning;
        r.planned = (int)want;
        plan.entries.push_back(StepEntry{r.id, 0, (int32_t)want, (int32_t)(want == r.length), 1});
        planned_.push_back(r.id);
        token_budget -= (int)want;
        int64_t id = r.id;
        waiting_.pop_front();
        insert_running(id);
    }
}

StepPlan Scheduler::schedule() {
    StepPlan plan;
    planned_.clear();
    int budget = cfg_.max_num_batched_tokens;
    if (cfg_.enable_chunked_prefill) {
        bool preempted = schedule_running(plan, budget, true);
        if (!preempted) schedule_waiting(plan, budget, true);
    } else {
        schedule_waiting(plan, budget, false);
        if (plan.entries.empty()) schedule_running(plan, budget, false);
    }
    return plan;
}

void Scheduler::step_done() {
    for (int64_t id : planned_) {
        auto it = reqs_.find(id);
        if (it == reqs_.end()) continue;
        it->second.num_computed += it->second.planned;
        it->second.planned = 0;
    }
    planned_.clear();
}

int Scheduler::append_token(int64_t req) {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return kErrUnknownRequest;
    it->second.length += 1;
    it->second.decoded = 1;
    return kOk;
}

int Scheduler::finish(int64_t req) {
    auto it = reqs_.find(req);
    if (it == reqs_.end()) return kErrUnknownRequest;
    running_.erase(std::remove(running_.begin(), running_.end(), req), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), req), waiting_.end());
    planned_.erase(std::remove(planned_.begin(), planned_.end(), req), planned_.end());
    if (cache_->has_request(req)) cache_->free_request(req);
    reqs_.erase(it);
    return kOk;
}

int Scheduler::status(int64_t req) const {
    auto it = reqs_.find(req);
    return it == reqs_.end() ? (int)kUnknown : it->second.status;
}

int64_t Scheduler::length(int64_t req) const {
    auto it = reqs_.find(req);
    return it == reqs_.end() ? (int64_t)kErrUnknownRequest : it->second.length;
}

int64_t Scheduler::num_computed(int64_t req) const {
    auto it = reqs_.find(req);
    return it == reqs_.end() ? (int64_t)kErrUnknownRequest : it->second.num_computed;
}

}  // namespace engine
