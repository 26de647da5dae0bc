// Request scheduler (host only): admission, token budget, chunking, preemption.
//
// Rules follow the reference's scheduler (backends/vllm/src/scheduler.rs), which
// works on three queues under a per-step budget of tokens and sequences
// (:40-149) in first-come-first-served order (backends/vllm/src/policy.rs:55-61):
//  * chunked prefill on (schedule_chunked_prefill, :1257-1379): running requests
//    first, decodes and prompt portions alike, then new prompts with what is left
//    of the budget; a portion is clipped to the remaining budget (:1588-1623);
//  * chunked prefill off (schedule_default, :1057-1217): if any whole prompt can
//    be admitted the step holds prompts only, otherwise every running request
//    decodes one token;
//  * a prompt longer than the limit, or one that no empty pool could hold, is
//    dropped as ignored (:957-992, :2120-2128); one that does not fit now blocks
//    the queue behind it;
//  * when a running request cannot get a page, the last running request is
//    preempted: its pages are freed and it goes back to the FRONT of the waiting
//    queue with nothing computed (recompute, :650-690, :1778-1826, :1860-1896); if
//    nobody else is left it preempts itself;
//  * a portion samples only when it reaches the end of the request (:1498-1521).
// Differences, each deliberate: a finished request gives its pages back at once
// (the reference never frees them, :2203-2216); prompt portions in flight stay in
// the running queue (the reference drops them, :1313-1338); the delay factor
// (:2077-2097) is not built.
//
// The scheduler knows lengths, not token values; the engine keeps the tokens.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.hpp"

namespace engine {

struct SchedulerConfig {
    int max_num_batched_tokens;
    int max_num_seqs;
    int64_t max_model_len;
    int enable_chunked_prefill;
};

enum RequestStatus : int { kWaiting = 0, kRunning = 1, kFinished = 2, kIgnored = 3, kUnknown = -1 };

struct StepEntry {
    int64_t req;
    int64_t context_len;  // tokens already in the cache
    int32_t num_tokens;   // tokens to run this step
    int32_t samples;      // 1 if the portion reaches the end of the request
    int32_t is_prompt;    // 1 while the request has not sampled its first token since (re)admission
};

struct StepPlan {
    std::vector<StepEntry> entries;
    std::vector<int64_t> preempted;  // went back to waiting, cache dropped
    std::vector<int64_t> ignored;    // dropped for good: too long for the limit or for the cache
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, const SchedulerConfig& cfg) : cache_(cache), cfg_(cfg) {}

    // A new request of `prompt_len` tokens joins the back of the waiting queue.
    int add_request(int64_t req, int64_t prompt_len);
    // Plans one step and claims its pages.
    StepPlan schedule();
    // The planned step ran: its tokens are computed.  (The step function advances
    // the cache itself; this mirrors it in the queue records.)
    void step_done();
    // A sampled token was appended to a running request.
    int append_token(int64_t req);
    // A running or waiting request ends (stop rule or abort): pages and slot go back.
    int finish(int64_t req);

    int status(int64_t req) const;
    int64_t length(int64_t req) const;
    int64_t num_computed(int64_t req) const;
    int num_waiting() const { return (int)waiting_.size(); }
    int num_running() const { return (int)running_.size(); }
    int64_t prompt_limit() const;
    int64_t num_preemptions() const { return num_preemptions_; }

private:
    struct Request {
        int64_t id;
        int64_t length;        // prompt + sampled tokens known so far
        int64_t num_computed;  // tokens in the cache
        int64_t arrival;       // admission order key (FCFS)
        int status;
        int decoded;           // sampled at least once since (re)admission
        int planned;           // tokens planned in the step under way
    };
    void preempt(Request& r, StepPlan& plan);
    bool schedule_running(StepPlan& plan, int& token_budget, bool chunk);
    void schedule_waiting(StepPlan& plan, int& token_budget, bool chunk);
    void insert_running(int64_t req);

    CacheManager* cache_;
    SchedulerConfig cfg_;
    std::unordered_map<int64_t, Request> reqs_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;  // ordered by arrival
    std::vector<int64_t> planned_;
    int64_t next_arrival_ = 0;
    int64_t num_preemptions_ = 0;
};

}  // namespace engine
