// C ABI over the cache manager and the scheduler, for the Python entry point.
// Handles are opaque pointers; every call returns a status (engine::CacheStatus)
// or a count.  No call throws across the boundary.
#include <cstring>
#include <new>

#include "cache_manager.hpp"
#include "scheduler.hpp"

using engine::CacheManager;
using engine::GroupSpec;
using engine::Scheduler;
using engine::SchedulerConfig;
using engine::StepPlan;

extern "C" {

void* cm_create(int page_size, int num_groups, const int* kinds, const int* windows, const int* num_pages,
                int max_seqs) {
    if (page_size <= 0 || num_groups < 0 || max_seqs <= 0) return nullptr;
    std::vector<GroupSpec> groups;
    for (int g = 0; g < num_groups; ++g) {
        if (num_pages[g] < 1) return nullptr;
        if (kinds[g] == engine::kWindowKeys && windows[g] <= 0) return nullptr;
        groups.push_back(GroupSpec{kinds[g], windows[g], num_pages[g]});
    }
    return new (std::nothrow) CacheManager(page_size, groups, max_seqs);
}
void cm_destroy(void* h) { delete static_cast<CacheManager*>(h); }
int cm_add_request(void* h, int64_t req) { return static_cast<CacheManager*>(h)->add_request(req); }
int cm_has_request(void* h, int64_t req) { return static_cast<CacheManager*>(h)->has_request(req); }
int cm_can_reserve(void* h, int64_t req, int64_t upto) { return static_cast<CacheManager*>(h)->can_reserve(req, upto); }
int cm_reserve(void* h, int64_t req, int64_t upto) { return static_cast<CacheManager*>(h)->reserve(req, upto); }
int cm_advance(void* h, int64_t req, int64_t n) { return static_cast<CacheManager*>(h)->advance(req, n); }
int cm_free_request(void* h, int64_t req) { return static_cast<CacheManager*>(h)->free_request(req); }
int64_t cm_num_tokens(void* h, int64_t req) { return static_cast<CacheManager*>(h)->num_tokens(req); }
int cm_state_slot(void* h, int64_t req) { return static_cast<CacheManager*>(h)->state_slot(req); }
int cm_table_len(void* h, int64_t req, int g) { return static_cast<CacheManager*>(h)->table_len(req, g); }
int cm_table(void* h, int64_t req, int g, int32_t* out, int cap) {
    return static_cast<CacheManager*>(h)->table(req, g, out, cap);
}
int cm_pages_needed(void* h, int64_t req, int g, int64_t upto) {
    return static_cast<CacheManager*>(h)->pages_needed(req, g, upto);
}
int cm_num_free_pages(void* h, int g) { return static_cast<CacheManager*>(h)->num_free_pages(g); }
int cm_num_usable_pages(void* h, int g) { return static_cast<CacheManager*>(h)->num_usable_pages(g); }
int cm_num_free_slots(void* h) { return static_cast<CacheManager*>(h)->num_free_slots(); }
int cm_num_requests(void* h) { return static_cast<CacheManager*>(h)->num_requests(); }
// Writes the audit text (empty = consistent) into `out`; returns its full length.
int cm_audit(void* h, char* out, int cap) {
    std::string s = static_cast<CacheManager*>(h)->audit();
    if (cap > 0) {
        int n = (int)std::min<size_t>(s.size(), (size_t)cap - 1);
        std::memcpy(out, s.data(), n);
        out[n] = 0;
    }
    return (int)s.size();
}

// A scheduler handle keeps the last plan, so that planning (which changes the queues) and
// copying the plan out (which needs arrays of the right size) are two calls and the second
// cannot fail after the first has acted.
struct SchedulerHandle {
    Scheduler scheduler;
    StepPlan plan;
    SchedulerHandle(CacheManager* cache, const SchedulerConfig& cfg) : scheduler(cache, cfg) {}
};
static Scheduler* sched(void* h) { return &static_cast<SchedulerHandle*>(h)->scheduler; }

void* sched_create(void* cache, int max_num_batched_tokens, int max_num_seqs, int64_t max_model_len,
                   int enable_chunked_prefill) {
    if (!cache || max_num_batched_tokens <= 0 || max_num_seqs <= 0 || max_model_len <= 0) return nullptr;
    SchedulerConfig cfg{max_num_batched_tokens, max_num_seqs, max_model_len, enable_chunked_prefill};
    return new (std::nothrow) SchedulerHandle(static_cast<CacheManager*>(cache), cfg);
}
void sched_destroy(void* h) { delete static_cast<SchedulerHandle*>(h); }
int sched_add_request(void* h, int64_t req, int64_t prompt_len) { return sched(h)->add_request(req, prompt_len); }
// Plans a step and keeps the plan in the handle.  counts[0..2] = entries, preempted, ignored:
// the sizes of the arrays that sched_plan fills.
int sched_schedule(void* h, int32_t* counts) {
    auto* sh = static_cast<SchedulerHandle*>(h);
    sh->plan = sh->scheduler.schedule();
    counts[0] = (int)sh->plan.entries.size();
    counts[1] = (int)sh->plan.preempted.size();
    counts[2] = (int)sh->plan.ignored.size();
    return engine::kOk;
}
// Copies the plan of the last sched_schedule: entries to the five arrays, preempted and ignored
// request ids to theirs (each at least as long as the count sched_schedule gave).
int sched_plan(void* h, int64_t* req, int64_t* context_len, int32_t* num_tokens, int32_t* samples,
               int32_t* is_prompt, int64_t* preempted, int64_t* ignored) {
    const StepPlan& plan = static_cast<SchedulerHandle*>(h)->plan;
    for (size_t i = 0; i < plan.entries.size(); ++i) {
        req[i] = plan.entries[i].req;
        context_len[i] = plan.entries[i].context_len;
        num_tokens[i] = plan.entries[i].num_tokens;
        samples[i] = plan.entries[i].samples;
        is_prompt[i] = plan.entries[i].is_prompt;
    }
    for (size_t i = 0; i < plan.preempted.size(); ++i) preempted[i] = plan.preempted[i];
    for (size_t i = 0; i < plan.ignored.size(); ++i) ignored[i] = plan.ignored[i];
    return engine::kOk;
}
void sched_step_done(void* h) { sched(h)->step_done(); }
int sched_append_token(void* h, int64_t req) { return sched(h)->append_token(req); }
int sched_finish(void* h, int64_t req) { return sched(h)->finish(req); }
int sched_status(void* h, int64_t req) { return sched(h)->status(req); }
int64_t sched_length(void* h, int64_t req) { return sched(h)->length(req); }
int64_t sched_num_computed(void* h, int64_t req) { return sched(h)->num_computed(req); }
int sched_num_waiting(void* h) { return sched(h)->num_waiting(); }
int sched_num_running(void* h) { return sched(h)->num_running(); }
int64_t sched_num_preemptions(void* h) { return sched(h)->num_preemptions(); }
int64_t sched_prompt_limit(void* h) { return sched(h)->prompt_limit(); }

}  // extern "C"
