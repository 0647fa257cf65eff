// C interface of the host runtime, loaded from Python with ctypes.
#include <cstring>

#include "cache_manager.h"
#include "scheduler.h"
#include "step_layout.h"

using namespace carbon;

extern "C" {

// ---- cache manager -------------------------------------------------------------------------
void* cm_create(int num_groups, const int* page_sizes, const int* num_pages, const int* windows, int max_requests,
                int max_pages_per_request) {
    if (num_groups < 0 || max_requests <= 0 || max_pages_per_request <= 0) return nullptr;
    std::vector<GroupSpec> groups;
    for (int g = 0; g < num_groups; ++g) {
        if (page_sizes[g] <= 0 || num_pages[g] < 0 || windows[g] < 0) return nullptr;
        groups.push_back(GroupSpec{page_sizes[g], num_pages[g], windows[g]});
    }
    return new CacheManager(groups, max_requests, max_pages_per_request);
}
void cm_destroy(void* h) { delete (CacheManager*)h; }
int cm_open(void* h, int64_t id) { return ((CacheManager*)h)->open(id); }
int cm_reserve(void* h, int64_t id, int new_len) { return ((CacheManager*)h)->reserve(id, new_len); }
int cm_commit(void* h, int64_t id, int new_len) { return ((CacheManager*)h)->commit(id, new_len); }
// commit for n requests at once; returns the first status that is not CACHE_OK (the others are still committed)
int cm_commit_many(void* h, const int64_t* ids, const int32_t* new_lens, int n) {
    int first = CACHE_OK;
    for (int i = 0; i < n; ++i) {
        int rc = ((CacheManager*)h)->commit(ids[i], new_lens[i]);
        if (rc != CACHE_OK && first == CACHE_OK) first = rc;
    }
    return first;
}
int cm_close(void* h, int64_t id) { return ((CacheManager*)h)->close(id); }
int cm_slot_of(void* h, int64_t id) { return ((CacheManager*)h)->slot_of(id); }
int cm_length_of(void* h, int64_t id) { return ((CacheManager*)h)->length_of(id); }
int cm_reserved_of(void* h, int64_t id) { return ((CacheManager*)h)->reserved_of(id); }
int cm_free_pages(void* h, int group) { return ((CacheManager*)h)->free_pages(group); }
int cm_held_pages(void* h, int64_t id, int group) { return ((CacheManager*)h)->held_pages(id, group); }
int cm_free_slots(void* h) { return ((CacheManager*)h)->free_slots(); }
int cm_open_requests(void* h) { return ((CacheManager*)h)->open_requests(); }
int cm_pages_for_lifetime(void* h, int group, int total_len, int max_chunk) {
    return ((CacheManager*)h)->pages_for_lifetime(group, total_len, max_chunk);
}
int cm_pages_to_reserve(void* h, int64_t id, int group, int new_len) {
    return ((CacheManager*)h)->pages_to_reserve(id, group, new_len);
}
const int32_t* cm_table(void* h, int group) { return ((CacheManager*)h)->table(group); }
int cm_check(void* h) { return ((CacheManager*)h)->check(); }

// ---- scheduler -----------------------------------------------------------------------------
void* sched_create(void* cache, int max_running, int max_step_tokens, int max_seq_len, int vocab_size,
                   const int* eos_ids, int n_eos) {
    if (!cache || max_running <= 0 || max_step_tokens <= 0 || max_seq_len <= 1 || vocab_size <= 0) return nullptr;
    return new Scheduler((CacheManager*)cache, max_running, max_step_tokens, max_seq_len, vocab_size,
                         std::vector<int>(eos_ids, eos_ids + n_eos));
}
void sched_destroy(void* h) { delete (Scheduler*)h; }
int sched_submit(void* h, int64_t id, const int32_t* prompt, int n, int max_tokens, int ignore_eos,
                 const int32_t* stop_ids, int n_stop) {
    return ((Scheduler*)h)->submit(id, prompt, n, max_tokens, ignore_eos != 0, stop_ids, n_stop);
}
// Lays out the next step.  Returns the number of entries; entries are written as 5 x int64 each
// (id, slot, start, count, sample) up to max_entries, token ids up to max_tokens.  A negative
// return means a buffer was too small.
static int write_plan(Scheduler* s, const std::vector<PlanEntry>& plan, int64_t* entries, int max_entries,
                      int32_t* tokens, int max_tokens, int* n_tokens) {
    const auto& toks = s->plan_tokens();
    if ((int)plan.size() > max_entries || (int)toks.size() > max_tokens) return -1;
    for (size_t i = 0; i < plan.size(); ++i) {
        entries[5 * i + 0] = plan[i].id;
        entries[5 * i + 1] = plan[i].slot;
        entries[5 * i + 2] = plan[i].start;
        entries[5 * i + 3] = plan[i].count;
        entries[5 * i + 4] = plan[i].sample;
    }
    if (!toks.empty()) memcpy(tokens, toks.data(), toks.size() * sizeof(int32_t));
    *n_tokens = (int)toks.size();
    return (int)plan.size();
}
int sched_plan(void* h, int64_t* entries, int max_entries, int32_t* tokens, int max_tokens, int* n_tokens) {
    Scheduler* s = (Scheduler*)h;
    return write_plan(s, s->plan(), entries, max_entries, tokens, max_tokens, n_tokens);
}
// The same for the step that is already on the device for the requests `ids` (Scheduler::plan_for).
int sched_plan_for(void* h, const int64_t* ids, int n, int64_t* entries, int max_entries, int32_t* tokens,
                   int max_tokens, int* n_tokens) {
    Scheduler* s = (Scheduler*)h;
    return write_plan(s, s->plan_for(ids, n), entries, max_entries, tokens, max_tokens, n_tokens);
}
int sched_remaining(void* h, int64_t id) { return ((Scheduler*)h)->remaining(id); }
int sched_waiting(void* h) { return ((Scheduler*)h)->waiting(); }
int sched_running(void* h) { return ((Scheduler*)h)->running(); }
int sched_commit(void* h, const int32_t* sampled, int n) { return ((Scheduler*)h)->commit(sampled, n); }
void sched_fail_step(void* h) { ((Scheduler*)h)->fail_step(); }
int sched_abort(void* h, int64_t id) { return ((Scheduler*)h)->abort(id); }
int sched_pop_finished(void* h, int64_t* ids, int* reasons, int max_n) {
    auto v = ((Scheduler*)h)->pop_finished();
    int n = (int)v.size() < max_n ? (int)v.size() : max_n;
    for (int i = 0; i < n; ++i) {
        ids[i] = v[i].first;
        reasons[i] = v[i].second;
    }
    return n;
}
int sched_num_tokens(void* h, int64_t id) {
    auto* t = ((Scheduler*)h)->tokens_of(id);
    return t ? (int)t->size() : -1;
}
int sched_prompt_len(void* h, int64_t id) { return ((Scheduler*)h)->prompt_len_of(id); }
int sched_copy_tokens(void* h, int64_t id, int32_t* out, int max_n) {
    auto* t = ((Scheduler*)h)->tokens_of(id);
    if (!t) return -1;
    int n = (int)t->size() < max_n ? (int)t->size() : max_n;
    if (n) memcpy(out, t->data(), n * sizeof(int32_t));
    return n;
}
void sched_forget(void* h, int64_t id) { ((Scheduler*)h)->forget(id); }
int sched_idle(void* h) { return ((Scheduler*)h)->idle() ? 1 : 0; }
void sched_stats(void* h, int64_t* out /* 7 values */) {
    SchedulerStats s = ((Scheduler*)h)->stats();
    out[0] = s.steps; out[1] = s.prefill_tokens; out[2] = s.decode_tokens; out[3] = s.finished; out[4] = s.failed;
    out[5] = s.running; out[6] = s.waiting;
}

// ---- step layout ---------------------------------------------------------------------------
// `args`: a StepLayoutArgs (step_layout.h), field for field.  Returns 0, a LayoutStatus or a CacheStatus.
int step_layout(void* cache, const void* args) { return layout_step(*(CacheManager*)cache, *(const StepLayoutArgs*)args); }

}  // extern "C"
