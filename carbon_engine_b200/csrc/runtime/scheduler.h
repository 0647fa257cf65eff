// Continuous-batching scheduler: admits requests, cuts prompts into portions under a token budget,
// lets every decoding request take its next token, finishes requests and frees what they hold.
//
// Policy, after the reference (src/scheduler.rs:589-692 admission, :719-841 prefill portions,
// :1156-1205 decode, :1522-1581 finish):
//  * requests wait in arrival order and only the head of the queue may be admitted;
//  * a request is admitted when a state slot is free and every cache group can still give the
//    pages of its whole life (prompt + max_new - 1 tokens) on top of what the running requests may
//    still take, so a running request never runs out of pages;
//  * if nothing is running and the head still does not fit, it ends with an error;
//  * max_new = clamp(max_tokens, 1, max_seq_len - prompt_len) (src/scheduler.rs:597-601);
//  * the first output token is sampled in the step that completes the prompt
//    (src/scheduler.rs:807-810); a request ends on an end-of-sequence or stop token unless it ignores
//    them, or when it has max_new tokens.
// Unlike the reference, which runs either a prefill step or a decode step (src/scheduler.rs:694-705),
// one step here carries one token of every decoding request and fills the rest of the token
// budget with portions of prompts.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.h"

namespace carbon {

enum FinishReason { FINISH_NONE = 0, FINISH_STOP = 1, FINISH_LENGTH = 2, FINISH_ABORT = 3, FINISH_ERROR = 4 };

enum SubmitStatus {
    SUBMIT_OK = 0,
    SUBMIT_EMPTY = -1,          // empty prompt
    SUBMIT_TOO_LONG = -2,       // prompt does not leave room for one new token within max_seq_len
    SUBMIT_BAD_TOKEN = -3,      // a token id outside the vocabulary
    SUBMIT_NEVER_FITS = -4,     // needs more pages than a pool has
    SUBMIT_DUPLICATE = -5,
};

struct PlanEntry {
    int64_t id;
    int slot;
    int start;       // tokens of the request already in the cache
    int count;       // tokens fed in this step
    int sample;      // 1 if the last fed token's logits are sampled
};

struct SchedulerStats {
    int64_t steps, prefill_tokens, decode_tokens, finished, failed;
    int running, waiting;
};

class Scheduler {
  public:
    Scheduler(CacheManager* cache, int max_running, int max_step_tokens, int max_seq_len, int vocab_size,
              const std::vector<int>& eos_ids);

    int submit(int64_t id, const int32_t* prompt, int n, int max_tokens, bool ignore_eos, const int32_t* stop_ids,
               int n_stop);
    // Admit what fits and lay out the next step.  Returns the entries; the fed token ids, entry after
    // entry, are in plan_tokens().
    const std::vector<PlanEntry>& plan();
    const std::vector<int32_t>& plan_tokens() const { return plan_tokens_; }
    // The step after the last one is already on the device for these requests, one token each, its token
    // ids taken there from the last step's picks.  Lays out exactly that step for those of them that still
    // run (a request that ended meanwhile is left out); nothing is admitted.  The fed token of an entry is
    // the one the last commit appended.
    const std::vector<PlanEntry>& plan_for(const int64_t* ids, int n);
    // Tokens the request may still generate; -1 for an unknown or ended request.
    int remaining(int64_t id) const;
    int waiting() const { return (int)waiting_.size(); }
    int running() const { return (int)running_.size(); }
    // The step ran: `sampled` holds one token for every entry with sample == 1, in order.
    int commit(const int32_t* sampled, int n);
    // The step failed: every request of the plan ends with an error, the others go on
    // (src/scheduler.rs:1436-1463).
    void fail_step();
    int abort(int64_t id);

    // Requests that ended since the last call: (id, reason).
    std::vector<std::pair<int64_t, int>> pop_finished();
    const std::vector<int32_t>* tokens_of(int64_t id) const;
    int prompt_len_of(int64_t id) const;
    void forget(int64_t id);            // drop a finished request's record
    bool idle() const { return waiting_.empty() && running_.empty(); }
    SchedulerStats stats() const;

  private:
    struct Request {
        int64_t id;
        std::vector<int32_t> tokens;
        std::vector<int32_t> stop_ids;
        int prompt_len, max_new, computed, generated;
        bool ignore_eos;
        int reason;
        std::vector<int> lifetime_pages;
    };
    CacheManager* cache_;
    int max_running_, max_step_tokens_, max_seq_len_, vocab_;
    std::vector<int> eos_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;
    std::unordered_map<int64_t, Request> requests_;
    std::vector<PlanEntry> plan_;
    std::vector<int32_t> plan_tokens_;
    std::vector<std::pair<int64_t, int>> finished_;
    SchedulerStats stats_{};

    void admit();
    bool fits(const Request& r) const;
    void finish(Request& r, int reason);
    int lifetime_len(const Request& r) const { return r.prompt_len + r.max_new - 1; }
};

}  // namespace carbon
