#include "scheduler.h"

#include <algorithm>

namespace carbon {

Scheduler::Scheduler(CacheManager* cache, int max_running, int max_step_tokens, int max_seq_len, int vocab_size,
                     const std::vector<int>& eos_ids)
    : cache_(cache), max_running_(std::min(max_running, cache->max_requests())),
      max_step_tokens_(std::max(max_step_tokens, max_running_)), max_seq_len_(max_seq_len), vocab_(vocab_size),
      eos_(eos_ids) {}

int Scheduler::submit(int64_t id, const int32_t* prompt, int n, int max_tokens, bool ignore_eos,
                      const int32_t* stop_ids, int n_stop) {
    if (requests_.count(id)) return SUBMIT_DUPLICATE;
    if (n <= 0) return SUBMIT_EMPTY;
    if (n >= max_seq_len_) return SUBMIT_TOO_LONG;
    for (int i = 0; i < n; ++i)
        if (prompt[i] < 0 || prompt[i] >= vocab_) return SUBMIT_BAD_TOKEN;
    Request r;
    r.id = id;
    r.tokens.assign(prompt, prompt + n);
    r.stop_ids.assign(stop_ids, stop_ids + n_stop);
    r.prompt_len = n;
    r.max_new = std::max(1, std::min(max_tokens, max_seq_len_ - n));
    r.computed = 0;
    r.generated = 0;
    r.ignore_eos = ignore_eos;
    r.reason = FINISH_NONE;
    int total = lifetime_len(r);
    for (int g = 0; g < cache_->num_groups(); ++g) {
        int need = cache_->pages_for_lifetime(g, total, max_step_tokens_);
        int row_need = (total + cache_->group(g).page_size - 1) / cache_->group(g).page_size;
        if (need > cache_->group(g).num_pages || row_need > cache_->max_pages_per_request()) return SUBMIT_NEVER_FITS;
        r.lifetime_pages.push_back(need);
    }
    requests_.emplace(id, std::move(r));
    waiting_.push_back(id);
    return SUBMIT_OK;
}

bool Scheduler::fits(const Request& r) const {
    for (int g = 0; g < cache_->num_groups(); ++g) {
        long long owed = 0;
        for (int64_t rid : running_) {
            const Request& o = requests_.at(rid);
            owed += std::max(0, o.lifetime_pages[g] - cache_->held_pages(rid, g));
        }
        if (cache_->free_pages(g) < owed + r.lifetime_pages[g]) return false;
    }
    return true;
}

void Scheduler::admit() {
    while (!waiting_.empty() && (int)running_.size() < max_running_ && cache_->free_slots() > 0) {
        Request& r = requests_.at(waiting_.front());
        if (!fits(r)) {
            if (!running_.empty()) return;      // the head waits for pages to come back
            // nothing is running and it still does not fit (src/scheduler.rs:709-715)
            waiting_.pop_front();
            finish(r, FINISH_ERROR);
            continue;
        }
        int slot = cache_->open(r.id);
        if (slot < 0) return;
        waiting_.pop_front();
        running_.push_back(r.id);
    }
}

const std::vector<PlanEntry>& Scheduler::plan() {
    plan_.clear();
    plan_tokens_.clear();
    admit();
    int budget = max_step_tokens_;
    // one token of every decoding request first, then portions of prompts in running order
    for (int pass = 0; pass < 2; ++pass) {
        for (int64_t rid : running_) {
            Request& r = requests_.at(rid);
            bool decoding = r.generated > 0;
            if ((pass == 0) != decoding) continue;
            int pending = (int)r.tokens.size() - r.computed;
            int count = std::min(pending, budget);
            if (count <= 0) continue;
            if (cache_->reserve(rid, r.computed + count) != CACHE_OK) continue;   // cannot happen after admission
            PlanEntry e{rid, cache_->slot_of(rid), r.computed, count, r.computed + count == (int)r.tokens.size()};
            plan_.push_back(e);
            plan_tokens_.insert(plan_tokens_.end(), r.tokens.begin() + r.computed, r.tokens.begin() + r.computed + count);
            budget -= count;
        }
    }
    return plan_;
}

const std::vector<PlanEntry>& Scheduler::plan_for(const int64_t* ids, int n) {
    plan_.clear();
    plan_tokens_.clear();
    for (int i = 0; i < n; ++i) {
        auto it = requests_.find(ids[i]);
        if (it == requests_.end() || it->second.reason != FINISH_NONE) continue;
        Request& r = it->second;
        int pending = (int)r.tokens.size() - r.computed;
        if (r.generated == 0 || pending <= 0 || cache_->slot_of(r.id) < 0) continue;
        if (cache_->reserve(r.id, r.computed + pending) != CACHE_OK) continue;
        plan_.push_back(PlanEntry{r.id, cache_->slot_of(r.id), r.computed, pending, true});
        plan_tokens_.insert(plan_tokens_.end(), r.tokens.begin() + r.computed, r.tokens.end());
    }
    return plan_;
}

int Scheduler::remaining(int64_t id) const {
    auto it = requests_.find(id);
    if (it == requests_.end() || it->second.reason != FINISH_NONE) return -1;
    return it->second.max_new - it->second.generated;
}

void Scheduler::finish(Request& r, int reason) {
    r.reason = reason;
    if (cache_->slot_of(r.id) >= 0) cache_->close(r.id);
    running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
    finished_.emplace_back(r.id, reason);
    if (reason == FINISH_ERROR) stats_.failed++;
    stats_.finished++;
}

int Scheduler::commit(const int32_t* sampled, int n) {
    int want = 0;
    for (const auto& e : plan_) want += e.sample;
    if (want != n) return -1;
    int k = 0;
    std::vector<PlanEntry> done;
    done.swap(plan_);
    plan_tokens_.clear();
    stats_.steps++;
    for (const auto& e : done) {
        auto it = requests_.find(e.id);
        if (it == requests_.end() || it->second.reason != FINISH_NONE) {   // aborted while the step ran
            k += e.sample;
            continue;
        }
        Request& r = it->second;
        if (r.generated > 0) stats_.decode_tokens += e.count; else stats_.prefill_tokens += e.count;
        r.computed += e.count;
        cache_->commit(r.id, r.computed);
        if (!e.sample) continue;
        int tok = sampled[k++];
        r.tokens.push_back(tok);
        r.generated++;
        bool stop = false;
        if (!r.ignore_eos) {
            stop = std::find(eos_.begin(), eos_.end(), tok) != eos_.end() ||
                   std::find(r.stop_ids.begin(), r.stop_ids.end(), tok) != r.stop_ids.end();
        }
        if (stop)
            finish(r, FINISH_STOP);
        else if (r.generated >= r.max_new)
            finish(r, FINISH_LENGTH);
    }
    return 0;
}

void Scheduler::fail_step() {
    std::vector<PlanEntry> done;
    done.swap(plan_);
    plan_tokens_.clear();
    for (const auto& e : done) {
        auto it = requests_.find(e.id);
        if (it != requests_.end() && it->second.reason == FINISH_NONE) finish(it->second, FINISH_ERROR);
    }
}

int Scheduler::abort(int64_t id) {
    auto it = requests_.find(id);
    if (it == requests_.end() || it->second.reason != FINISH_NONE) return -1;
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
    finish(it->second, FINISH_ABORT);
    return 0;
}

std::vector<std::pair<int64_t, int>> Scheduler::pop_finished() {
    std::vector<std::pair<int64_t, int>> out;
    out.swap(finished_);
    return out;
}

const std::vector<int32_t>* Scheduler::tokens_of(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? nullptr : &it->second.tokens;
}

int Scheduler::prompt_len_of(int64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? -1 : it->second.prompt_len;
}

void Scheduler::forget(int64_t id) {
    auto it = requests_.find(id);
    if (it != requests_.end() && it->second.reason != FINISH_NONE) requests_.erase(it);
}

SchedulerStats Scheduler::stats() const {
    SchedulerStats s = stats_;
    s.running = (int)running_.size();
    s.waiting = (int)waiting_.size();
    return s;
}

}  // namespace carbon
