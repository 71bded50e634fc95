// Continuous-batching scheduler with portioned prompts.
//
// Queues and vocabulary follow the reference's Scheduler
// (crates/vllm-scheduler/src/scheduler.rs:75-82,139-364): waiting (FIFO),
// running (admission order), finished; a token budget per step
// (max_num_batched_tokens), a seat limit (max_num_seqs), FIFO-head-only
// admission (:184-213), finish rules "stop ids first, then max_new_tokens"
// (crates/vllm-scheduler/src/request.rs:180-192).  Differences, on purpose:
//  * a prompt longer than the budget continues in later steps (the reference
//    only ever schedules a prompt's first portion, scheduler.rs:202-228);
//  * pages are reserved portion by portion, not all at admission;
//  * when pages run out nothing is swapped (the reference's swap moves no
//    data, crates/vllm-paged-attention/src/allocator.rs:113-126): the most
//    recently admitted running request is preempted, its pages and slot come
//    back, it returns to the front of the waiting queue with its generated
//    tokens kept, and is recomputed later as one longer prompt.  A request
//    that cannot fit the pool even alone ends with an error;
//  * max_model_len is enforced when a request is added (the reference stores
//    it unused, scheduler.rs:44,55).
//
// Every request is "tokens known so far" (prompt + generated) and "tokens in
// the cache"; a step entry is the next portion of what is known but not yet
// computed.  The entry that reaches the end asks for logits at its last token;
// a decoded token is simply a portion of one.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.hpp"

namespace railgun {

enum FinishReason : int {
    FINISH_NONE = 0,
    FINISH_MAX_TOKENS = 1,
    FINISH_STOP_TOKEN = 2,
    FINISH_CANCELLED = 3,
    FINISH_ERROR = 4,
};

enum SchedStatus : int {
    SCHED_OK = 0,
    SCHED_EMPTY_PROMPT = -1,
    SCHED_TOO_LONG = -2,
    SCHED_DUPLICATE = -3,
    SCHED_UNKNOWN = -4,
    SCHED_BAD_ARGUMENT = -5,
};

struct SchedConfig {
    int max_num_batched_tokens = 4096;   // scheduler.rs:47-58 defaults
    int max_num_seqs = 256;
    int max_prefill_chunk = 0;           // 0: a portion is bounded by the budget alone
    int max_model_len = 4096;
};

struct SchedRequest {
    int64_t id = 0;
    std::vector<int> tokens;             // prompt, then generated tokens
    int prompt_len = 0;
    int max_new_tokens = 0;
    std::vector<int> stop_ids;
    float temperature = 0.f;             // sampling parameters: they outlive a preemption, the slot's record does not
    float top_p = 1.f;
    int top_k = 0;
    uint64_t seed = 0;
    int finish = FINISH_NONE;
    int num_preemptions = 0;
    uint64_t arrival = 0;
    int num_generated() const { return (int)tokens.size() - prompt_len; }
};

struct StepEntry {
    int64_t id;
    int start;
    int count;
    int want_last;
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, const SchedConfig& cfg) : cache_(cache), cfg_(cfg) {}

    int add_request(int64_t id, const int* prompt, int n, int max_new_tokens, const int* stop, int n_stop,
                    float temperature = 0.f, int top_k = 0, float top_p = 1.f, uint64_t seed = 0) {
        if (n <= 0) return SCHED_EMPTY_PROMPT;              // request.rs:143 asserts a non-empty prompt
        if (max_new_tokens < 1 || !(temperature >= 0.f) || top_k < 0 || !(top_p > 0.f && top_p <= 1.f))
            return SCHED_BAD_ARGUMENT;
        if (all_.count(id)) return SCHED_DUPLICATE;
        if (n + max_new_tokens > cfg_.max_model_len) return SCHED_TOO_LONG;
        SchedRequest r;
        r.id = id;
        r.tokens.assign(prompt, prompt + n);
        r.prompt_len = n;
        r.max_new_tokens = max_new_tokens;
        r.stop_ids.assign(stop, stop + n_stop);
        r.temperature = temperature; r.top_k = top_k; r.top_p = top_p; r.seed = seed;
        r.arrival = next_arrival_++;
        all_.emplace(id, std::move(r));
        waiting_.push_back(id);
        return SCHED_OK;
    }

    // Decide the next step.  Fills entries() and preempted().
    int schedule() {
        entries_.clear();
        preempted_.clear();
        int budget = cfg_.max_num_batched_tokens;

        // 1. running requests, decoding ones first (a portion of one token), then unfinished prompts
        std::vector<int64_t> order;
        for (int64_t id : running_) if (remaining(id) == 1) order.push_back(id);
        for (int64_t id : running_) if (remaining(id) > 1) order.push_back(id);
        for (int64_t id : order) {
            if (budget <= 0) break;
            if (std::find(running_.begin(), running_.end(), id) == running_.end()) continue;   // preempted meanwhile
            SchedRequest& r = all_[id];
            const int computed = cache_->num_computed(id);
            int n = portion((int)r.tokens.size() - computed, budget);
            bool placed = false;
            while (true) {
                if (cache_->reserve(id, computed + n) == CACHE_OK) { placed = true; break; }
                // out of pages: the most recently admitted running request gives way
                const int64_t victim = running_.back();
                if (victim == id) {
                    if (running_.size() == 1) {
                        // alone and still too large for the pool
                        finish(id, FINISH_ERROR, "out of KV cache blocks");
                    } else {
                        preempt(id, budget);
                    }
                    break;
                }
                preempt(victim, budget);
            }
            if (!placed) continue;
            entries_.push_back({id, computed, n, computed + n == (int)r.tokens.size() ? 1 : 0});
            budget -= n;
        }

        // 2. admit from the head of the waiting queue
        while (preempted_.empty() && !waiting_.empty() && budget > 0 &&
               (int)running_.size() < cfg_.max_num_seqs && cache_->free_slots() > 0) {
            const int64_t id = waiting_.front();
            SchedRequest& r = all_[id];
            const int n = portion((int)r.tokens.size(), budget);
            // one spare page per group keeps room for the running requests' next tokens
            if (!cache_->can_reserve(id, n, running_.empty() ? 0 : 1)) {
                if (running_.empty() && !fits_alone((int)r.tokens.size())) {
                    waiting_.pop_front();
                    finish_unadmitted(id, FINISH_ERROR, "out of KV cache blocks");
                    continue;
                }
                break;
            }
            waiting_.pop_front();
            if (cache_->add_request(id) < 0 || cache_->reserve(id, n) != CACHE_OK) {
                if (cache_->has(id)) cache_->release(id);
                waiting_.push_front(id);
                break;
            }
            running_.push_back(id);
            write_record(r);
            entries_.push_back({id, 0, n, n == (int)r.tokens.size() ? 1 : 0});
            budget -= n;
        }
        return (int)entries_.size();
    }

    // The step ran: entries' tokens are in the cache; `ids`/`tokens` give the token sampled for
    // every entry that asked for logits.  Returns how many requests finished.
    int update(const int64_t* ids, const int* tokens, int n) {
        for (const StepEntry& e : entries_)
            if (cache_->has(e.id)) cache_->commit(e.id, e.start + e.count);
        int finished = 0;
        for (int i = 0; i < n; ++i) {
            auto it = all_.find(ids[i]);
            if (it == all_.end() || it->second.finish != FINISH_NONE) continue;
            SchedRequest& r = it->second;
            r.tokens.push_back(tokens[i]);
            if (RequestRecord* rec = cache_->record(ids[i])) {
                rec->num_generated = r.num_generated();
                rec->last_token = tokens[i];
            }
            int reason = FINISH_NONE;
            if (std::find(r.stop_ids.begin(), r.stop_ids.end(), tokens[i]) != r.stop_ids.end())
                reason = FINISH_STOP_TOKEN;
            else if (r.num_generated() >= r.max_new_tokens)
                reason = FINISH_MAX_TOKENS;
            if (reason != FINISH_NONE) {
                finish(ids[i], reason, "");
                ++finished;
            }
        }
        entries_.clear();
        return finished;
    }

    // Whether the step after the one just decided is known before this one's tokens are: every running request
    // decodes one token that cannot end it by length, and nothing was preempted.  A request that still waits was
    // refused admission in this decision (no seat, no pages or no budget), and none of those comes back unless a
    // request ends.  (A stop token may still end a request, and a request may arrive; the caller checks its guess
    // against the next decision.)
    bool next_step_predictable() const {
        if (entries_.empty() || !preempted_.empty()) return false;
        if (entries_.size() != running_.size()) return false;
        for (const StepEntry& e : entries_) {
            if (e.count != 1 || !e.want_last) return false;
            const SchedRequest& r = all_.at(e.id);
            if (r.num_generated() + 1 >= r.max_new_tokens) return false;
        }
        return true;
    }

    int abort(int64_t id) {
        auto it = all_.find(id);
        if (it == all_.end()) return SCHED_UNKNOWN;
        if (it->second.finish != FINISH_NONE) return SCHED_OK;
        auto w = std::find(waiting_.begin(), waiting_.end(), id);
        if (w != waiting_.end()) {
            waiting_.erase(w);
            finish_unadmitted(id, FINISH_CANCELLED, "");
        } else {
            finish(id, FINISH_CANCELLED, "");
        }
        entries_.erase(std::remove_if(entries_.begin(), entries_.end(),
                                      [&](const StepEntry& e) { return e.id == id; }), entries_.end());
        return SCHED_OK;
    }

    void forget(int64_t id) {
        auto it = all_.find(id);
        if (it != all_.end() && it->second.finish != FINISH_NONE) {
            all_.erase(it);
            finished_.erase(std::remove(finished_.begin(), finished_.end(), id), finished_.end());
        }
    }

    const std::vector<StepEntry>& entries() const { return entries_; }
    const std::vector<int64_t>& preempted() const { return preempted_; }
    const std::vector<int64_t>& finished() const { return finished_; }
    const SchedRequest* find(int64_t id) const {
        auto it = all_.find(id);
        return it == all_.end() ? nullptr : &it->second;
    }
    const std::string& error_of(int64_t id) const {
        static const std::string none;
        auto it = errors_.find(id);
        return it == errors_.end() ? none : it->second;
    }
    int num_waiting() const { return (int)waiting_.size(); }
    int num_running() const { return (int)running_.size(); }
    CacheManager* cache() const { return cache_; }

private:
    // The slot's record of a request that has just been given a slot (admitted, maybe after a preemption).
    void write_record(const SchedRequest& r) {
        RequestRecord* rec = cache_->record(r.id);
        if (!rec) return;
        rec->prompt_len = r.prompt_len;
        rec->num_generated = r.num_generated();
        rec->max_new_tokens = r.max_new_tokens;
        rec->last_token = r.tokens.back();
        rec->temperature = r.temperature; rec->top_k = r.top_k; rec->top_p = r.top_p; rec->seed = r.seed;
    }
    int remaining(int64_t id) const {
        const SchedRequest& r = all_.at(id);
        return (int)r.tokens.size() - cache_->num_computed(id);
    }
    int portion(int remaining_tokens, int budget) const {
        int n = std::min(remaining_tokens, budget);
        if (cfg_.max_prefill_chunk > 0 && remaining_tokens > 1) n = std::min(n, cfg_.max_prefill_chunk);
        return n;
    }
    bool fits_alone(int len) const {
        for (int g = 0; g < cache_->num_groups(); ++g) {
            const CacheGroup& G = cache_->group(g);
            if (G.window > 0) continue;      // a windowed group gives pages back as it goes
            if ((len + G.page_size - 1) / G.page_size > G.num_pages) return false;
        }
        return true;
    }
    void drop_entry(int64_t id, int& budget) {
        for (auto it = entries_.begin(); it != entries_.end(); ++it)
            if (it->id == id) {
                budget += it->count;
                entries_.erase(it);
                return;
            }
    }
    void preempt(int64_t id, int& budget) {
        drop_entry(id, budget);
        cache_->release(id);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        waiting_.push_front(id);
        all_[id].num_preemptions++;
        preempted_.push_back(id);
    }
    void finish(int64_t id, int reason, const char* error) {
        if (cache_->has(id)) cache_->release(id);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        finish_unadmitted(id, reason, error);
    }
    void finish_unadmitted(int64_t id, int reason, const char* error) {
        all_[id].finish = reason;
        if (error && *error) errors_[id] = error;
        finished_.push_back(id);
    }

    CacheManager* cache_;
    SchedConfig cfg_;
    std::unordered_map<int64_t, SchedRequest> all_;
    std::unordered_map<int64_t, std::string> errors_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;
    std::vector<int64_t> finished_;
    std::vector<StepEntry> entries_;
    std::vector<int64_t> preempted_;
    uint64_t next_arrival_ = 0;
};

}  // namespace railgun
