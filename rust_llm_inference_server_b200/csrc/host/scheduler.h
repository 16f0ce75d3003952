// Iteration-level scheduling over the paged cache (continuous batching).
//
// One rule, as in crates/engine/src/scheduler.rs:1-22 of akshajnad/rust_llm_inference_server: a
// request is its tokens (prompt plus generated) and `num_computed`; each step computes the next
// portion of the gap.  That covers prompts, prompts cut into portions under the token budget,
// decoding (gap 1) and recomputation after preemption (gap = everything).
//
// Policy (scheduler.rs:193-306):
//  * running requests first, oldest first, inside `max_batched_tokens`;
//  * when a running request needs a page and none is free, the NEWEST running request is
//    preempted: its pages and state slot are given back and it recomputes from the start later
//    (its registered pages stay cached, so the recomputation is mostly a prefix hit);
//    a step that preempted admits nobody;
//  * admission is first come, first served, preempted requests before new ones, the head of the
//    line is never skipped; a request is admitted only if its whole known length fits with the
//    watermark to spare, and that length is reserved at once in the groups that keep all tokens;
//  * "static" policy admits only when nothing is running.
#pragma once

#include <deque>

#include "kvcache.h"

namespace rlis {

struct SchedulerConfig {
    int max_num_seqs = 64;
    int max_batched_tokens = 2048;
    bool continuous = true;       // false: static batching
    bool prefix_caching = true;
    int watermark_blocks = -1;    // pages kept free at admission; negative: max(1, pages / 100)
};

struct ScheduledSeq {
    SeqId id;
    size_t start, end;  // compute tokens [start, end) this step
};

struct Schedule {
    std::vector<ScheduledSeq> seqs;
    std::vector<SeqId> preempted;
    size_t num_tokens() const {
        size_t n = 0;
        for (auto& s : seqs) n += s.end - s.start;
        return n;
    }
};

class Scheduler {
public:
    Scheduler(SchedulerConfig cfg, std::vector<GroupConfig> groups)
        : cfg_(cfg), cache_(std::move(groups), cfg.max_num_seqs) {
        if (cfg_.max_batched_tokens < cfg_.max_num_seqs)
            throw std::invalid_argument("max_batched_tokens must cover one decode token per sequence");
        if (cfg_.prefix_caching && !cache_.prefix_reuse_possible()) cfg_.prefix_caching = false;
        cache_.set_watermark(cfg_.watermark_blocks);
    }

    CacheManager& cache() { return cache_; }
    const SchedulerConfig& config() const { return cfg_; }

    void add(SeqId id, std::vector<int32_t> tokens) {
        if (tokens.empty()) throw std::invalid_argument("empty sequence");
        SeqState s;
        s.id = id;
        s.arrival = next_arrival_++;
        s.tokens = std::move(tokens);
        waiting_.push_back(std::move(s));
    }

    Schedule schedule() {
        Schedule out;
        size_t budget = cfg_.max_batched_tokens;
        schedule_running(out, budget);
        const bool may_admit = cfg_.continuous ? out.preempted.empty() : running_.empty();
        if (may_admit) admit(out, budget);
        return out;
    }

    // The executor computed tokens up to `end`: newly full pages enter the prefix registry, and
    // window groups give back the pages every later query has passed.
    void advance(SeqId id, size_t end) {
        SeqState* s = find_running(id);
        if (!s) return;
        if (end > s->tokens.size()) throw std::logic_error("advanced past the known tokens");
        s->num_computed = end;
        cache_.release_behind(id, end);
        if (!cfg_.prefix_caching) return;
        const size_t ps = cache_.group(0).page_size;
        while ((s->registered + 1) * ps <= end) {
            const size_t i = s->registered;
            s->chain = next_page_hash(s->chain, s->tokens.data() + i * ps, ps);
            cache_.register_page(id, i, s->chain);
            ++s->registered;
        }
    }

    // A request that was preempted since its last step still takes the token that step sampled.
    void append_token(SeqId id, int32_t token) {
        if (SeqState* s = find_any_mutable(id)) s->tokens.push_back(token);
    }

    // Takes back the newest token (a placeholder of a step that was planned but never launched).
    // Tokens that have been computed stay.
    void drop_last_token(SeqId id) {
        SeqState* s = find_any_mutable(id);
        if (!s || s->tokens.size() <= 1 || s->tokens.size() <= s->num_computed)
            throw std::logic_error("drop_last_token: no uncomputed token to take back");
        s->tokens.pop_back();
    }

    size_t num_tokens(SeqId id) const {
        const SeqState* s = find_any(id);
        return s ? s->tokens.size() : 0;
    }

    // Replaces the token at `index` (a placeholder that was appended for a step launched before
    // the token was known).  The sequence may have been preempted in the meantime.
    void set_token(SeqId id, size_t index, int32_t token) {
        SeqState* s = find_any_mutable(id);
        if (!s) return;
        if (index >= s->tokens.size()) throw std::out_of_range("set_token: no such token");
        s->tokens[index] = token;
    }

    bool is_caught_up(SeqId id) const {
        for (auto& s : running_)
            if (s.id == id) return s.num_computed == s.tokens.size();
        return false;
    }

    void remove(SeqId id) {
        auto drop = [id](auto& q) {
            q.erase(std::remove_if(q.begin(), q.end(), [id](const SeqState& s) { return s.id == id; }), q.end());
        };
        drop(running_);
        drop(waiting_);
        drop(preempted_);
        cache_.free(id);
    }

    std::vector<int32_t> tokens(SeqId id, size_t start, size_t end) const {
        const SeqState* s = find_any(id);
        if (!s) throw std::out_of_range("unknown sequence");
        if (start > end || end > s->tokens.size()) throw std::out_of_range("token range");
        return std::vector<int32_t>(s->tokens.begin() + start, s->tokens.begin() + end);
    }

    bool has_work() const { return !(running_.empty() && waiting_.empty() && preempted_.empty()); }
    size_t num_running() const { return running_.size(); }
    size_t num_waiting() const { return waiting_.size() + preempted_.size(); }
    uint64_t num_preemptions() const { return num_preemptions_; }
    uint64_t admitted_tokens() const { return admitted_tokens_; }
    uint64_t cached_tokens() const { return cached_tokens_; }

    // Consistency of the queues with the cache; empty when fine.
    std::string check() const {
        std::string e = cache_.check_invariants();
        if (!e.empty()) return e;
        for (auto& s : running_)
            for (int g = 0; g < cache_.num_groups(); ++g)
                if (cache_.group(g).window == 0 && cache_.reserved_tokens(s.id, g) < s.num_computed)
                    return "running request computed more tokens than it holds slots for";
        for (auto& s : waiting_)
            if (cache_.contains(s.id) || cache_.state_slot(s.id) >= 0) return "queued request holds pages or a state slot";
        for (auto& s : preempted_)
            if (cache_.contains(s.id) || cache_.state_slot(s.id) >= 0) return "preempted request holds pages or a state slot";
        for (size_t i = 1; i < running_.size(); ++i)
            if (running_[i - 1].arrival >= running_[i].arrival) return "running is not sorted by arrival";
        return "";
    }

private:
    struct SeqState {
        SeqId id = 0;
        uint64_t arrival = 0;
        std::vector<int32_t> tokens;
        size_t num_computed = 0;
        size_t registered = 0;  // leading pages entered in the prefix registry
        uint64_t chain = 0;     // hash chain through them
    };

    const SeqState* find_any(SeqId id) const {
        for (auto& s : running_) if (s.id == id) return &s;
        for (auto& s : waiting_) if (s.id == id) return &s;
        for (auto& s : preempted_) if (s.id == id) return &s;
        return nullptr;
    }

    SeqState* find_any_mutable(SeqId id) {
        return const_cast<SeqState*>(static_cast<const Scheduler*>(this)->find_any(id));
    }

    SeqState* find_running(SeqId id) {
        for (auto& s : running_)
            if (s.id == id) return &s;
        return nullptr;
    }

    void schedule_running(Schedule& out, size_t& budget) {
        size_t i = 0;
        while (i < running_.size() && budget > 0) {
            SeqState& s = running_[i];
            const size_t want = std::min(s.tokens.size() - s.num_computed, budget);
            if (want == 0) { ++i; continue; }
            if (cache_.reserve(s.id, s.num_computed + want)) {
                out.seqs.push_back({s.id, s.num_computed, s.num_computed + want});
                budget -= want;
                ++i;
            } else {
                // Out of pages: the newest running request gives way; if that is this one, it
                // waits its turn (the loop ends because running_ shrank to i).
                SeqState victim = std::move(running_.back());
                running_.pop_back();
                preempt(std::move(victim), out);
            }
        }
    }

    void preempt(SeqState s, Schedule& out) {
        cache_.free(s.id);
        // (the victim is the last of `running_`, which this step has not reached yet, so no
        // portion of it is in `out.seqs`)
        s.num_computed = 0;
        s.registered = 0;
        s.chain = 0;
        out.preempted.push_back(s.id);
        ++num_preemptions_;
        auto at = std::find_if(preempted_.begin(), preempted_.end(),
                               [&](const SeqState& p) { return p.arrival >= s.arrival; });
        preempted_.insert(at, std::move(s));
    }

    void admit(Schedule& out, size_t& budget) {
        const bool ignore_budget = !cfg_.continuous;
        while (running_.size() < size_t(cfg_.max_num_seqs) && (ignore_budget || budget > 0)) {
            auto& queue = preempted_.empty() ? waiting_ : preempted_;
            if (queue.empty()) break;
            SeqState& head = queue.front();
            const size_t n = head.tokens.size();
            // Cached leading pages, never the one that holds the last token: its logits are
            // needed, so at least one token is always computed (scheduler.rs:267-272).
            std::vector<uint64_t> hashes;
            if (cfg_.prefix_caching)
                hashes = page_hashes(head.tokens.data(), n - 1, cache_.group(0).page_size);
            std::vector<int> evictable;
            const size_t matched = cache_.prefix_match(hashes, &evictable);
            const size_t window_tokens = size_t(cfg_.max_batched_tokens);
            if (!cache_.fits(n, window_tokens, matched, evictable)) break;
            if (cache_.num_free_state_slots() == 0) break;
            SeqState s = std::move(queue.front());
            queue.pop_front();
            if (matched > 0) {
                cache_.adopt_prefix(s.id, hashes, matched);
                s.num_computed = matched * cache_.group(0).page_size;
                s.registered = matched;
                s.chain = hashes[matched - 1];
            }
            admitted_tokens_ += n;
            cached_tokens_ += s.num_computed;
            cache_.acquire_state_slot(s.id);
            // Reserve the whole known length now in the groups that keep every token, so later
            // admissions cannot overcommit; window groups are reserved portion by portion.
            if (!cache_.reserve(s.id, n, /*windows_too=*/false)) throw std::logic_error("admission was checked");
            const size_t want = std::min(n - s.num_computed, budget);
            if (want > 0) {
                if (!cache_.reserve(s.id, s.num_computed + want)) throw std::logic_error("admission was checked");
                out.seqs.push_back({s.id, s.num_computed, s.num_computed + want});
                budget -= want;
            }
            auto at = std::find_if(running_.begin(), running_.end(),
                                   [&](const SeqState& r) { return r.arrival >= s.arrival; });
            running_.insert(at, std::move(s));
        }
    }

    SchedulerConfig cfg_;
    CacheManager cache_;
    std::deque<SeqState> waiting_;
    std::deque<SeqState> preempted_;   // sorted by arrival
    std::vector<SeqState> running_;    // sorted by arrival; the last one is the preemption victim
    uint64_t next_arrival_ = 0;
    uint64_t num_preemptions_ = 0;
    uint64_t admitted_tokens_ = 0;
    uint64_t cached_tokens_ = 0;
};

}  // namespace rlis
