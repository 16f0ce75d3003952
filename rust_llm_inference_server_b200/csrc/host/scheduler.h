// Which requests run in the next step, and on how many of their tokens.
//
// A request is a list of tokens (its prompt, then what was generated) and a count `done` of how
// many of them are in the cache.  Every step works off a piece of the gap between the two, so a
// fresh prompt, a prompt cut into portions, a decoding request (gap 1) and a request that lost its
// pages and starts over (gap = everything) are one case (the rule of
// crates/engine/src/scheduler.rs:1-22 of akshajnad/rust_llm_inference_server).
//
// The decisions are those of crates/engine/src/scheduler.rs:193-306; the shape is this engine's:
//  * requests are `active_` (they hold pages and a state slot) or in `line_` (they hold nothing).
//    The line is one queue in order of arrival: a request that was sent back to it arrived before
//    every request that was never admitted (admission never skips the head of the line), so
//    "sent-back requests first, oldest first, then newcomers" is simply that order;
//  * a step is planned in two passes over a token budget.  Pass one walks the active requests,
//    oldest first, and gives each the room for its next piece; when the cache has no page left, the
//    YOUNGEST active request is sent back to the line, pages and state slot returned, and the walk
//    goes on (if the youngest is the one being served, the walk is over).  Pass two admits from the
//    head of the line while seats, budget and pages allow, through `CacheManager::admit`, one
//    transaction over the prefix cache, every group's pages and the state slots; a step that sent
//    anybody back admits nobody, and under the "static" policy nobody is admitted while anybody
//    is active.
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
    std::vector<SeqId> preempted;   // sent back to the line in this step, in that order
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
        Request r;
        r.id = id;
        r.ticket = next_ticket_++;
        r.tokens = std::move(tokens);
        line_.push_back(std::move(r));      // tickets only grow: the line stays sorted
    }

    Schedule schedule() {
        Schedule plan;
        size_t budget = size_t(cfg_.max_batched_tokens);
        serve_active(plan, budget);
        const bool doors_open = cfg_.continuous ? plan.preempted.empty() : active_.empty();
        if (doors_open) admit_from_line(plan, budget);
        return plan;
    }

    // The step computed the request's tokens up to `end`.  Pages that are full now get their names
    // (the hash of everything up to their end), and window groups return what no later query reads.
    void advance(SeqId id, size_t end) {
        Request* r = find_in(active_, id);
        if (!r) return;
        if (end > r->tokens.size()) throw std::logic_error("advanced past the known tokens");
        r->done = end;
        cache_.release_behind(id, end);
        if (!cfg_.prefix_caching) return;
        const size_t page = cache_.group(0).page_size;
        for (; (r->named + 1) * page <= end; ++r->named) {
            r->chain = next_page_hash(r->chain, r->tokens.data() + r->named * page, page);
            cache_.register_page(id, r->named, r->chain);
        }
    }

    // Wherever the request is: one that was sent back to the line since its last step still takes
    // the token that step sampled.
    void append_token(SeqId id, int32_t token) {
        if (Request* r = find(id)) r->tokens.push_back(token);
    }

    // Replaces the token at `index`: the value of a placeholder that was appended for a step
    // launched before the token was known.
    void set_token(SeqId id, size_t index, int32_t token) {
        Request* r = find(id);
        if (!r) return;
        if (index >= r->tokens.size()) throw std::out_of_range("set_token: no such token");
        r->tokens[index] = token;
    }

    // Takes back the newest token (a placeholder of a step that was planned but never launched).
    // Tokens that are in the cache stay.
    void drop_last_token(SeqId id) {
        Request* r = find(id);
        if (!r || r->tokens.size() <= 1 || r->tokens.size() <= r->done)
            throw std::logic_error("drop_last_token: no uncomputed token to take back");
        r->tokens.pop_back();
    }

    size_t num_tokens(SeqId id) const {
        const Request* r = find(id);
        return r ? r->tokens.size() : 0;
    }

    bool is_caught_up(SeqId id) const {
        const Request* r = find_in(active_, id);
        return r != nullptr && r->done == r->tokens.size();
    }

    void remove(SeqId id) {
        auto gone = [id](const Request& r) { return r.id == id; };
        active_.erase(std::remove_if(active_.begin(), active_.end(), gone), active_.end());
        line_.erase(std::remove_if(line_.begin(), line_.end(), gone), line_.end());
        cache_.free(id);
    }

    std::vector<int32_t> tokens(SeqId id, size_t start, size_t end) const {
        const Request* r = find(id);
        if (!r) throw std::out_of_range("unknown sequence");
        if (start > end || end > r->tokens.size()) throw std::out_of_range("token range");
        return std::vector<int32_t>(r->tokens.begin() + start, r->tokens.begin() + end);
    }

    bool has_work() const { return !(active_.empty() && line_.empty()); }
    size_t num_running() const { return active_.size(); }
    size_t num_waiting() const { return line_.size(); }
    uint64_t num_preemptions() const { return sent_back_; }
    uint64_t admitted_tokens() const { return admitted_tokens_; }
    uint64_t cached_tokens() const { return cached_tokens_; }

    // Consistency of the two sets with the cache; empty when fine.
    std::string check() const {
        std::string e = cache_.check_invariants();
        if (!e.empty()) return e;
        for (auto& r : active_)
            for (int g = 0; g < cache_.num_groups(); ++g)
                if (cache_.group(g).window == 0 && cache_.reserved_tokens(r.id, g) < r.done)
                    return "an active request has more tokens in the cache than slots reserved";
        for (auto& r : line_)
            if (cache_.contains(r.id) || cache_.state_slot(r.id) >= 0) return "a request in the line holds pages or a state slot";
        for (size_t i = 1; i < active_.size(); ++i)
            if (active_[i - 1].ticket >= active_[i].ticket) return "the active requests are not in order of arrival";
        for (size_t i = 1; i < line_.size(); ++i)
            if (line_[i - 1].ticket >= line_[i].ticket) return "the line is not in order of arrival";
        return "";
    }

private:
    struct Request {
        SeqId id = 0;
        uint64_t ticket = 0;        // order of arrival
        std::vector<int32_t> tokens;
        size_t done = 0;            // tokens in the cache
        size_t named = 0;           // leading pages that have their names in the prefix cache
        uint64_t chain = 0;         // the name of the last of them
        size_t gap() const { return tokens.size() - done; }
    };

    template <typename Set> static auto find_in(Set& set, SeqId id) -> decltype(&*set.begin()) {
        for (auto& r : set)
            if (r.id == id) return &r;
        return nullptr;
    }
    Request* find(SeqId id) {
        Request* r = find_in(active_, id);
        return r ? r : find_in(line_, id);
    }
    const Request* find(SeqId id) const {
        const Request* r = find_in(active_, id);
        return r ? r : find_in(line_, id);
    }

    // Pass one: every active request, oldest first, gets room for its next piece or somebody goes.
    void serve_active(Schedule& plan, size_t& budget) {
        for (size_t i = 0; i < active_.size() && budget > 0;) {
            Request& r = active_[i];
            const size_t piece = std::min(r.gap(), budget);
            if (piece == 0) {
                ++i;
            } else if (cache_.reserve(r.id, r.done + piece)) {
                plan.seqs.push_back({r.id, r.done, r.done + piece});
                budget -= piece;
                ++i;
            } else {
                send_back_youngest(plan);       // active_ shrinks; when it shrinks to i, r itself went
            }
        }
    }

    // The youngest active request (the walk above has not reached it, so none of its tokens are in
    // the plan) returns everything and starts over later; what it had named stays in the prefix
    // cache, so starting over is mostly a lookup.
    void send_back_youngest(Schedule& plan) {
        Request r = std::move(active_.back());
        active_.pop_back();
        cache_.free(r.id);
        r.done = r.named = 0;
        r.chain = 0;
        plan.preempted.push_back(r.id);
        ++sent_back_;
        auto at = std::find_if(line_.begin(), line_.end(), [&](const Request& q) { return q.ticket > r.ticket; });
        line_.insert(at, std::move(r));
    }

    // Pass two: the head of the line comes in while there is a seat, budget (the static policy
    // fills its batch regardless of the budget) and the cache admits it.
    void admit_from_line(Schedule& plan, size_t& budget) {
        const bool any_budget = !cfg_.continuous;
        while (!line_.empty() && active_.size() < size_t(cfg_.max_num_seqs) && (any_budget || budget > 0)) {
            Request& head = line_.front();
            const size_t n = head.tokens.size();
            const CacheManager::Admission adm =
                cache_.admit(head.id, head.tokens.data(), n, size_t(cfg_.max_batched_tokens), cfg_.prefix_caching);
            if (!adm.ok) break;                 // nobody overtakes the head of the line
            Request r = std::move(line_.front());
            line_.pop_front();
            r.named = adm.cached_pages;
            r.chain = adm.chain;
            r.done = adm.cached_pages * cache_.group(0).page_size;
            admitted_tokens_ += n;
            cached_tokens_ += r.done;
            const size_t piece = std::min(r.gap(), budget);
            if (piece > 0) {
                // (the groups that keep every token are reserved to the end; this takes the window groups' share)
                if (!cache_.reserve(r.id, r.done + piece)) throw std::logic_error("admission had checked the room");
                plan.seqs.push_back({r.id, r.done, r.done + piece});
                budget -= piece;
            }
            auto at = std::find_if(active_.begin(), active_.end(), [&](const Request& q) { return q.ticket > r.ticket; });
            active_.insert(at, std::move(r));
        }
    }

    SchedulerConfig cfg_;
    CacheManager cache_;
    std::vector<Request> active_;   // in order of arrival; the last one is the first to be sent back
    std::deque<Request> line_;      // in order of arrival; holds nothing in the cache
    uint64_t next_ticket_ = 0;
    uint64_t sent_back_ = 0;
    uint64_t admitted_tokens_ = 0;
    uint64_t cached_tokens_ = 0;
};

}  // namespace rlis
