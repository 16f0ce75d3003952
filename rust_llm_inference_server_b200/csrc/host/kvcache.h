// Paged cache bookkeeping: which physical pages hold which request's tokens.  Host logic only;
// the tensors live on the device and are addressed by the page ids handed out here.
//
// It keeps the behaviour of crates/kvcache/src/lib.rs of akshajnad/rust_llm_inference_server
// (pages reused last-returned-first, counted holders, full pages found again by the hash of their
// prefix and recycled oldest first, all-or-nothing reservation, a consistency check) in a design
// of its own, built around *groups*: layers with the same cache needs (geometry, keep-all or a
// window) share one pool of pages and one block table per request.  A window group gives pages
// back once every later query has passed them.  Beside the pages sits a pool of fixed-size
// per-request state slots, and admission of a request is one transaction over all of them.
#pragma once

#include <algorithm>
#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace rlis {

using SeqId = int64_t;
using PageId = int32_t;
constexpr PageId kNoPage = -1;

struct GroupConfig {
    int num_pages = 0;
    int page_size = 0;
    int window = 0;  // 0: every earlier token stays visible; W > 0: only the last W tokens
};

// Chained 64-bit hash of one full page of tokens on top of the hash of everything before it
// (role of next_block_hash, crates/kvcache/src/lib.rs:47-53; the hash function is our own).
inline uint64_t next_page_hash(uint64_t prev, const int32_t* tokens, size_t n) {
    uint64_t h = 0xcbf29ce484222325ull;
    auto eat = [&h](uint64_t v, int bytes) {
        for (int i = 0; i < bytes; ++i) {
            h ^= (v >> (8 * i)) & 0xffu;
            h *= 0x100000001b3ull;
        }
    };
    eat(prev, 8);
    for (size_t i = 0; i < n; ++i) eat(static_cast<uint32_t>(tokens[i]), 4);
    h ^= h >> 30; h *= 0xbf58476d1ce4e5b9ull;
    h ^= h >> 27; h *= 0x94d049bb133111ebull;
    h ^= h >> 31;
    return h;
}

inline std::vector<uint64_t> page_hashes(const int32_t* tokens, size_t n_tokens, int page_size) {
    std::vector<uint64_t> out;
    uint64_t prev = 0;
    for (size_t b = 0; (b + 1) * page_size <= n_tokens; ++b) {
        prev = next_page_hash(prev, tokens + b * page_size, page_size);
        out.push_back(prev);
    }
    return out;
}

// The pages of one group.  Every page is in exactly one of three places:
//   held   one or more requests have it in their tables (`holders` counts them);
//   kept   nobody holds it, but it is full and known by the hash of the tokens up to its end: it
//          sits in the keep-list, a doubly linked list threaded through the page records, newest
//          at the tail, from where a request with the same prefix can take it back;
//   blank  on the blank stack; the page returned last is handed out first.
// A page is handed out from the blank stack while that has any; only then is the head of the
// keep-list (the page nobody has wanted for longest) stripped of its name and reused.
// Behaviour after crates/kvcache/src/lib.rs:57-166 (free list, reference counts, evictable cached
// blocks reclaimed least-recently-freed first).
class PagePool {
public:
    explicit PagePool(int num_pages) : page_(num_pages) {
        blank_.reserve(num_pages);
        for (int b = num_pages - 1; b >= 0; --b) blank_.push_back(b);   // page 0 goes out first
    }

    int num_pages() const { return static_cast<int>(page_.size()); }
    int num_free() const { return static_cast<int>(blank_.size()) + kept_; }   // what a reservation can draw on
    int num_evictable() const { return kept_; }
    uint32_t refcount(PageId b) const { return page_.at(b).holders; }

    PageId lookup(uint64_t name) const {
        auto it = by_name_.find(name);
        return it == by_name_.end() ? kNoPage : it->second;
    }

    // Gives page b its name.  A page keeps the first name it gets, and a name the first page that
    // takes it: a second page with the same contents stays anonymous.
    void register_page(PageId b, uint64_t name) {
        Page& pg = page_.at(b);
        if (pg.named || by_name_.count(name)) return;
        pg.named = true;
        pg.name = name;
        by_name_.emplace(name, b);
    }

    // One more holder of a named page; if it was waiting in the keep-list it leaves it.
    void acquire(PageId b) {
        Page& pg = page_.at(b);
        if (pg.holders == 0) {
            if (!pg.in_keep) throw std::logic_error("acquired a page that is neither held nor kept");
            unlink(b);
        }
        ++pg.holders;
    }

    PageId allocate() {
        PageId b;
        if (!blank_.empty()) {
            b = blank_.back();
            blank_.pop_back();
        } else if (keep_head_ != kNoPage) {
            b = keep_head_;
            unlink(b);
            by_name_.erase(page_[b].name);
            page_[b].named = false;
        } else {
            return kNoPage;
        }
        if (page_[b].holders != 0) throw std::logic_error("handed out a page that is still held");
        page_[b].holders = 1;
        return b;
    }

    void decref(PageId b) {
        Page& pg = page_.at(b);
        if (pg.holders == 0) throw std::logic_error("page " + std::to_string(b) + " freed twice");
        if (--pg.holders != 0) return;
        if (pg.named) append(b);
        else blank_.push_back(b);
    }

    // Consistency with `holders[b]`, the number of tables that hold page b; empty when fine.
    std::string check(const std::vector<uint32_t>& holders) const {
        const int n = num_pages();
        std::vector<char> idle(n, 0);
        std::ostringstream err;
        for (PageId b : blank_) {
            if (idle[b]++) { err << "page " << b << " is on the blank stack twice"; return err.str(); }
            if (page_[b].named || page_[b].in_keep) { err << "blank page " << b << " still has a name"; return err.str(); }
        }
        int walked = 0;
        PageId before = kNoPage;
        for (PageId b = keep_head_; b != kNoPage; before = b, b = page_[b].next) {
            if (++walked > n) return "the keep-list has a loop";
            if (idle[b]++) { err << "page " << b << " is both blank and kept, or kept twice"; return err.str(); }
            if (!page_[b].named || !page_[b].in_keep || page_[b].prev != before) { err << "kept page " << b << " has stale links"; return err.str(); }
        }
        if (before != keep_tail_ || walked != kept_) return "the keep-list and its counters disagree";
        size_t named = 0;
        for (int b = 0; b < n; ++b) named += page_[b].named ? 1 : 0;
        if (named != by_name_.size()) return "named pages and the name index disagree";
        for (auto& kv : by_name_)
            if (!page_[kv.second].named || page_[kv.second].name != kv.first) { err << "the name index points at page " << kv.second << " with another name"; return err.str(); }
        for (int b = 0; b < n; ++b) {
            if (page_[b].holders != holders[b]) { err << "page " << b << ": " << page_[b].holders << " holders recorded but " << holders[b] << " tables hold it"; return err.str(); }
            if ((page_[b].holders == 0) != (idle[b] != 0)) { err << "page " << b << ": " << page_[b].holders << " holders, blank or kept: " << int(idle[b]); return err.str(); }
        }
        return "";
    }

private:
    struct Page {
        uint32_t holders = 0;
        bool named = false, in_keep = false;
        uint64_t name = 0;
        PageId prev = kNoPage, next = kNoPage;    // neighbours in the keep-list
    };

    void append(PageId b) {
        Page& pg = page_[b];
        pg.prev = keep_tail_;
        pg.next = kNoPage;
        pg.in_keep = true;
        if (keep_tail_ != kNoPage) page_[keep_tail_].next = b;
        else keep_head_ = b;
        keep_tail_ = b;
        ++kept_;
    }

    void unlink(PageId b) {
        Page& pg = page_[b];
        if (pg.prev != kNoPage) page_[pg.prev].next = pg.next;
        else keep_head_ = pg.next;
        if (pg.next != kNoPage) page_[pg.next].prev = pg.prev;
        else keep_tail_ = pg.prev;
        pg.prev = pg.next = kNoPage;
        pg.in_keep = false;
        --kept_;
    }

    std::vector<Page> page_;
    std::vector<PageId> blank_;
    std::unordered_map<uint64_t, PageId> by_name_;
    PageId keep_head_ = kNoPage, keep_tail_ = kNoPage;
    int kept_ = 0;
};

// A request's logical-to-physical map in one group: token i lives in pages[i / page_size] at
// offset i % page_size.  In a window group the leading entries become kNoPage once released.
struct SeqTable {
    std::vector<PageId> pages;
    size_t num_tokens = 0;   // tokens that have a slot reserved
    size_t first_live = 0;   // pages before this index were given back
};

class CacheManager {
public:
    CacheManager(std::vector<GroupConfig> groups, int num_state_slots)
        : groups_(std::move(groups)) {
        for (auto& g : groups_) {
            if (g.page_size <= 0 || g.num_pages < 0 || g.window < 0)
                throw std::invalid_argument("cache group needs page_size > 0, num_pages >= 0, window >= 0");
            pools_.emplace_back(g.num_pages);
        }
        for (int s = num_state_slots - 1; s >= 0; --s) free_slots_.push_back(s);
        num_state_slots_ = num_state_slots;
    }

    int num_groups() const { return static_cast<int>(groups_.size()); }
    const GroupConfig& group(int g) const { return groups_.at(g); }
    int num_free_pages(int g) const { return pools_.at(g).num_free(); }
    int num_cached_pages(int g) const { return pools_.at(g).num_evictable(); }
    int num_free_state_slots() const { return static_cast<int>(free_slots_.size()); }
    int num_state_slots() const { return num_state_slots_; }
    bool contains(SeqId s) const { return tables_.count(s) != 0; }

    size_t pages_for(int g, size_t tokens) const {
        const size_t ps = groups_[g].page_size;
        return (tokens + ps - 1) / ps;
    }

    // Fraction of pages held by requests, over all groups (cached-but-unused pages do not count).
    double utilization() const {
        size_t total = 0, used = 0;
        for (size_t g = 0; g < groups_.size(); ++g) {
            total += pools_[g].num_pages();
            used += pools_[g].num_pages() - pools_[g].num_free();
        }
        return total ? double(used) / double(total) : 0.0;
    }

    // Prefix reuse needs every group to keep all tokens and to share one page size.
    bool prefix_reuse_possible() const {
        if (groups_.empty()) return false;
        for (auto& g : groups_)
            if (g.window != 0 || g.page_size != groups_[0].page_size) return false;
        return true;
    }

    // Pages that reserve(seq, total) would take from group g.
    size_t pages_needed(SeqId seq, int g, size_t total_tokens) const {
        auto it = tables_.find(seq);
        size_t have_pages = 0, have_tokens = 0;
        if (it != tables_.end()) {
            have_pages = it->second[g].pages.size();
            have_tokens = it->second[g].num_tokens;
        }
        if (total_tokens <= have_tokens) return 0;
        size_t want = pages_for(g, total_tokens);
        return want > have_pages ? want - have_pages : 0;
    }

    // Ensures slots for tokens [0, total_tokens) in every group (`windows_too`) or in the groups
    // that keep all tokens only.  All or nothing: on false nothing has changed.
    bool reserve(SeqId seq, size_t total_tokens, bool windows_too = true) {
        for (size_t g = 0; g < groups_.size(); ++g) {
            if (!windows_too && groups_[g].window != 0) continue;
            if (pages_needed(seq, int(g), total_tokens) > size_t(pools_[g].num_free())) return false;
        }
        auto& tabs = table_entry(seq);
        for (size_t g = 0; g < groups_.size(); ++g) {
            if (!windows_too && groups_[g].window != 0) continue;
            SeqTable& t = tabs[g];
            if (total_tokens <= t.num_tokens) continue;
            const size_t want = pages_for(int(g), total_tokens);
            while (t.pages.size() < want) {
                PageId b = pools_[g].allocate();
                if (b == kNoPage) throw std::logic_error("free count was checked");
                t.pages.push_back(b);
            }
            t.num_tokens = total_tokens;
        }
        return true;
    }

    // Tokens [0, num_computed) are in the cache and every later query sits at a position
    // >= num_computed.  In a group with window W such a query sees keys > position - W only,
    // so a page whose last token index is <= num_computed - W is given back.
    // Returns the number of pages released.
    int release_behind(SeqId seq, size_t num_computed) {
        auto it = tables_.find(seq);
        if (it == tables_.end()) return 0;
        int released = 0;
        for (size_t g = 0; g < groups_.size(); ++g) {
            const size_t W = groups_[g].window, ps = groups_[g].page_size;
            if (W == 0 || num_computed < W) continue;
            SeqTable& t = it->second[g];
            const size_t dead_upto = num_computed - W;  // token indices <= this are never read again
            while (t.first_live < t.pages.size() && (t.first_live + 1) * ps - 1 <= dead_upto) {
                PageId b = t.pages[t.first_live];
                if (b != kNoPage) {
                    pools_[g].decref(b);
                    t.pages[t.first_live] = kNoPage;
                    ++released;
                }
                ++t.first_live;
            }
        }
        return released;
    }

    // Gives back every page and the state slot of `seq`.  Unknown requests are ignored.
    void free(SeqId seq) {
        auto it = tables_.find(seq);
        if (it != tables_.end()) {
            for (size_t g = 0; g < groups_.size(); ++g)
                for (PageId b : it->second[g].pages)
                    if (b != kNoPage) pools_[g].decref(b);
            tables_.erase(it);
        }
        auto st = slot_of_.find(seq);
        if (st != slot_of_.end()) {
            free_slots_.push_back(st->second);
            slot_of_.erase(st);
        }
    }

    // The request's fixed-size state slot; taken on first use, -1 when none is left.
    int acquire_state_slot(SeqId seq) {
        auto st = slot_of_.find(seq);
        if (st != slot_of_.end()) return st->second;
        if (free_slots_.empty()) return -1;
        int s = free_slots_.back();
        free_slots_.pop_back();
        slot_of_[seq] = s;
        return s;
    }

    int state_slot(SeqId seq) const {
        auto st = slot_of_.find(seq);
        return st == slot_of_.end() ? -1 : st->second;
    }

    const std::vector<PageId>& table(SeqId seq, int g) const {
        static const std::vector<PageId> empty;
        auto it = tables_.find(seq);
        return it == tables_.end() ? empty : it->second.at(g).pages;
    }

    size_t reserved_tokens(SeqId seq, int g) const {
        auto it = tables_.find(seq);
        return it == tables_.end() ? 0 : it->second.at(g).num_tokens;
    }

    // ---- prefix reuse (only when prefix_reuse_possible()) ----

    // How many leading hashes are cached in every group, and per group how many of those pages
    // are evictable now (adopting them takes them out of the free count).
    size_t prefix_match(const std::vector<uint64_t>& hashes, std::vector<int>* evictable) const {
        size_t n = hashes.size();
        for (size_t g = 0; g < groups_.size(); ++g) {
            size_t m = 0;
            while (m < n && pools_[g].lookup(hashes[m]) != kNoPage) ++m;
            n = std::min(n, m);
        }
        if (evictable) {
            evictable->assign(groups_.size(), 0);
            for (size_t g = 0; g < groups_.size(); ++g)
                for (size_t i = 0; i < n; ++i)
                    if (pools_[g].refcount(pools_[g].lookup(hashes[i])) == 0) ++(*evictable)[g];
        }
        return n;
    }

    // Whether a request of `num_tokens` tokens whose first `matched` pages are cached fits now,
    // leaving `watermark(g)` pages free in every group.  A window group is asked for what the
    // request can hold there at once: its window plus one portion of `portion_tokens`.
    bool fits(size_t num_tokens, size_t portion_tokens, size_t matched,
              const std::vector<int>& matched_evictable) const {
        for (size_t g = 0; g < groups_.size(); ++g) {
            const size_t toks = groups_[g].window ? std::min(num_tokens, size_t(groups_[g].window) + portion_tokens) : num_tokens;
            const size_t need = pages_for(int(g), toks) - std::min(matched, pages_for(int(g), toks));
            const long avail = long(pools_[g].num_free()) - (g < matched_evictable.size() ? matched_evictable[g] : 0);
            if (long(need) + long(watermark(int(g))) > avail) return false;
        }
        return true;
    }

    // Pages kept free at admission so that running requests can grow
    // (crates/engine/src/engine.rs:268: max(1, pages / 100)).
    int watermark(int g) const { return watermark_ >= 0 ? watermark_ : std::max(1, groups_[g].num_pages / 100); }
    // A fixed number of pages instead of the default rule; negative restores the rule.
    void set_watermark(int pages) { watermark_ = pages; }

    // Longest request that can ever be admitted.
    size_t max_seq_tokens() const {
        size_t best = SIZE_MAX;
        for (size_t g = 0; g < groups_.size(); ++g) {
            if (groups_[g].window != 0) continue;
            long pages = long(groups_[g].num_pages) - watermark(int(g));
            best = std::min(best, size_t(std::max(0l, pages)) * groups_[g].page_size);
        }
        return best;
    }

    // What `admit` did for a request.
    struct Admission {
        bool ok = false;
        size_t cached_pages = 0;     // leading pages found in the cache and taken over
        uint64_t chain = 0;          // hash of the last of them (0: none)
    };

    // Admission as one transaction: the request `seq` with `n` known tokens gets, or does not get,
    // everything it needs to start: the cached pages of its prefix (never the page that holds its
    // last token: that token's logits are wanted, so it has to be computed), room for all `n` tokens
    // in the groups that keep every token (reserved now, so that a later admission cannot take it;
    // window groups are reserved portion by portion) with `watermark` pages to spare in every group,
    // and a state slot.  When anything is missing nothing has changed.
    Admission admit(SeqId seq, const int32_t* tokens, size_t n, size_t portion_tokens, bool use_prefix) {
        Admission out;
        if (n == 0 || tables_.count(seq) || slot_of_.count(seq)) throw std::logic_error("admit: request is empty or holds something already");
        std::vector<uint64_t> names;
        if (use_prefix && prefix_reuse_possible()) names = page_hashes(tokens, n - 1, groups_[0].page_size);
        std::vector<int> kept;
        const size_t found = prefix_match(names, &kept);
        if (!fits(n, portion_tokens, found, kept) || free_slots_.empty()) return out;
        if (found > 0) {
            adopt_prefix(seq, names, found);
            out.chain = names[found - 1];
        }
        acquire_state_slot(seq);
        if (!reserve(seq, n, /*windows_too=*/false)) throw std::logic_error("admit: room was checked");
        out.ok = true;
        out.cached_pages = found;
        return out;
    }

    // Starts `seq` on the cached pages of the first n hashes (all full pages).
    size_t adopt_prefix(SeqId seq, const std::vector<uint64_t>& hashes, size_t n) {
        if (tables_.count(seq)) throw std::logic_error("adopt into a request that already holds pages");
        if (n == 0) return 0;
        auto& tabs = table_entry(seq);
        for (size_t g = 0; g < groups_.size(); ++g) {
            for (size_t i = 0; i < n; ++i) {
                PageId b = pools_[g].lookup(hashes[i]);
                if (b == kNoPage) throw std::logic_error("adopting a page that is not cached");
                pools_[g].acquire(b);
                tabs[g].pages.push_back(b);
            }
            tabs[g].num_tokens = n * groups_[g].page_size;
        }
        return n;
    }

    // Page `index` of `seq` is full and computed: enter it in the registry under `hash`.
    void register_page(SeqId seq, size_t index, uint64_t hash) {
        auto it = tables_.find(seq);
        if (it == tables_.end()) return;
        for (size_t g = 0; g < groups_.size(); ++g) {
            auto& pages = it->second[g].pages;
            if (index < pages.size() && pages[index] != kNoPage) pools_[g].register_page(pages[index], hash);
        }
    }

    // Empty string when consistent: every table has exactly the pages its tokens need, every
    // count equals the number of tables holding the page, no page is free and held, free twice,
    // or lost; every state slot is free or held by exactly one request.
    std::string check_invariants() const {
        for (size_t g = 0; g < groups_.size(); ++g) {
            std::vector<uint32_t> holders(pools_[g].num_pages(), 0);
            for (auto& kv : tables_) {
                const SeqTable& t = kv.second[g];
                if (t.pages.size() < pages_for(int(g), t.num_tokens) ||
                    (groups_[g].window == 0 && t.pages.size() != pages_for(int(g), t.num_tokens))) {
                    std::ostringstream e;
                    e << "request " << kv.first << " group " << g << ": " << t.pages.size() << " pages for " << t.num_tokens << " tokens";
                    return e.str();
                }
                for (size_t i = 0; i < t.pages.size(); ++i) {
                    PageId b = t.pages[i];
                    if ((b == kNoPage) != (i < t.first_live)) {
                        std::ostringstream e;
                        e << "request " << kv.first << " group " << g << ": page entry " << i << " and first live page " << t.first_live << " disagree";
                        return e.str();
                    }
                    if (b != kNoPage) {
                        if (b < 0 || b >= pools_[g].num_pages()) return "page id out of range";
                        ++holders[b];
                    }
                }
            }
            std::string e = pools_[g].check(holders);
            if (!e.empty()) return "group " + std::to_string(g) + ": " + e;
        }
        std::vector<char> seen(num_state_slots_, 0);
        for (int s : free_slots_) { if (s < 0 || s >= num_state_slots_ || seen[s]++) return "state slot free twice or out of range"; }
        for (auto& kv : slot_of_) { if (kv.second < 0 || kv.second >= num_state_slots_ || seen[kv.second]++) return "state slot held twice, or held and free"; }
        for (int s = 0; s < num_state_slots_; ++s) if (!seen[s]) return "state slot " + std::to_string(s) + " is lost";
        return "";
    }

private:
    std::vector<SeqTable>& table_entry(SeqId seq) {
        auto it = tables_.find(seq);
        if (it == tables_.end()) it = tables_.emplace(seq, std::vector<SeqTable>(groups_.size())).first;
        return it->second;
    }

    std::vector<GroupConfig> groups_;
    std::vector<PagePool> pools_;
    std::unordered_map<SeqId, std::vector<SeqTable>> tables_;
    std::vector<int> free_slots_;
    std::unordered_map<SeqId, int> slot_of_;
    int num_state_slots_ = 0;
    int watermark_ = -1;
};

}  // namespace rlis
