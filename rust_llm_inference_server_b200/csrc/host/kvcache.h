// Paged cache bookkeeping: which physical pages hold which request's tokens.  Host logic only;
// the tensors live on the device and are addressed by the page ids handed out here.
//
// What it does, after crates/kvcache/src/lib.rs of akshajnad/rust_llm_inference_server
// (free list, reference counts, hashed-page prefix reuse with least-recently-freed reclaim,
// all-or-nothing reservation, invariants check), re-designed around *groups*: layers with the
// same cache needs (geometry, keep-all or a window) share one pool of pages and one block table
// per request.  A window group gives pages back once every later query has passed them.  Beside
// the pages sits a pool of fixed-size per-request state slots.
#pragma once

#include <algorithm>
#include <cstdint>
#include <map>
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

// One group's pages: free list (last in, first out), reference counts, and the registry of
// full pages by content hash.  A registered page whose count falls to zero stays cached
// ("evictable") and is reclaimed, oldest first, only when the free list is empty.
class PagePool {
public:
    explicit PagePool(int num_pages)
        : refcount_(num_pages, 0), has_hash_(num_pages, 0), hash_of_(num_pages, 0),
          evict_tick_(num_pages, 0) {
        free_.reserve(num_pages);
        for (int b = num_pages - 1; b >= 0; --b) free_.push_back(b);
    }

    int num_pages() const { return static_cast<int>(refcount_.size()); }
    int num_free() const { return static_cast<int>(free_.size() + evictable_.size()); }
    int num_evictable() const { return static_cast<int>(evictable_.size()); }
    uint32_t refcount(PageId b) const { return refcount_.at(b); }

    PageId lookup(uint64_t hash) const {
        auto it = cached_.find(hash);
        return it == cached_.end() ? kNoPage : it->second;
    }

    // First writer wins: a second page with the same content stays unregistered.
    void register_page(PageId b, uint64_t hash) {
        if (!has_hash_[b] && cached_.find(hash) == cached_.end()) {
            has_hash_[b] = 1;
            hash_of_[b] = hash;
            cached_[hash] = b;
        }
    }

    // Takes a reference to a registered page, reviving it if it was evictable.
    void acquire(PageId b) {
        if (evict_tick_[b] != 0) {
            evictable_.erase(evict_tick_[b]);
            evict_tick_[b] = 0;
        }
        ++refcount_[b];
    }

    PageId allocate() {
        PageId b;
        if (!free_.empty()) {
            b = free_.back();
            free_.pop_back();
        } else if (!evictable_.empty()) {
            auto it = evictable_.begin();
            b = it->second;
            evictable_.erase(it);
            evict_tick_[b] = 0;
            cached_.erase(hash_of_[b]);
            has_hash_[b] = 0;
        } else {
            return kNoPage;
        }
        if (refcount_[b] != 0) throw std::logic_error("allocated a page that is still referenced");
        refcount_[b] = 1;
        return b;
    }

    void decref(PageId b) {
        if (refcount_.at(b) == 0) throw std::logic_error("page " + std::to_string(b) + " freed twice");
        if (--refcount_[b] == 0) {
            if (has_hash_[b]) {
                evict_tick_[b] = ++tick_;
                evictable_[tick_] = b;
            } else {
                free_.push_back(b);
            }
        }
    }

    // Consistency of the pool with `holders[b]` = number of tables that hold page b.
    std::string check(const std::vector<uint32_t>& holders) const {
        const int n = num_pages();
        std::vector<char> in_free(n, 0);
        std::ostringstream err;
        for (PageId b : free_) {
            if (in_free[b]++) { err << "page " << b << " is on the free list twice"; return err.str(); }
            if (has_hash_[b]) { err << "free page " << b << " is still registered"; return err.str(); }
        }
        for (auto& kv : evictable_) {
            PageId b = kv.second;
            if (in_free[b]++) { err << "page " << b << " is both free and evictable"; return err.str(); }
            if (evict_tick_[b] != kv.first || !has_hash_[b]) { err << "evictable page " << b << " has stale bookkeeping"; return err.str(); }
        }
        size_t registered = 0;
        for (int b = 0; b < n; ++b) registered += has_hash_[b] ? 1 : 0;
        if (registered != cached_.size()) return "registered pages and cache entries disagree";
        for (auto& kv : cached_)
            if (!has_hash_[kv.second] || hash_of_[kv.second] != kv.first) { err << "cache entry points at page " << kv.second << " with another hash"; return err.str(); }
        for (int b = 0; b < n; ++b) {
            if (refcount_[b] != holders[b]) { err << "page " << b << ": count " << refcount_[b] << " but " << holders[b] << " tables hold it"; return err.str(); }
            if ((refcount_[b] == 0) != (in_free[b] != 0)) { err << "page " << b << ": count " << refcount_[b] << ", free or evictable: " << int(in_free[b]); return err.str(); }
        }
        return "";
    }

private:
    std::vector<uint32_t> refcount_;
    std::vector<PageId> free_;
    std::vector<char> has_hash_;
    std::vector<uint64_t> hash_of_;
    std::unordered_map<uint64_t, PageId> cached_;
    std::map<uint64_t, PageId> evictable_;  // by tick of the last release, oldest first
    std::vector<uint64_t> evict_tick_;      // 0 = not evictable
    uint64_t tick_ = 0;
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
    // leaving `watermark(g)` pages free in every group.  Window groups are asked for
    // `window_tokens` tokens only (what the next portion can need), not for the whole request.
    bool fits(size_t num_tokens, size_t window_tokens, size_t matched,
              const std::vector<int>& matched_evictable) const {
        for (size_t g = 0; g < groups_.size(); ++g) {
            const size_t toks = groups_[g].window ? std::min(num_tokens, window_tokens) : num_tokens;
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
