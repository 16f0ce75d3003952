// Python bindings of the host runtime (cache manager, scheduler, step packing).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "kvcache.h"
#include "scheduler.h"

namespace py = pybind11;
using namespace rlis;

namespace {

// Fills one step's index arrays for the kernels in a single pass (role of PagedBatch::new,
// crates/model/src/paged.rs:256-296, which the reference measured at 12 % of its engine's CPU
// time).  All arrays are int32 and preallocated by the caller:
//   positions[T], seq_of_token[T], slots[G][T], block_tables[G][B][max_blocks], ctx_lens[B],
//   cu_seqlens[B+1], state_slots[B].
// Raises if a position has no page reserved.
void pack_step(const CacheManager& cache, const std::vector<SeqId>& ids,
               const std::vector<int64_t>& starts, const std::vector<int64_t>& lens,
               py::array_t<int32_t> positions, py::array_t<int32_t> seq_of_token,
               py::array_t<int32_t> slots, py::array_t<int32_t> block_tables,
               py::array_t<int32_t> ctx_lens, py::array_t<int32_t> cu_seqlens,
               py::array_t<int32_t> state_slots) {
    const size_t B = ids.size();
    const int G = cache.num_groups();
    if (starts.size() != B || lens.size() != B) throw std::invalid_argument("pack_step: list lengths differ");
    size_t T = 0;
    for (auto l : lens) {
        if (l <= 0) throw std::invalid_argument("empty sequence in batch");
        T += size_t(l);
    }
    auto pos = positions.mutable_unchecked<1>();
    auto sot = seq_of_token.mutable_unchecked<1>();
    auto sl = slots.mutable_unchecked<2>();
    auto bt = block_tables.mutable_unchecked<3>();
    auto cl = ctx_lens.mutable_unchecked<1>();
    auto cu = cu_seqlens.mutable_unchecked<1>();
    auto ss = state_slots.mutable_unchecked<1>();
    if (size_t(pos.shape(0)) < T || size_t(sot.shape(0)) < T || sl.shape(0) < G || size_t(sl.shape(1)) < T ||
        bt.shape(0) < G || size_t(bt.shape(1)) < B || size_t(cl.shape(0)) < B || size_t(cu.shape(0)) < B + 1 ||
        size_t(ss.shape(0)) < B)
        throw std::invalid_argument("pack_step: an output array is too small");
    const size_t max_blocks = bt.shape(2);
    size_t t = 0;
    cu(0) = 0;
    for (size_t b = 0; b < B; ++b) {
        const size_t start = size_t(starts[b]), len = size_t(lens[b]);
        for (size_t i = 0; i < len; ++i) {
            pos(t + i) = int32_t(start + i);
            sot(t + i) = int32_t(b);
        }
        for (int g = 0; g < G; ++g) {
            const auto& pages = cache.table(ids[b], g);
            const size_t ps = cache.group(g).page_size;
            const size_t need = (start + len + ps - 1) / ps;
            if (pages.size() < need || cache.reserved_tokens(ids[b], g) < start + len)
                throw std::runtime_error("request " + std::to_string(ids[b]) + ": position " +
                                         std::to_string(start + len - 1) + " has no page reserved in cache group " + std::to_string(g));
            if (need > max_blocks) throw std::invalid_argument("pack_step: block table is narrower than the request");
            for (size_t p = 0; p < max_blocks; ++p) bt(g, b, p) = p < pages.size() ? pages[p] : kNoPage;
            for (size_t i = 0; i < len; ++i) {
                const size_t p = start + i;
                const PageId page = pages[p / ps];
                if (page == kNoPage) throw std::runtime_error("request " + std::to_string(ids[b]) + ": a new token falls in a page that was given back");
                sl(g, t + i) = int32_t(size_t(page) * ps + p % ps);
            }
        }
        cl(b) = int32_t(start + len);
        ss(b) = cache.state_slot(ids[b]);
        t += len;
        cu(b + 1) = int32_t(t);
    }
}

}  // namespace

PYBIND11_MODULE(_rlis_host, m) {
    m.doc() = "Host runtime of the engine: paged cache bookkeeping and the scheduler (C++).";

    py::class_<GroupConfig>(m, "GroupConfig")
        .def(py::init([](int num_pages, int page_size, int window) {
                 GroupConfig g; g.num_pages = num_pages; g.page_size = page_size; g.window = window; return g;
             }), py::arg("num_pages"), py::arg("page_size"), py::arg("window") = 0)
        .def_readwrite("num_pages", &GroupConfig::num_pages)
        .def_readwrite("page_size", &GroupConfig::page_size)
        .def_readwrite("window", &GroupConfig::window);

    m.def("page_hashes", [](const std::vector<int32_t>& tokens, int page_size) {
        return page_hashes(tokens.data(), tokens.size(), page_size);
    });
    m.def("next_page_hash", [](uint64_t prev, const std::vector<int32_t>& tokens) {
        return next_page_hash(prev, tokens.data(), tokens.size());
    });

    py::class_<CacheManager>(m, "CacheManager")
        .def(py::init<std::vector<GroupConfig>, int>(), py::arg("groups"), py::arg("num_state_slots"))
        .def("num_groups", &CacheManager::num_groups)
        .def("group", &CacheManager::group)
        .def("num_free_pages", &CacheManager::num_free_pages)
        .def("num_cached_pages", &CacheManager::num_cached_pages)
        .def("num_free_state_slots", &CacheManager::num_free_state_slots)
        .def("num_state_slots", &CacheManager::num_state_slots)
        .def("contains", &CacheManager::contains)
        .def("pages_for", &CacheManager::pages_for)
        .def("utilization", &CacheManager::utilization)
        .def("prefix_reuse_possible", &CacheManager::prefix_reuse_possible)
        .def("pages_needed", &CacheManager::pages_needed)
        .def("reserve", &CacheManager::reserve, py::arg("seq"), py::arg("total_tokens"), py::arg("windows_too") = true)
        .def("release_behind", &CacheManager::release_behind)
        .def("free", &CacheManager::free)
        .def("acquire_state_slot", &CacheManager::acquire_state_slot)
        .def("state_slot", &CacheManager::state_slot)
        .def("table", &CacheManager::table)
        .def("reserved_tokens", &CacheManager::reserved_tokens)
        .def("prefix_match", [](const CacheManager& c, const std::vector<uint64_t>& hashes) {
            std::vector<int> ev;
            size_t n = c.prefix_match(hashes, &ev);
            return py::make_tuple(n, ev);
        })
        .def("fits", &CacheManager::fits)
        .def("watermark", &CacheManager::watermark)
        .def("set_watermark", &CacheManager::set_watermark)
        .def("max_seq_tokens", &CacheManager::max_seq_tokens)
        .def("admit", [](CacheManager& c, SeqId seq, const std::vector<int32_t>& tokens, size_t portion_tokens, bool use_prefix) {
            CacheManager::Admission a = c.admit(seq, tokens.data(), tokens.size(), portion_tokens, use_prefix);
            return py::make_tuple(a.ok, a.cached_pages);
        }, py::arg("seq"), py::arg("tokens"), py::arg("portion_tokens"), py::arg("use_prefix") = true)
        .def("adopt_prefix", &CacheManager::adopt_prefix)
        .def("register_page", &CacheManager::register_page)
        .def("check_invariants", &CacheManager::check_invariants)
        .def("pack_step", [](const CacheManager& c, const std::vector<SeqId>& ids, const std::vector<int64_t>& starts,
                             const std::vector<int64_t>& lens, py::array_t<int32_t> positions,
                             py::array_t<int32_t> seq_of_token, py::array_t<int32_t> slots,
                             py::array_t<int32_t> block_tables, py::array_t<int32_t> ctx_lens,
                             py::array_t<int32_t> cu_seqlens, py::array_t<int32_t> state_slots) {
                 pack_step(c, ids, starts, lens, positions, seq_of_token, slots, block_tables, ctx_lens, cu_seqlens, state_slots);
             },
             py::arg("ids"), py::arg("starts"), py::arg("lens"), py::arg("positions").noconvert(),
             py::arg("seq_of_token").noconvert(), py::arg("slots").noconvert(),
             py::arg("block_tables").noconvert(), py::arg("ctx_lens").noconvert(),
             py::arg("cu_seqlens").noconvert(), py::arg("state_slots").noconvert());

    py::class_<SchedulerConfig>(m, "SchedulerConfig")
        .def(py::init([](int max_num_seqs, int max_batched_tokens, bool continuous, bool prefix_caching, int watermark_blocks) {
                 SchedulerConfig c; c.max_num_seqs = max_num_seqs; c.max_batched_tokens = max_batched_tokens;
                 c.continuous = continuous; c.prefix_caching = prefix_caching; c.watermark_blocks = watermark_blocks; return c;
             }), py::arg("max_num_seqs") = 64, py::arg("max_batched_tokens") = 2048,
             py::arg("continuous") = true, py::arg("prefix_caching") = true, py::arg("watermark_blocks") = -1)
        .def_readwrite("watermark_blocks", &SchedulerConfig::watermark_blocks)
        .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
        .def_readwrite("max_batched_tokens", &SchedulerConfig::max_batched_tokens)
        .def_readwrite("continuous", &SchedulerConfig::continuous)
        .def_readwrite("prefix_caching", &SchedulerConfig::prefix_caching);

    py::class_<Scheduler>(m, "Scheduler")
        .def(py::init<SchedulerConfig, std::vector<GroupConfig>>(), py::arg("config"), py::arg("groups"))
        .def("cache", &Scheduler::cache, py::return_value_policy::reference_internal)
        .def("config", &Scheduler::config)
        .def("add", &Scheduler::add)
        .def("schedule", [](Scheduler& s) {
            Schedule out = s.schedule();
            std::vector<std::tuple<SeqId, size_t, size_t>> seqs;
            for (auto& x : out.seqs) seqs.emplace_back(x.id, x.start, x.end);
            return py::make_tuple(seqs, out.preempted);
        })
        .def("advance", &Scheduler::advance)
        .def("append_token", &Scheduler::append_token)
        .def("set_token", &Scheduler::set_token)
        .def("drop_last_token", &Scheduler::drop_last_token)
        .def("num_tokens", &Scheduler::num_tokens)
        .def("is_caught_up", &Scheduler::is_caught_up)
        .def("remove", &Scheduler::remove)
        .def("tokens", &Scheduler::tokens)
        .def("has_work", &Scheduler::has_work)
        .def("num_running", &Scheduler::num_running)
        .def("num_waiting", &Scheduler::num_waiting)
        .def("num_preemptions", &Scheduler::num_preemptions)
        .def("admitted_tokens", &Scheduler::admitted_tokens)
        .def("cached_tokens", &Scheduler::cached_tokens)
        .def("check", &Scheduler::check);
}
