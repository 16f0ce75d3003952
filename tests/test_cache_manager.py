"""The cache manager (C++, csrc/host/kvcache.h) without a GPU: no page is lost, held twice or
freed twice, under random orders of requests; windows give pages back; state slots."""

import random

import pytest

from rust_llm_inference_server_b200.cache import host

H = host()


def mgr(pages=12, ps=4, window=0, slots=4, groups=None):
    groups = groups or [H.GroupConfig(pages, ps, window)]
    return H.CacheManager(groups, slots)


def test_reserve_grows_by_whole_pages_and_is_all_or_nothing():
    # expectations of crates/kvcache/src/lib.rs:446-532 restated for this manager
    m = mgr(pages=4, ps=4)
    assert m.reserve(1, 5) and m.table(1, 0) == [0, 1] and m.num_free_pages(0) == 2
    assert m.reserve(1, 8) and m.table(1, 0) == [0, 1]
    assert m.pages_needed(1, 0, 9) == 1
    before = (m.table(1, 0), m.num_free_pages(0))
    assert not m.reserve(2, 13)                       # needs 4 pages, 2 free
    assert (m.table(1, 0), m.num_free_pages(0)) == before and not m.contains(2)
    assert m.reserve(2, 8) and m.num_free_pages(0) == 0
    assert not m.reserve(1, 9)
    m.free(2)
    assert m.num_free_pages(0) == 2 and m.check_invariants() == ""
    assert m.reserve(1, 9) and m.table(1, 0)[-1] == 3  # last freed, first reused
    m.free(1)
    m.free(1)                                          # unknown requests are ignored
    assert m.num_free_pages(0) == 4 and m.utilization() == 0.0


def test_prefix_pages_are_shared_counted_and_reclaimed_oldest_first():
    m = mgr(pages=4, ps=2)
    toks = [5, 6, 7, 8, 9]
    hs = H.page_hashes(toks, 2)
    assert len(hs) == 2 and hs == H.page_hashes(toks[:4], 2)
    assert H.page_hashes([5, 6, 7, 9], 2)[0] == hs[0] and H.page_hashes([5, 6, 7, 9], 2)[1] != hs[1]
    assert H.next_page_hash(hs[0], [7, 8]) == hs[1]
    assert m.reserve(1, 5)
    m.register_page(1, 0, hs[0]); m.register_page(1, 1, hs[1])
    assert m.prefix_match(hs) == (2, [0])
    m.free(1)                                          # registered pages stay cached
    assert m.num_free_pages(0) == 4 and m.num_cached_pages(0) == 2
    assert m.prefix_match(hs) == (2, [2])
    assert m.adopt_prefix(2, hs, 2) == 2 and m.table(2, 0) == [0, 1]
    assert m.reserved_tokens(2, 0) == 4 and m.num_cached_pages(0) == 0
    assert m.adopt_prefix(3, hs, 1) == 1               # shared by two requests
    assert m.check_invariants() == ""
    m.free(2); m.free(3)
    # free list is used before cached pages; then the least recently freed cached page goes first
    assert m.reserve(4, 4) and set(m.table(4, 0)) == {2, 3}
    assert m.reserve(5, 2) and m.table(5, 0) == [1]    # page 1 was released before page 0
    assert m.prefix_match(hs) == (1, [1])
    assert m.check_invariants() == ""


def test_window_group_gives_pages_back_as_queries_pass():
    m = mgr(pages=6, ps=4, window=6)
    assert not m.prefix_reuse_possible()
    assert m.reserve(1, 16) and m.num_free_pages(0) == 2
    assert m.release_behind(1, 5) == 0                 # fewer tokens than the window
    # 12 computed, window 6: later queries (position >= 12) read keys > 6 only: page 0 (0..3) is dead,
    # page 1 (4..7) still holds key 7
    assert m.release_behind(1, 12) == 1 and m.table(1, 0)[:2] == [-1, 1]
    assert m.release_behind(1, 13) == 1 and m.table(1, 0)[:3] == [-1, -1, 2]   # key 7 is dead now
    assert m.num_free_pages(0) == 4 and m.check_invariants() == ""
    assert m.reserve(1, 24) and m.check_invariants() == ""
    m.free(1)
    assert m.num_free_pages(0) == 6 and m.check_invariants() == ""


def test_groups_reserve_together_or_not_at_all():
    m = mgr(groups=[H.GroupConfig(8, 4, 0), H.GroupConfig(2, 4, 8)])
    assert m.reserve(1, 8)
    before = m.num_free_pages(0)
    assert not m.reserve(2, 4)                         # group 1 is full
    assert m.num_free_pages(0) == before and not m.contains(2)
    assert m.reserve(2, 4, False)                      # groups that keep all tokens only
    assert m.table(2, 1) == [] and m.table(2, 0) == [2]
    assert m.max_seq_tokens() == (8 - 1) * 4
    assert m.check_invariants() == ""


def test_admission_is_one_transaction_over_pages_prefix_and_state_slots():
    """A request gets the cached pages of its prefix, room for all its tokens in the groups that
    keep everything, and a state slot, or nothing at all."""
    m = mgr(groups=[H.GroupConfig(8, 4, 0), H.GroupConfig(6, 4, 8)], slots=2)
    m.set_watermark(1)
    toks = list(range(20))
    assert m.admit(1, toks, 8) == (True, 0)              # (no prefix reuse with a window group)
    assert m.reserved_tokens(1, 0) == 20 and m.table(1, 1) == [] and m.state_slot(1) >= 0
    # the keep-all group has 3 pages left: 12 tokens and the watermark do not fit
    snapshot = (m.num_free_pages(0), m.num_free_pages(1), m.num_free_state_slots())
    assert m.admit(2, list(range(12)), 8) == (False, 0)
    assert (m.num_free_pages(0), m.num_free_pages(1), m.num_free_state_slots()) == snapshot and not m.contains(2)
    assert m.admit(2, list(range(8)), 8) == (True, 0)
    # no state slot left: nothing changes either
    snapshot = (m.num_free_pages(0), m.num_free_pages(1))
    assert m.admit(3, [1], 8) == (False, 0) and (m.num_free_pages(0), m.num_free_pages(1)) == snapshot
    with pytest.raises(RuntimeError):
        m.admit(1, toks, 8)                              # holds something already
    m.free(1); m.free(2)
    assert m.check_invariants() == ""
    # a window group is asked for its window plus one portion, not for the whole request
    w = mgr(groups=[H.GroupConfig(64, 4, 0), H.GroupConfig(5, 4, 8)], slots=2)
    w.set_watermark(0)
    assert w.admit(1, list(range(100)), 8) == (True, 0)      # 8 + 8 tokens: 4 of 5 pages
    assert w.admit(2, list(range(100)), 16) == (False, 0)    # 8 + 16 tokens: 6 pages
    # prefix reuse: the pages of a finished request are taken over, except the one with the last token
    p = mgr(pages=8, ps=4, slots=2)
    p.set_watermark(0)
    assert p.admit(1, toks, 8) == (True, 0)
    for i, h in enumerate(H.page_hashes(toks, 4)):
        p.register_page(1, i, h)
    p.free(1)
    assert p.admit(2, toks, 8) == (True, 4) and p.reserved_tokens(2, 0) == 20    # 5 full pages, 4 taken over
    assert p.admit(3, toks[:9] + [77, 78], 8, False) == (True, 0)                # asked not to look
    assert p.check_invariants() == ""


def test_state_slots_are_unique_and_return():
    m = mgr(slots=2)
    a, b = m.acquire_state_slot(1), m.acquire_state_slot(2)
    assert {a, b} == {0, 1} and m.acquire_state_slot(1) == a
    assert m.acquire_state_slot(3) == -1 and m.state_slot(3) == -1
    m.free(1)
    assert m.acquire_state_slot(3) == a and m.check_invariants() == ""


@pytest.mark.parametrize("seed", range(6))
def test_random_operations_keep_every_invariant(seed):
    """Role of the reference's property test (crates/kvcache/src/lib.rs:570-636): random
    reserve / free / register / adopt / release operations over a small pool."""
    rng = random.Random(seed)
    for _ in range(60):
        ps = rng.randint(1, 5)
        window = rng.choice([0, 0, 3, 7])
        groups = [H.GroupConfig(12, ps, 0)]
        if rng.random() < 0.5:
            groups.append(H.GroupConfig(rng.randint(4, 12), ps, window))
        m = H.CacheManager(groups, 5)
        tokens = {}      # request -> its token list
        computed = {}
        for _ in range(60):
            op = rng.choice(["reserve", "reserve", "free", "register", "adopt", "release", "slot"])
            seq = rng.randint(0, 5)
            if op == "reserve":
                total = rng.randint(1, 30)
                frees = [m.num_free_pages(g) for g in range(m.num_groups())]
                tabs = [m.table(seq, g) for g in range(m.num_groups())]
                ok = m.reserve(seq, total)
                if not ok:   # a failed reservation changes nothing
                    assert frees == [m.num_free_pages(g) for g in range(m.num_groups())]
                    assert tabs == [m.table(seq, g) for g in range(m.num_groups())]
                else:
                    toks = tokens.setdefault(seq, [])
                    while len(toks) < total:
                        toks.append(rng.randint(0, 2))
                    for g in range(m.num_groups()):
                        assert m.reserved_tokens(seq, g) >= total
            elif op == "free":
                m.free(seq); tokens.pop(seq, None); computed.pop(seq, None)
            elif op == "register" and seq in tokens and m.prefix_reuse_possible():
                hs = H.page_hashes(tokens[seq], ps)
                for i, h in enumerate(hs):
                    m.register_page(seq, i, h)
            elif op == "adopt" and not m.contains(seq) and m.prefix_reuse_possible():
                toks = [rng.randint(0, 2) for _ in range(rng.randint(1, 12))]
                hs = H.page_hashes(toks, ps)
                n, _ = m.prefix_match(hs)
                if n:
                    m.adopt_prefix(seq, hs, n)
                    tokens[seq] = toks[:n * ps]
            elif op == "release" and seq in tokens:
                c = rng.randint(computed.get(seq, 0), len(tokens[seq]))
                computed[seq] = c
                m.release_behind(seq, c)
            elif op == "slot":
                m.acquire_state_slot(seq)
            assert m.check_invariants() == "", (seed, op)
        for seq in range(6):
            m.free(seq)
        assert m.check_invariants() == ""
        for g in range(m.num_groups()):    # the full pool returns
            assert m.num_free_pages(g) == m.group(g).num_pages
        assert m.num_free_state_slots() == 5


def test_pool_sizing_caps_window_groups_at_what_they_can_hold():
    from rust_llm_inference_server_b200.cache import plan_groups, size_groups
    from rust_llm_inference_server_b200.parts import KVCacheSpec
    specs = [KVCacheSpec(2, 64, None), KVCacheSpec(2, 64, 128), KVCacheSpec(2, 64, None)]
    groups = plan_groups(specs, 16)
    assert [g.slots for g in groups] == [[0, 2], [1]] and [g.window for g in groups] == [0, 128]
    size_groups(groups, 1 << 26, 2)
    assert groups[0].num_pages == groups[1].num_pages            # no seats known: equal shares
    equal = groups[0].num_pages
    size_groups(groups, 1 << 26, 2, max_num_seqs=4, max_batched_tokens=256)
    assert groups[1].num_pages == 4 * ((128 + 256) // 16 + 2) and groups[0].num_pages > equal
    used = sum(g.num_pages * g.bytes_per_page(2) for g in groups)
    assert used <= 1 << 26 and (1 << 26) - used < sum(g.bytes_per_page(2) for g in groups)
