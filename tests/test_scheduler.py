"""The scheduler's decisions (C++, csrc/host/scheduler.h) without a GPU, driven by a fake executor.

The traces asserted here are the ones the reference asserts for the same situations
(crates/engine/src/scheduler.rs:486-766)."""

import random

import pytest

from rust_llm_inference_server_b200.cache import host

H = host()


def toks(i, n):
    return [i * 100000 + k for k in range(n)]


def sched(num_blocks, continuous=True, max_batched=64, prefix=False, watermark=1, max_seqs=8,
          block_size=4, groups=None):
    cfg = H.SchedulerConfig(max_seqs, max_batched, continuous, prefix, watermark)
    return H.Scheduler(cfg, groups or [H.GroupConfig(num_blocks, block_size, 0)])


def simulate(s, prompts, outputs, max_seqs=8, max_batched=None):
    """A fake executor: runs whatever is scheduled, "samples" token 7 whenever a sequence is
    caught up, finishes it after outputs[id] tokens."""
    produced = {}
    for i, p in enumerate(prompts):
        s.add(i, p)
    finished, max_batch = [], 0
    for _ in range(100000):
        if not s.has_work():
            return finished, max_batch
        seqs, pre = s.schedule()
        assert seqs, "no progress with work pending"
        assert len(seqs) <= max_seqs
        if max_batched:
            assert sum(e - b for _, b, e in seqs) <= max_batched
        max_batch = max(max_batch, len(seqs))
        for sid, b, e in seqs:
            ps = s.cache().group(0).page_size
            assert len(s.cache().table(sid, 0)) * ps >= e, "scheduled without slots"
            s.advance(sid, e)
            if s.is_caught_up(sid):
                produced[sid] = produced.get(sid, 0) + 1
                if produced[sid] == outputs[sid]:
                    s.remove(sid); finished.append(sid)
                else:
                    s.append_token(sid, 7)
        assert s.check() == ""
    raise AssertionError("simulation did not finish")


def test_everything_finishes_and_pages_return():
    s = sched(64)
    prompts = [toks(i, 1 + (i * 7) % 30) for i in range(20)]
    outputs = [1 + (i * 5) % 25 for i in range(20)]
    finished, max_batch = simulate(s, prompts, outputs)
    assert len(finished) == 20 and max_batch == 8
    assert s.cache().num_free_pages(0) == 64 and s.cache().num_free_state_slots() == 8


def test_memory_pressure_preempts_and_still_finishes():
    s = sched(12)
    finished, _ = simulate(s, [toks(i, 4) for i in range(8)], [20] * 8)
    assert len(finished) == 8 and s.num_preemptions() > 0
    assert s.cache().num_free_pages(0) == 12


def three_full():
    s = sched(3, watermark=0)
    for i in range(3):
        s.add(i, toks(i, 4))
    seqs, _ = s.schedule()
    assert len(seqs) == 3
    for sid, b, e in seqs:
        s.advance(sid, e); s.append_token(sid, 7)
    return s


def test_newest_running_sequence_is_the_victim():
    s = three_full()
    seqs, pre = s.schedule()
    assert pre == [2, 1] and seqs == [(0, 4, 5)]
    assert s.check() == ""


def test_preempted_are_readmitted_before_new_ones_and_recompute_everything():
    s = three_full()
    assert s.schedule()[1] == [2, 1]
    s.add(9, toks(9, 1))
    s.remove(0)
    seqs, _ = s.schedule()
    assert seqs == [(1, 0, 5)]        # oldest preempted first; the sampled token is recomputed too


def test_long_prompts_are_cut_by_the_token_budget():
    s = sched(64, max_batched=16)
    s.add(0, toks(0, 40))
    chunks = []
    for _ in range(3):
        (sid, b, e), = s.schedule()[0]
        s.advance(sid, e); chunks.append((b, e))
    assert chunks == [(0, 16), (16, 32), (32, 40)] and s.is_caught_up(0)


def test_decodes_come_before_a_new_long_prompt():
    s = sched(64, max_batched=16)
    s.add(0, toks(0, 4))
    (sid, b, e), = s.schedule()[0]
    s.advance(sid, e); s.append_token(0, 7)
    s.add(1, toks(1, 100))
    assert s.schedule()[0] == [(0, 4, 5), (1, 0, 15)]


def test_static_policy_waits_for_the_batch_to_drain():
    s = sched(64, continuous=False)
    s.add(0, toks(0, 4))
    (sid, b, e), = s.schedule()[0]
    s.advance(sid, e); s.append_token(0, 7)
    s.add(1, toks(1, 4))
    assert [x[0] for x in s.schedule()[0]] == [0]
    s.remove(0)
    assert [x[0] for x in s.schedule()[0]] == [1]
    s2 = sched(64, continuous=False)
    fin, _ = simulate(s2, [toks(i, n) for i, n in enumerate([3, 9, 1, 17, 5, 2, 8, 30, 4, 6])],
                      [5, 1, 9, 3, 7, 2, 4, 6, 8, 10])
    assert len(fin) == 10


def test_shared_prefix_is_adopted_not_recomputed():
    s = sched(64, prefix=True)
    prompt = list(range(40))
    s.add(0, prompt)
    assert s.schedule()[0] == [(0, 0, 40)]
    s.advance(0, 40); s.remove(0)
    s.add(1, prompt)                       # 9 full pages come from the cache; the page with the
    assert s.schedule()[0] == [(1, 36, 40)]  # last token is computed so that its logits exist
    s.add(2, prompt[:20] + list(range(900, 915)))
    seqs, _ = s.schedule()
    assert [x for x in seqs if x[0] == 2] == [(2, 20, 35)]
    assert (s.admitted_tokens(), s.cached_tokens()) == (40 + 40 + 35, 36 + 20)
    assert s.check() == ""


def test_cached_pages_make_recomputation_cheap():
    cfg = H.SchedulerConfig(8, 64, True, True, 0)
    s = H.Scheduler(cfg, [H.GroupConfig(3, 4, 0)])
    for i in range(3):
        s.add(i, toks(i, 4))
    for sid, b, e in s.schedule()[0]:
        s.advance(sid, e); s.append_token(sid, 7)
    assert s.schedule()[1] == [2, 1]
    s.remove(0)
    assert s.schedule()[0][0] == (1, 4, 5)


def test_sequences_of_one_step_cannot_share_uncomputed_pages():
    for blocks in (12, 24, 48):
        s = sched(blocks, prefix=True)
        shared = list(range(16))
        prompts = [shared + list(range(1000 * i, 1000 * i + 1 + i)) if i % 2 == 0 else toks(i, 9 + i)
                   for i in range(8)]
        fin, _ = simulate(s, prompts, [9, 4, 12, 3, 8, 6, 2, 11])
        assert len(fin) == 8 and s.cached_tokens() >= 16
        assert s.cache().num_free_pages(0) == blocks


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_finish_without_starvation_or_leaks(seed):
    rng = random.Random(seed)
    for trial in range(50):
        n = 1 + rng.randrange(30)
        blocks = 8 + rng.randrange(40)
        mb = 8 + rng.randrange(64)
        s = sched(blocks, continuous=(trial % 4 != 0), max_batched=mb, prefix=(trial % 3 == 0))
        cap = s.cache().max_seq_tokens()
        prompts, outputs = [], []
        for i in range(n):
            p = 1 + rng.randrange(cap // 2)
            prompts.append([rng.randrange(3) for _ in range(p)] if trial % 3 == 0 else toks(i, p))
            outputs.append(1 + rng.randrange(cap - p))
        fin, _ = simulate(s, prompts, outputs, max_batched=None if trial % 4 == 0 else mb)
        assert len(fin) == n, trial
        assert s.cache().num_free_pages(0) == blocks and s.cache().num_free_state_slots() == 8


def test_window_group_pages_cycle_during_a_long_run():
    groups = [H.GroupConfig(64, 4, 0), H.GroupConfig(10, 4, 8)]
    s = sched(0, max_batched=8, groups=groups)
    assert not s.config().prefix_caching        # switched off: a window group cannot share pages
    fin, _ = simulate(s, [toks(0, 30), toks(1, 5)], [40, 60], max_batched=8)
    assert sorted(fin) == [0, 1]
    assert s.cache().num_free_pages(1) == 10 and s.cache().num_free_pages(0) == 64


def test_bad_configurations_and_requests_are_refused():
    with pytest.raises(ValueError):
        sched(8, max_batched=4, max_seqs=8)   # must cover one decode token per sequence
    s = sched(8)
    with pytest.raises(ValueError):
        s.add(0, [])


def test_a_step_ahead_with_placeholders_registers_the_real_tokens():
    """The engine's decode-ahead: a placeholder is appended for the token still on the device, the
    next step is scheduled on it, the value arrives later, and only then is the step's progress
    recorded, so that a page it fills enters the prefix registry under its real tokens."""
    s = sched(32, prefix=True, block_size=4)
    prompt = toks(1, 6)
    s.add(0, prompt)
    (seqs, _) = s.schedule()
    assert [tuple(x) for x in seqs] == [(0, 0, 6)]
    s.advance(0, 6)
    # the token sampled by that step is still on the device: schedule the next step on a placeholder
    s.append_token(0, 0)
    (seqs, pre) = s.schedule()
    assert [tuple(x) for x in seqs] == [(0, 6, 7)] and not pre
    assert s.tokens(0, 6, 7) == [0]
    s.set_token(0, 6, 41)                                 # it arrives
    assert s.tokens(0, 0, 7) == prompt + [41]
    s.append_token(0, 0)                                  # and the step after is launched on the next placeholder
    s.advance(0, 7)
    (seqs, _) = s.schedule()
    assert [tuple(x) for x in seqs] == [(0, 7, 8)]
    s.set_token(0, 7, 42)
    s.advance(0, 8)                                       # the second page (tokens 4..7) is full: registered as 41, 42
    with pytest.raises(IndexError):
        s.set_token(0, 99, 1)
    s.set_token(12345, 0, 1)                              # an unknown request (finished meanwhile): ignored
    s.remove(0)
    # a second request with the same eight tokens finds both pages
    s.add(1, prompt + [41, 42, 5])
    (seqs, _) = s.schedule()
    assert [tuple(x) for x in seqs] == [(1, 8, 9)] and s.cached_tokens() == 8
    # had the page been registered with the placeholder, this request would have found one page only
    assert s.check() == ""


class FakeAheadEngine:
    """The engine's loop with decode-ahead (engine/engine.py: step, _may_run_ahead, _launch,
    _collect) over the host module alone: tokens are "sampled" as a function of the request and
    the position, so that the outcome can be compared with a loop that never runs ahead."""

    def __init__(self, s, prompts, max_tokens, check_pages=True, ahead=True):
        self.s, self.cache = s, s.cache()
        self.tokens = {i: list(p) for i, p in enumerate(prompts)}
        self.prompt_len = {i: len(p) for i, p in enumerate(prompts)}
        self.max_tokens, self.check_pages, self.ahead = max_tokens, check_pages, ahead
        self.done, self.inflight, self.fallbacks, self.preemptions, self.ahead_steps = {}, None, 0, 0, 0
        for i, p in enumerate(prompts):
            s.add(i, p)

    @staticmethod
    def sample(sid, pos):
        return (sid * 31 + pos * 7) % 97 + 1

    def may_run_ahead(self, cur):
        seqs, rows = cur
        if not self.ahead or not rows or len(rows) != len(seqs) or self.s.num_waiting():
            return False
        if any(sid not in self.tokens or len(self.tokens[sid]) + 1 - self.prompt_len[sid] >= self.max_tokens
               for sid in rows):
            return False
        if self.check_pages:
            need = sum(self.cache.pages_needed(sid, 0, len(self.tokens[sid]) + 1) for sid in rows)
            if need > self.cache.num_free_pages(0):
                return False
        return True

    def launch(self, prev):
        if prev is not None:
            for sid in prev[1]:
                self.s.append_token(sid, 0)
        seqs, pre = self.s.schedule()
        seqs = [tuple(x) for x in seqs]
        self.preemptions += len(pre)
        if prev is not None:
            want = [(sid, len(self.tokens[sid]), len(self.tokens[sid]) + 1) for sid in prev[1]]
            if pre or seqs != want:
                for sid in prev[1]:
                    self.s.drop_last_token(sid)
                self.fallbacks += 1
                return None
            self.ahead_steps += 1
            return (seqs, list(prev[1]))
        if not seqs:
            assert not self.s.has_work(), "no progress with work pending"
            return None
        rows = [sid for sid, b, e in seqs if e == len(self.tokens[sid])]
        for sid, b, e in seqs:
            self.s.advance(sid, e)
        return (seqs, rows)

    def collect(self, cur, nxt):
        for sid in cur[1]:
            if sid not in self.tokens:
                continue
            t = self.tokens[sid]
            t.append(self.sample(sid, len(t)))
            if len(t) - self.prompt_len[sid] >= self.max_tokens:
                self.done[sid] = self.tokens.pop(sid)
                self.s.remove(sid)
            elif nxt is not None:
                self.s.set_token(sid, len(t) - 1, t[-1])
            else:
                self.s.append_token(sid, t[-1])
        if nxt is not None:
            for sid, b, e in nxt[0]:
                if sid in self.tokens:
                    self.s.advance(sid, e)

    def run(self):
        for _ in range(100000):
            if not self.s.has_work() and self.inflight is None:
                return self.done
            cur, self.inflight = self.inflight, None
            if cur is None:
                cur = self.launch(None)
                if cur is None:
                    continue
            nxt = self.launch(cur) if self.may_run_ahead(cur) else None
            self.collect(cur, nxt)
            self.inflight = nxt
            assert self.s.check() == ""
            for sid, t in self.tokens.items():           # the scheduler's copy agrees with the engine's
                n = self.s.num_tokens(sid)
                assert self.s.tokens(sid, 0, len(t)) == t and n in (len(t), len(t) + 1)
        raise AssertionError("did not finish")


@pytest.mark.parametrize("case", [
    dict(pages=5, page=8, prompts=[8, 8], max_tokens=24),        # two requests, nobody waiting when pages run out
    dict(pages=4, page=16, prompts=[16, 16], max_tokens=40),
    dict(pages=9, page=4, prompts=[5, 9, 3], max_tokens=17),
])
def test_decode_ahead_never_meets_a_preemption_and_falls_back_when_it_would(case):
    """With too few pages for every running request to grow, a decode step has to preempt
    (crates/engine/src/scheduler.rs:227-246).  The engine asks the cache before it launches a step
    ahead, so the step that preempts is an ordinary one; without that check the plan of the step
    ahead differs from what was expected, the placeholders are taken back, and the loop goes on
    step by step.  Either way: the tokens of a loop that never runs ahead, all pages back."""
    def run(**kw):
        s = sched(case["pages"], block_size=case["page"], max_seqs=4, prefix=True)
        e = FakeAheadEngine(s, [toks(i + 1, n) for i, n in enumerate(case["prompts"])], case["max_tokens"], **kw)
        done = e.run()
        assert s.cache().num_free_pages(0) == case["pages"] and s.check() == ""
        return done, e
    base, eb = run(ahead=False)
    assert eb.preemptions > 0 and len(base) == len(case["prompts"])
    checked, ec = run()
    assert checked == base and ec.preemptions > 0 and ec.fallbacks == 0 and ec.ahead_steps > 0
    unchecked, eu = run(check_pages=False)
    assert unchecked == base and eu.preemptions > 0 and eu.fallbacks > 0


def test_a_token_sampled_for_a_request_that_was_preempted_meanwhile_is_kept():
    s = sched(3, block_size=4, max_seqs=2, watermark=0)
    s.add(0, toks(1, 4)); s.add(1, toks(2, 4))
    seqs, _ = s.schedule()
    for sid, b, e in seqs:
        s.advance(sid, e)
    s.append_token(0, 7); s.append_token(1, 7)            # both need a second page; one is left
    seqs, pre = s.schedule()
    assert [tuple(x) for x in seqs] == [(0, 4, 5)] and pre == [1]
    s.append_token(1, 9)                                  # the token of a step launched before the preemption
    assert s.tokens(1, 0, 6) == toks(2, 4) + [7, 9]
    s.drop_last_token(1)
    assert s.num_tokens(1) == 5
    s.drop_last_token(0)                                  # request 0: five tokens, four of them computed
    with pytest.raises(RuntimeError):
        s.drop_last_token(0)                              # a computed token is never taken back
