"""The engine loop: admits requests, lets the scheduler cut each step, runs the step function,
samples, finishes and frees.

Role of `Engine::{iterate, step}` and `Sequence::accept` (crates/engine/src/engine.rs:500-531,
617-726, 404-429) without the thread, channels and text side: token ids in, token ids out.

Decode-ahead.  While every running request decodes, the next step needs nothing from the host but
the tokens just sampled, and those are on the device already.  The engine then launches step k + 1
(its token ids copied on the device from step k's sampler output) before it waits for step k's
ids, so the host's work on step k (reading the ids, end-of-sequence checks, scheduling, packing
the next step) runs while the GPU computes.  A request that ends on an end-of-sequence token has
by then one more step in flight; that step's row is dropped when it arrives.  Tokens and their
order are those of the step-by-step loop (the reference's loop is step by step,
engine.rs:617-726).  A step is launched ahead only when every request's next token is known to
have a slot in the cache; when pages are short the loop goes step by step and the scheduler
preempts as it always does (scheduler.rs:227-246).  Should the plan of a step launched ahead still
differ from "every request, one token more", the placeholders are taken back and the loop falls
back to step by step: it never raises with placeholders in place.

Failures.  A step whose packing or launch raises fails the requests of that step only: each ends
with reason "error", gives back its pages and state slot, and the other requests go on
(engine.rs:516-528).  The kernels' bounded waits leave an error word on the device; it comes to
the host with every step's sampled ids, and a step that set it fails its requests the same way.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field

import numpy as np
import torch

from .. import ops
from ..cache import CacheStorage, host, plan_groups, size_groups
from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, float_bits
from ..ops import profile
from .runner import ModelRunner, StepEntry, StepError


class RequestError(ValueError):
    """A request the engine refuses at intake (crates/engine/src/engine.rs:332-356)."""


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: list
    token_ids: list
    finish_reason: str            # "stop" (end-of-sequence token), "length" (max_tokens) or "error"
    ttft: float                   # seconds from arrival to the first token
    decode_time: float            # seconds from the first token to the last
    error: str | None = None      # what failed, for finish_reason "error"

    @property
    def decode_tokens_per_sec(self) -> float:
        """(completion - 1) / decode_time (crates/engine/src/engine.rs:140-158)."""
        n = len(self.token_ids)
        return (n - 1) / self.decode_time if n > 1 and self.decode_time > 0 else 0.0


@dataclass
class _Sequence:
    id: int
    tokens: list
    prompt_len: int
    sampler: Sampler
    max_tokens: int
    ignore_eos: bool
    arrived: float
    first_token_at: float | None = None
    finished: bool = False


@dataclass
class _Launched:
    """A step that has been launched; its sampled ids may still be on their way to the host."""
    seqs: list                    # (request id, start, end) as scheduled
    rows: list                    # the _Sequence of each wanted row (requests whose tokens are all computed)
    n_tokens: int
    n_seqs: int
    all_decode: bool
    logits: object = None
    slot: int = 0                 # which pinned buffers and event hold its ids
    plain: list = field(default_factory=list)      # per row: parameters of the Gumbel-max kernel or None
    filt: list = field(default_factory=list)       # per row: parameters of the filtering kernel or None
    pos: list = field(default_factory=list)        # per row: index of the token being sampled
    ahead: bool = False           # launched before its input tokens were known to the host
    ids_dev: object = None        # device ids of all rows, when one kernel sampled them all
    prep_us: float = 0.0          # host time: scheduling, packing, upload
    forward_us: float = 0.0       # host time: launching the model
    sample_us: float = 0.0        # host time: launching the samplers


@dataclass
class StepEvent:
    """What one engine step did (the stream the reference sends as `Event`s,
    crates/engine/src/engine.rs:115-120, without the text)."""
    n_tokens: int
    n_seqs: int
    all_decoding: bool            # every scheduled request ran exactly one token
    new_tokens: dict              # request id -> token sampled in this step
    finished: list                # RequestOutput of the requests that ended in this step


@dataclass
class EngineStats:
    steps: int = 0
    generated_tokens: int = 0
    step_tokens: int = 0
    preemptions: int = 0
    admitted_tokens: int = 0
    prefix_hit_tokens: int = 0
    running: int = 0
    waiting: int = 0
    kv_utilization: float = 0.0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    failed_requests: int = 0      # requests ended with reason "error"
    ahead_fallbacks: int = 0      # steps planned ahead whose placeholders were taken back
    # host microseconds of the last step and summed over all steps (crates/engine/src/engine.rs:717-724
    # logs prep_us / forward_us / sample_us per step); `wait` is the time blocked on the sampled ids
    prep_us: float = 0.0
    forward_us: float = 0.0
    sample_us: float = 0.0
    wait_us: float = 0.0
    total_prep_us: float = 0.0
    total_forward_us: float = 0.0
    total_sample_us: float = 0.0
    total_wait_us: float = 0.0


class LLMEngine:
    def __init__(self, model, cfg: EngineConfig | None = None):
        cfg = cfg or EngineConfig()
        cfg.validate()
        self.cfg = cfg
        self.model = model
        h = host()
        groups = plan_groups(model.cache_slot_specs, cfg.block_size)
        elem = torch.tensor([], dtype=model.dtype).element_size()
        if cfg.num_blocks is not None:
            for g in groups:
                g.num_pages = int(cfg.num_blocks)
        else:
            size_groups(groups, cfg.kv_cache_bytes, elem, cfg.max_num_seqs,
                        max(cfg.max_batched_tokens, cfg.max_num_seqs))
        if any(g.num_pages < 2 for g in groups):
            raise ValueError(f"kv cache of {cfg.kv_cache_bytes} bytes holds fewer than 2 blocks")
        self.groups = groups
        max_batched = max(cfg.max_batched_tokens, cfg.max_num_seqs)   # engine.rs:265
        # A request that starts on cached pages skips the tokens they hold; a mixer with state of
        # its own would miss them, so prefix reuse is off for such models (and, inside the
        # scheduler, for models with a window group).
        has_state = any(s is not None for s in model.call_state_specs)
        sc = h.SchedulerConfig(cfg.max_num_seqs, max_batched, cfg.policy == "continuous",
                               cfg.prefix_caching and not has_state)
        self.sched = h.Scheduler(sc, [h.GroupConfig(g.num_pages, g.page_size, g.window) for g in groups])
        self.cache = self.sched.cache()
        self.storage = CacheStorage(groups, model.call_state_specs, cfg.max_num_seqs, model.dtype, model.device)
        # longest prompt plus completion: the option, the model's positions, and what the pool
        # can hold with the watermark to spare (engine.rs:263-280)
        self.max_seq_len = int(min(cfg.max_seq_len, model.spec.max_positions, self.cache.max_seq_tokens()))
        self.runner = ModelRunner(model, self.cache, self.storage, self.max_seq_len)
        self.runner.use_graphs = bool(cfg.cuda_graphs)
        self.eos_ids = set(model.spec.eos_token_ids)
        self.seqs: dict[int, _Sequence] = {}
        self._next_id = 0
        self.stats = EngineStats()
        # Two steps can be in flight (decode-ahead), so what the host writes or reads per step
        # exists twice: pinned parameter and id buffers and the event that says the ids arrived.
        # The device-side buffers are used in stream order and exist once.
        n = cfg.max_num_seqs
        pinned = lambda shape: [torch.zeros(shape, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._params_host, self._fparams_host = pinned((n, 2)), pinned((n, 5))
        self._ids_host, self._fids_host = pinned((n,)), pinned((n,))
        self._params_dev = torch.empty((n, 2), dtype=torch.int32, device=model.device)
        self._fparams_dev = torch.empty((n, 5), dtype=torch.int32, device=model.device)
        self._ids_dev = torch.zeros((n,), dtype=torch.int32, device=model.device)
        self._fids_dev = torch.zeros((n,), dtype=torch.int32, device=model.device)
        self._sampled = [torch.cuda.Event(), torch.cuda.Event()]
        self._pen_host = self._pen_dev = None      # histories of the rows with a repetition penalty
        self._slot = 0
        self._inflight: _Launched | None = None
        self._failed: list = []             # outputs of requests that failed with their step
        # the kernels' error word (bounded waits that ran out) travels with every step's ids
        self._err_dev = torch.zeros((1,), dtype=torch.int32, device=model.device)
        self._err_host = pinned((1,))
        self._decode_ahead = bool(cfg.decode_ahead)
        # (tests switch this off to reach the fallback of a step ahead whose plan is not the expected one)
        self._ahead_checks_pages = True

    # ---- intake ----

    def add_request(self, prompt_token_ids, params: SamplingParams | None = None) -> int:
        params = params or SamplingParams()
        params.validate()
        prompt = [int(t) for t in prompt_token_ids]
        if not prompt:
            raise RequestError("empty prompt or max_tokens of 0")
        V = self.model.spec.vocab_size
        if min(prompt) < 0 or max(prompt) >= V:
            raise RequestError(f"prompt holds a token id outside the vocabulary of {V}")
        total = len(prompt) + params.max_tokens
        if total > self.max_seq_len:
            raise RequestError(f"{total} tokens exceeds max_seq_len {self.max_seq_len}")
        sid = self._next_id
        self._next_id += 1
        self.seqs[sid] = _Sequence(sid, prompt, len(prompt), Sampler(params), params.max_tokens,
                                   params.ignore_eos, time.perf_counter())
        self.sched.add(sid, prompt)
        return sid

    def cancel(self, request_id: int) -> None:
        """Drops a request wherever it is and gives back what it holds (engine.rs:562-573)."""
        if self.seqs.pop(request_id, None) is not None:
            self.sched.remove(request_id)

    def has_work(self) -> bool:
        return self.sched.has_work() or self._inflight is not None

    # ---- one iteration ----

    def step(self) -> list:
        """One turn of the loop: makes sure a step is in flight, launches the one after it where
        that is possible (see the module's head), then reads the first one's tokens.  Returns the
        requests that ended with them (finished, or failed with their step)."""
        cur, self._inflight = self._inflight, None
        if cur is None:
            cur = self._launch(None)
        if cur is None:
            ended = self._take_failed()
            self._publish()
            self.last_step = StepEvent(0, 0, False, {}, ended)
            return ended
        nxt = self._launch(cur) if self._may_run_ahead(cur) else None
        new_tokens, finished = self._collect(cur, nxt)
        finished.extend(self._take_failed())
        self._inflight = nxt
        self._publish()
        self.last_step = StepEvent(cur.n_tokens, cur.n_seqs, cur.all_decode, new_tokens, finished)
        return finished

    def _may_run_ahead(self, cur: _Launched) -> bool:
        """The step after `cur` can be launched before `cur`'s tokens are known: every request of
        `cur` gets a token from the device (one kernel for all), goes on after it whatever it is,
        unless it is an end-of-sequence token, nobody waits to be admitted, and the cache has a
        slot for every request's next token (else the scheduler would have to preempt, and that
        is decided step by step)."""
        if not self._decode_ahead or not cur.rows or len(cur.rows) != len(cur.seqs) or cur.ids_dev is None:
            return False
        if self.sched.num_waiting() != 0:
            return False
        for s in cur.rows:
            if s.id not in self.seqs or len(s.tokens) + 1 - s.prompt_len >= s.max_tokens:
                return False
            if s.sampler.params.repetition_penalty != 1.0:      # its history has to be complete on the host
                return False
        # the step ahead computes the token that `cur` samples: index len(tokens), so len + 1 slots
        cache = self.cache
        for g in range(len(self.groups) if self._ahead_checks_pages else 0):
            need = sum(cache.pages_needed(s.id, g, len(s.tokens) + 1) for s in cur.rows)
            if need > cache.num_free_pages(g):
                return False
        return True

    def _launch(self, prev: _Launched | None) -> _Launched | None:
        """Schedules and launches a step and its sampler; waits for nothing.  With `prev`, the step
        is the one after `prev`, whose tokens are still on the device: every request gets a
        placeholder, and the token ids are copied on the device from `prev`'s sampler output.
        Returns None when nothing was launched: no work, the step's requests failed, or (with
        `prev`) the plan was not the expected one and the placeholders were taken back."""
        t0 = time.perf_counter()
        if prev is not None:
            for s in prev.rows:
                self.sched.append_token(s.id, 0)
        seqs, preempted = self.sched.schedule()
        self.stats.preemptions += len(preempted)
        if prev is not None:
            want = [(s.id, len(s.tokens), len(s.tokens) + 1) for s in prev.rows]
            if preempted or [tuple(x) for x in seqs] != want:
                # Not "everybody, one token more" after all.  What the plan reserved stays reserved,
                # a preempted request stays preempted (it recomputes with its real tokens later);
                # only the placeholders go, and `prev` is collected as a step on its own.
                for s in prev.rows:
                    self.sched.drop_last_token(s.id)
                self.stats.ahead_fallbacks += 1
                return None
        if not seqs:
            if self.sched.has_work():
                # no progress is possible: fail everything rather than spin (engine.rs:516-522)
                ids = list(self.seqs)
                for sid in ids:
                    self.cancel(sid)
                raise RuntimeError(f"scheduler made no progress with {len(ids)} requests pending")
            return None
        entries = []
        rows = []
        for sid, start, end in seqs:
            s = self.seqs[sid]
            if prev is not None:
                entries.append(StepEntry(sid, [0], start, [0]))
                rows.append(s)
                continue
            caught_up = end == len(s.tokens)
            entries.append(StepEntry(sid, s.tokens[start:end], start, [end - start - 1] if caught_up else []))
            if caught_up:
                rows.append(s)
        try:
            st = self.runner.prepare(entries)
            if prev is not None:
                st.take_tokens(prev.ids_dev[:len(rows)])
            t1 = time.perf_counter()
            logits = self.runner.forward(st)
            t2 = time.perf_counter()
            self.stats.h2d_bytes += st.h2d_bytes
            self.stats.steps += 1
            self.stats.step_tokens += st.n_tokens
            self._slot ^= 1
            out = _Launched(list(seqs), rows, st.n_tokens, st.n_seqs, st.all_decode, logits, self._slot,
                            ahead=prev is not None)
            if rows:
                with profile.span("sampler"):
                    self._enqueue_sampler(out)
        except (StepError, ops.KernelError) as err:
            # only this step's requests fail; the others go on (engine.rs:523-528)
            self._fail([sid for sid, _, _ in seqs], f"{type(err).__name__}: {err}")
            return None
        t3 = time.perf_counter()
        out.prep_us, out.forward_us, out.sample_us = (t1 - t0) * 1e6, (t2 - t1) * 1e6, (t3 - t2) * 1e6
        if prev is None:
            # (for a step launched ahead this waits until its input tokens are real: `_collect`)
            for sid, start, end in seqs:
                self.sched.advance(sid, end)
        return out

    def _fail(self, ids: list, why: str) -> None:
        """Ends the given requests with reason "error": pages and state slots go back, tokens
        generated so far are returned with the message."""
        now = time.perf_counter()
        for sid in ids:
            s = self.seqs.get(sid)
            if s is None:
                continue
            out = self._finish(s, "error", now)
            out.error = why
            self.stats.failed_requests += 1
            self._failed.append(out)

    def _take_failed(self) -> list:
        out, self._failed = self._failed, []
        return out

    def _enqueue_sampler(self, L: _Launched) -> None:
        """Launches the samplers of a step's wanted rows and the copy of their ids to pinned
        memory.  Greedy and temperature rows: the device's Gumbel-max kernel; top-k / top-p rows:
        the device's filtering kernel; a repetition penalty is applied to the logits on the device
        before either (crates/engine/src/engine.rs:643-708 samples greedy and temperature rows on
        the device and filters on the host)."""
        rows, n, k = L.rows, len(L.rows), L.slot
        self._penalise(L)
        L.pos = [len(s.tokens) + (1 if L.ahead else 0) for s in rows]
        L.plain = [s.sampler.device_mode(p) for s, p in zip(rows, L.pos)]
        L.filt = [s.sampler.filtered_mode(p) if m is None else None for s, p, m in zip(rows, L.pos, L.plain)]
        n_plain = sum(m is not None for m in L.plain)
        n_filt = sum(f is not None for f in L.filt)
        if n_plain:
            ph = self._params_host[k].numpy().view(np.uint32)
            for i in range(n):
                ph[i] = L.plain[i] if L.plain[i] is not None else (0, 0)
            self._params_dev[:n].copy_(self._params_host[k][:n], non_blocking=True)
            ops.sample_rows(L.logits, self._params_dev[:n], self._ids_dev[:n])
            self._ids_host[k][:n].copy_(self._ids_dev[:n], non_blocking=True)
            self.stats.h2d_bytes += n * 8
        if n_filt:
            fh = self._fparams_host[k].numpy().view(np.uint32)
            for i in range(n):
                fh[i] = L.filt[i] if L.filt[i] is not None else (float_bits(1.0), 1, float_bits(1.0), 0, 0)
            self._fparams_dev[:n].copy_(self._fparams_host[k][:n], non_blocking=True)
            ops.sample_filtered(L.logits, self._fparams_dev[:n], self._fids_dev[:n])
            self._fids_host[k][:n].copy_(self._fids_dev[:n], non_blocking=True)
            self.stats.h2d_bytes += n * 20
        if n_plain or n_filt:
            ops.take_device_errors(self._err_dev)
            self._err_host[k].copy_(self._err_dev, non_blocking=True)
            self._sampled[k].record()               # on the current stream
            self.stats.d2h_bytes += n * 4 + 4
        if n_plain == n:
            L.ids_dev = self._ids_dev
        elif n_filt == n:
            L.ids_dev = self._fids_dev

    def _penalise(self, L: _Launched) -> None:
        """Repetition penalties, on the device and in place on the step's logits, before the sampling
        kernels see them: the histories of the rows that have one go up in one copy.  (Such rows
        are never launched ahead: their history is complete on the host.)"""
        pen = [(i, s) for i, s in enumerate(L.rows) if s.sampler.params.repetition_penalty != 1.0]
        if not pen:
            return
        total = sum(len(s.tokens) for _, s in pen)
        n = len(pen)
        need = total + 3 * n + 1
        if self._pen_host is None or self._pen_host.numel() < need:
            size = max(need, 2 * (self._pen_host.numel() if self._pen_host is not None else 4096))
            self._pen_host = torch.zeros((size,), dtype=torch.int32, pin_memory=True)
            self._pen_dev = torch.zeros((size,), dtype=torch.int32, device=self.model.device)
        h = self._pen_host.numpy()
        # layout: rows [n], offsets [n + 1], penalties [n] (float bits), then the tokens
        o_off, o_pen, o_tok = n, 2 * n + 1, 3 * n + 1
        at = 0
        for j, (i, s) in enumerate(pen):
            h[j] = i
            h[o_off + j] = at
            h[o_pen + j] = np.float32(s.sampler.params.repetition_penalty).view(np.int32)
            h[o_tok + at:o_tok + at + len(s.tokens)] = s.tokens
            at += len(s.tokens)
        h[o_off + n] = at
        d = self._pen_dev
        d[:need].copy_(self._pen_host[:need], non_blocking=True)
        ops.repetition_penalty(L.logits, d[:n], d[o_tok:o_tok + total], d[o_off:o_off + n + 1],
                               d[o_pen:o_pen + n].view(torch.float32))
        self.stats.h2d_bytes += need * 4

    def _collect(self, L: _Launched, nxt: _Launched | None):
        """Waits for a launched step's ids, records the tokens and finishes requests.  `nxt`: the
        step launched after it with placeholders, which now get their values."""
        new_tokens, finished = {}, []
        rows, n, k = L.rows, len(L.rows), L.slot
        st = self.stats
        st.prep_us, st.forward_us, st.sample_us, st.wait_us = L.prep_us, L.forward_us, L.sample_us, 0.0
        if rows:
            t0 = time.perf_counter()
            self._sampled[k].synchronize()
            st.wait_us = (time.perf_counter() - t0) * 1e6
            code = self._device_error(k)
            if code:
                # a bounded wait ran out inside a kernel of this step (or of the one launched after
                # it): what they computed is not to be trusted
                ids = [s.id for s in rows] + ([s.id for s in nxt.rows] if nxt is not None else [])
                self._fail(ids, f"a bounded wait of a kernel ran out on the device (code {code}); "
                                "the step's results were dropped")
                return new_tokens, finished
            a, b = self._ids_host[k][:n].tolist(), self._fids_host[k][:n].tolist()
            tokens = [a[i] if L.plain[i] is not None else b[i] for i in range(n)]
            now = time.perf_counter()
            for s, tok in zip(rows, tokens):
                if s.id not in self.seqs:           # cancelled, or ended one step earlier (its row ran ahead)
                    continue
                new_tokens[s.id] = int(tok)
                out = self._accept(s, int(tok), now, placeholder=nxt is not None)
                if out is not None:
                    finished.append(out)
        st.total_prep_us += st.prep_us
        st.total_forward_us += st.forward_us
        st.total_sample_us += st.sample_us
        st.total_wait_us += st.wait_us
        if nxt is not None:
            # its input tokens are real now: pages they fill may enter the prefix registry
            for sid, start, end in nxt.seqs:
                if sid in self.seqs:
                    self.sched.advance(sid, end)
        return new_tokens, finished

    def _device_error(self, slot: int) -> int:
        """The kernels' error word as it came to the host with the ids of the step in `slot`."""
        return int(self._err_host[slot][0])

    def _accept(self, s: _Sequence, token: int, now: float, placeholder: bool = False):
        """Records a sampled token; finishes the request on end-of-sequence (not appended) unless
        `ignore_eos`, or at `max_tokens` (engine.rs:404-429).  `placeholder`: the scheduler holds
        a placeholder for this token already (the next step has been launched)."""
        if s.first_token_at is None:
            s.first_token_at = now
        if token in self.eos_ids and not s.ignore_eos:
            return self._finish(s, "stop", now)
        s.tokens.append(token)
        self.stats.generated_tokens += 1
        if len(s.tokens) - s.prompt_len >= s.max_tokens:
            return self._finish(s, "length", now)
        if placeholder:
            self.sched.set_token(s.id, len(s.tokens) - 1, token)
        else:
            self.sched.append_token(s.id, token)
        return None

    def _finish(self, s: _Sequence, reason: str, now: float) -> RequestOutput:
        s.finished = True
        self.sched.remove(s.id)
        del self.seqs[s.id]
        first = s.first_token_at if s.first_token_at is not None else now
        return RequestOutput(s.id, s.tokens[:s.prompt_len], s.tokens[s.prompt_len:], reason,
                             first - s.arrived, now - first)

    def _publish(self) -> None:
        st = self.stats
        st.running = self.sched.num_running()
        st.waiting = self.sched.num_waiting()
        st.kv_utilization = self.cache.utilization()
        st.admitted_tokens = self.sched.admitted_tokens()
        st.prefix_hit_tokens = self.sched.cached_tokens()

    def run_to_completion(self) -> list:
        done = []
        while self.has_work():
            done.extend(self.step())
        return done
