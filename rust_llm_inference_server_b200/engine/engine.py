"""The engine loop: admits requests, lets the scheduler cut each step, runs the step function,
samples, finishes and frees.

Role of `Engine::{iterate, step}` and `Sequence::accept` (crates/engine/src/engine.rs:500-531,
617-726, 404-429) without the thread, channels and text side: token ids in, token ids out.
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
from .runner import ModelRunner, StepEntry


class RequestError(ValueError):
    """A request the engine refuses at intake (crates/engine/src/engine.rs:332-356)."""


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: list
    token_ids: list
    finish_reason: str            # "stop" (end-of-sequence token) or "length" (max_tokens)
    ttft: float                   # seconds from arrival to the first token
    decode_time: float            # seconds from the first token to the last

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
            size_groups(groups, cfg.kv_cache_bytes, elem)
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
        self._params_host = torch.empty((cfg.max_num_seqs, 2), dtype=torch.int32, pin_memory=True)
        self._params_dev = torch.empty((cfg.max_num_seqs, 2), dtype=torch.int32, device=model.device)
        self._ids_dev = torch.empty((cfg.max_num_seqs,), dtype=torch.int32, device=model.device)
        self._ids_host = torch.empty((cfg.max_num_seqs,), dtype=torch.int32, pin_memory=True)
        self._fparams_host = torch.empty((cfg.max_num_seqs, 5), dtype=torch.int32, pin_memory=True)
        self._fparams_dev = torch.empty((cfg.max_num_seqs, 5), dtype=torch.int32, device=model.device)
        self._fids_dev = torch.zeros((cfg.max_num_seqs,), dtype=torch.int32, device=model.device)
        self._fids_host = torch.zeros((cfg.max_num_seqs,), dtype=torch.int32, pin_memory=True)
        self._sampled = torch.cuda.Event()      # the sampled ids have arrived in pinned memory

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
        return self.sched.has_work()

    # ---- one iteration ----

    def step(self) -> list:
        """Schedules, runs and samples one step; returns the requests that finished in it."""
        seqs, preempted = self.sched.schedule()
        self.stats.preemptions += len(preempted)
        if not seqs:
            self.last_step = StepEvent(0, 0, False, {}, [])
            if self.sched.has_work():
                # no progress is possible: fail everything rather than spin (engine.rs:516-522)
                ids = list(self.seqs)
                for sid in ids:
                    self.cancel(sid)
                raise RuntimeError(f"scheduler made no progress with {len(ids)} requests pending")
            return []
        entries = []
        sample_rows = []            # (sequence, row among the wanted rows)
        for sid, start, end in seqs:
            s = self.seqs[sid]
            caught_up = end == len(s.tokens)
            entries.append(StepEntry(sid, s.tokens[start:end], start, [end - start - 1] if caught_up else []))
            if caught_up:
                sample_rows.append(s)
        st = self.runner.prepare(entries)
        logits = self.runner.forward(st)
        self.stats.h2d_bytes += st.h2d_bytes
        self.stats.steps += 1
        self.stats.step_tokens += st.n_tokens
        for sid, start, end in seqs:
            self.sched.advance(sid, end)
        finished = []
        new_tokens = {}
        if sample_rows:
            tokens = self._sample(logits, sample_rows)
            now = time.perf_counter()
            for s, tok in zip(sample_rows, tokens):
                new_tokens[s.id] = int(tok)
                out = self._accept(s, int(tok), now)
                if out is not None:
                    finished.append(out)
        self._publish()
        self.last_step = StepEvent(st.n_tokens, st.n_seqs, st.all_decode, new_tokens, finished)
        return finished

    def _sample(self, logits: torch.Tensor, rows: list) -> list:
        """One token per caught-up request.  Greedy and temperature rows: the device's Gumbel-max
        kernel; top-k / top-p rows: the device's filtering kernel; rows with a repetition penalty:
        the host (crates/engine/src/engine.rs:643-708 has the same split, with all filtering on
        the host).  Only token ids come back, except for host rows."""
        n = len(rows)
        pos = [len(s.tokens) for s in rows]
        plain = [s.sampler.device_mode(p) for s, p in zip(rows, pos)]
        filt = [s.sampler.filtered_mode(p) if m is None else None for s, p, m in zip(rows, pos, plain)]
        out = [0] * n
        launched = False
        if any(m is not None for m in plain):
            ph = self._params_host.numpy().view(np.uint32)
            for i in range(n):
                ph[i] = plain[i] if plain[i] is not None else (0, 0)
            self._params_dev[:n].copy_(self._params_host[:n], non_blocking=True)
            ops.sample_rows(logits, self._params_dev[:n], self._ids_dev[:n])
            self._ids_host[:n].copy_(self._ids_dev[:n], non_blocking=True)
            self.stats.h2d_bytes += n * 8
            launched = True
        if any(f is not None for f in filt):
            fh = self._fparams_host.numpy().view(np.uint32)
            for i in range(n):
                fh[i] = filt[i] if filt[i] is not None else (float_bits(1.0), 1, float_bits(1.0), 0, 0)
            self._fparams_dev[:n].copy_(self._fparams_host[:n], non_blocking=True)
            ops.sample_filtered(logits, self._fparams_dev[:n], self._fids_dev[:n])
            self._fids_host[:n].copy_(self._fids_dev[:n], non_blocking=True)
            self.stats.h2d_bytes += n * 20
            launched = True
        if launched:
            self._sampled.record()                  # on the current stream
            self._sampled.synchronize()
            self.stats.d2h_bytes += n * 4
            a, b = self._ids_host[:n].tolist(), self._fids_host[:n].tolist()
            for i in range(n):
                if plain[i] is not None:
                    out[i] = a[i]
                elif filt[i] is not None:
                    out[i] = b[i]
        host_idx = [i for i in range(n) if plain[i] is None and filt[i] is None]
        if host_idx:
            sel = torch.tensor(host_idx, device=logits.device)
            rows_host = logits.index_select(0, sel).to("cpu").numpy()
            self.stats.d2h_bytes += rows_host.nbytes
            for j, i in enumerate(host_idx):
                s = rows[i]
                out[i] = s.sampler.sample_host(rows_host[j], s.tokens, pos[i])
        return out

    def _accept(self, s: _Sequence, token: int, now: float):
        """Records a sampled token; finishes the request on end-of-sequence (not appended) unless
        `ignore_eos`, or at `max_tokens` (engine.rs:404-429)."""
        if s.first_token_at is None:
            s.first_token_at = now
        if token in self.eos_ids and not s.ignore_eos:
            return self._finish(s, "stop", now)
        s.tokens.append(token)
        self.stats.generated_tokens += 1
        if len(s.tokens) - s.prompt_len >= s.max_tokens:
            return self._finish(s, "length", now)
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
