"""Trace replay: feeds given token ids through the model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the same model,
step function, cache manager and kernels that generation uses.  The reference has no such program;
its tests do the same by hand (teacher-forced steps in crates/model/tests/parity.rs:167-201,
explicit step tables over paged caches in crates/model/src/paged.rs:409-444).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, `<out>/<step>.f32` holds the float32 logits
[wanted, vocab], little-endian, in the order of the entries and of `want`.  After every step a
line `done <step>` is printed and flushed.
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch

from ..cache import CacheStorage, make_cache_manager, plan_groups
from ..models import load_model
from .runner import ModelRunner, StepEntry

REPLAY_PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 64


class ReplaySession:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = REPLAY_PAGE_SIZE,
                 device: str = "cuda"):
        if not torch.cuda.is_available():
            raise RuntimeError("trace replay needs a CUDA device; there is no CPU path")
        self.model = load_model(model_dir, dtype, device)
        groups = plan_groups(self.model.cache_slot_specs, page_size)
        if page_size <= 0:
            raise ValueError(f"page size must be positive, got {page_size}")
        # The pool holds exactly `max_tokens` tokens, so pages are used again as requests end.
        n_pages = max(1, (int(max_tokens) + page_size - 1) // page_size)
        for g in groups:
            g.num_pages = n_pages
        self.cache = make_cache_manager(groups, MAX_LIVE_REQUESTS)
        self.storage = CacheStorage(groups, self.model.call_state_specs, MAX_LIVE_REQUESTS,
                                    self.model.dtype, self.model.device)
        self.runner = ModelRunner(self.model, self.cache, self.storage,
                                  max_seq_len=n_pages * page_size)
        self._ids: dict[str, int] = {}
        self._count: dict[int, int] = {}
        self._next_id = 0

    def _seq(self, name) -> int:
        key = str(name)
        if key not in self._ids:
            self._ids[key] = self._next_id
            self._count[self._next_id] = 0
            self._next_id += 1
        return self._ids[key]

    def step(self, record: dict):
        """Runs one step; returns float32 logits [wanted, vocab] on the CPU, or None."""
        entries = []
        for e in record.get("entries", []):
            sid = self._seq(e["id"])
            toks = [int(t) for t in e["tokens"]]
            start = self._count[sid]
            if self.cache.acquire_state_slot(sid) < 0:
                raise RuntimeError(f"more than {MAX_LIVE_REQUESTS} live requests")
            if not self.cache.reserve(sid, start + len(toks)):
                raise RuntimeError(f"request {e['id']}: out of cache pages at {start + len(toks)} tokens "
                                   f"(the pool was made for --max-tokens)")
            entries.append(StepEntry(sid, toks, start, [int(w) for w in e.get("want", [])]))
        logits = None
        if entries:
            out = self.runner.step(entries)
            for en in entries:
                self._count[en.seq_id] += len(en.tokens)
                self.cache.release_behind(en.seq_id, self._count[en.seq_id])
            if out is not None:
                logits = out.to("cpu", torch.float32)
            else:
                torch.cuda.synchronize()
        for name in record.get("end", []):
            key = str(name)
            if key in self._ids:
                sid = self._ids.pop(key)
                self.cache.free(sid)
                self._count.pop(sid, None)
        return logits


def run_replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, stream=None,
               page_size: int = REPLAY_PAGE_SIZE) -> int:
    stream = stream if stream is not None else sys.stdin
    os.makedirs(out_dir, exist_ok=True)
    session = ReplaySession(model_dir, dtype, max_tokens, page_size)
    for line in stream:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = session.step(record)
        if logits is not None:
            arr = np.ascontiguousarray(logits.numpy(), dtype="<f4")
            tmp = os.path.join(out_dir, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        print(f"done {step}", flush=True)
    return 0
