"""Perplexity over a token stream, computed as the reference does (crates/engine/src/perplexity.rs:
26-80, the llama.cpp method): windows of `ctx` tokens, the first token of each replaced by the
begin-of-sequence id, and only the second half of each window scored, so every scored token has
at least ctx / 2 tokens of context."""

from __future__ import annotations

import math
import time
from dataclasses import asdict, dataclass

import torch

from .. import ops
from ..cache import CacheStorage, make_cache_manager, plan_groups
from .runner import ModelRunner, StepEntry


@dataclass
class Perplexity:
    ppl: float
    ppl_stderr: float       # one standard error, from the variance of the per-token NLL
    mean_nll: float
    tokens_scored: int
    windows: int
    ctx: int
    seconds: float

    def to_dict(self) -> dict:
        return asdict(self)


def perplexity(model, tokens, bos: int, ctx: int = 512, max_windows: int = 0, page_size: int = 16,
               progress=None) -> Perplexity:
    if ctx < 4:
        raise ValueError("ctx must be at least 4")
    windows = len(tokens) // ctx
    if max_windows > 0:
        windows = min(windows, max_windows)
    if windows <= 0:
        raise ValueError(f"corpus of {len(tokens)} tokens is shorter than one window of {ctx}")
    groups = plan_groups(model.cache_slot_specs, page_size)
    for g in groups:
        g.num_pages = (ctx + page_size - 1) // page_size
    cache = make_cache_manager(groups, 1)
    storage = CacheStorage(groups, model.call_state_specs, 1, model.dtype, model.device)
    runner = ModelRunner(model, cache, storage, max_seq_len=groups[0].num_pages * page_size if groups else ctx)
    first = ctx // 2
    total = total_sq = 0.0
    n = 0
    t0 = time.perf_counter()
    for w in range(windows):
        chunk = [int(t) for t in tokens[w * ctx:(w + 1) * ctx]]
        chunk[0] = int(bos)
        cache.acquire_state_slot(w)
        if not cache.reserve(w, ctx):
            raise RuntimeError("perplexity: the window does not fit its cache")
        # rows first .. ctx-2 predict tokens first+1 .. ctx-1; the last row has no target
        logits = runner.step([StepEntry(w, chunk, 0, list(range(first, ctx - 1)))])
        targets = torch.tensor(chunk[first + 1:], dtype=torch.int32, device=model.device)
        nll = ops.nll_rows(logits, targets).double().cpu()
        cache.free(w)
        total += float(nll.sum())
        total_sq += float((nll * nll).sum())
        n += nll.numel()
        if progress:
            progress(w + 1, windows, math.exp(total / n))
    mean = total / n
    var = max(total_sq / n - mean * mean, 0.0)
    ppl = math.exp(mean)
    return Perplexity(ppl, ppl * math.sqrt(var / n), mean, n, windows, ctx, time.perf_counter() - t0)
