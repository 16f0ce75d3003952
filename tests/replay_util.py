"""Traces for the replay tests: the same requests replayed whole, with the last 32 tokens decoded
one by one, in portions of changing size, and mixed with other requests in a small pool."""

from __future__ import annotations

import numpy as np


def whole_trace(reqs: dict) -> list:
    """Each request alone and whole; logits at every position."""
    steps = []
    for i, (name, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": name, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [name]})
    return steps


def decode_trace(reqs: dict, tail: int = 32) -> list:
    """Most of a request in one step, the last `tail` tokens one by one."""
    steps, k = [], 0
    for name, toks in reqs.items():
        n = len(toks)
        head = max(1, n - tail)
        steps.append({"step": k, "entries": [{"id": name, "tokens": toks[:head], "want": [head - 1]}], "end": []})
        k += 1
        for i in range(head, n):
            steps.append({"step": k, "entries": [{"id": name, "tokens": [toks[i]], "want": [0]}],
                          "end": [name] if i == n - 1 else []})
            k += 1
        if head == n:
            steps[-1]["end"] = [name]
    return steps


def chunk_trace(reqs: dict, seed: int = 0) -> list:
    """Portions of changing size, down to two tokens (and ones)."""
    rng = np.random.default_rng(seed)
    sizes = [2, 7, 3, 16, 5, 33, 2, 17, 15, 1, 64, 9]
    steps, k = [], 0
    for name, toks in reqs.items():
        pos, j = 0, int(rng.integers(0, len(sizes)))
        while pos < len(toks):
            sz = min(sizes[j % len(sizes)], len(toks) - pos)
            j += 1
            steps.append({"step": k, "entries": [{"id": name, "tokens": toks[pos:pos + sz],
                                                   "want": list(range(sz))}],
                          "end": [name] if pos + sz == len(toks) else []})
            pos += sz
            k += 1
    return steps


def mixed_trace(reqs: dict, seed: int = 0, max_live: int = 4) -> list:
    """Up to `max_live` live requests: portions of some beside decoded tokens of others; a request
    may sit out a step.  Requests start as earlier ones end, so their pages are used again."""
    rng = np.random.default_rng(seed)
    pending = list(reqs.items())
    live: dict[str, list] = {}      # name -> [tokens, pos]
    steps, k = [], 0
    while pending or live:
        while pending and len(live) < max_live:
            name, toks = pending.pop(0)
            live[name] = [toks, 0]
        entries, ended = [], []
        for name in list(live):
            toks, pos = live[name]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            left = len(toks) - pos
            mode = rng.random()
            if mode < 0.4:
                sz = 1
            elif mode < 0.7:
                sz = int(rng.integers(2, 6))
            else:
                sz = int(rng.integers(6, 40))
            sz = min(sz, left)
            entries.append({"id": name, "tokens": toks[pos:pos + sz], "want": list(range(sz))})
            live[name][1] = pos + sz
            if pos + sz == len(toks):
                ended.append(name)
                del live[name]
        if entries:
            steps.append({"step": k, "entries": entries, "end": ended})
            k += 1
    return steps


def live_token_peak(steps: list, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held: dict[str, int] = {}
    peak = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for name in st["end"]:
            held.pop(name, None)
    return peak


def collect(session_or_fn, steps: list) -> dict:
    """Runs the steps; returns {(request, position): logits row}."""
    out, pos = {}, {}
    for st in steps:
        logits = session_or_fn(st)
        r = 0
        for e in st["entries"]:
            p0 = pos.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], p0 + w)] = logits[r].numpy().copy()
                r += 1
            pos[e["id"]] = p0 + len(e["tokens"])
        for name in st["end"]:
            pos.pop(name, None)
    return out
