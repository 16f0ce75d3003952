"""Named timing spans over the stages of a step, switched on by RLIS_PROFILE=1 (or `enable()`).

Role of `profile::span` / `take_report` (crates/model/src/profile.rs:22-49, call sites
crates/model/src/llama.rs:265-270, attention.rs:73-102, layers.rs:181-185).  The reference
synchronises the device before and after every stage; here a span is a pair of CUDA events on the
launching stream, so the kernels keep running back to back and the host is not stalled.  The times
are read, per name, when the report is taken.  While spans are on, steps are not replayed from
CUDA graphs (events inside a replayed graph carry no time), and kernels of neighbouring spans may
overlap by what programmatic dependent launch lets them (a few microseconds at most).

Off (the default), `span()` returns one shared object whose enter and exit do nothing.
"""

from __future__ import annotations

import os

import torch

enabled = os.environ.get("RLIS_PROFILE", "0") not in ("", "0")

_open: list = []        # (name, start event, end event) not yet read
_totals: dict = {}      # name -> [milliseconds, count]
_pool: list = []        # events to use again


class _Off:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_OFF = _Off()


class _Span:
    __slots__ = ("name", "start", "end")

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.start = _pool.pop() if _pool else torch.cuda.Event(enable_timing=True)
        self.end = _pool.pop() if _pool else torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.end.record()
        _open.append((self.name, self.start, self.end))
        if len(_open) >= 4096:
            _drain()
        return False


def span(name: str):
    """`with span("qkv proj"): ...` times what the block launches on the current stream."""
    return _Span(name) if enabled else _OFF


def enable(on: bool = True) -> None:
    global enabled
    enabled = bool(on)


def _drain() -> None:
    if not _open:
        return
    _open[-1][2].synchronize()
    for name, a, b in _open:
        b.synchronize()
        t = _totals.setdefault(name, [0.0, 0])
        t[0] += a.elapsed_time(b)
        t[1] += 1
        _pool.append(a)
        _pool.append(b)
    _open.clear()


def take_report() -> dict:
    """{name: (total milliseconds, spans)} since the last report, in the order the names were first
    seen; clears the totals.  Waits for the spans that are still running."""
    _drain()
    out = {k: (v[0], v[1]) for k, v in _totals.items()}
    _totals.clear()
    return out


def format_report(report: dict) -> str:
    total = sum(ms for ms, _ in report.values()) or 1.0
    lines = [f"{'stage':<24}{'ms':>10}{'spans':>8}{'share':>8}"]
    for name, (ms, n) in report.items():
        lines.append(f"{name:<24}{ms:>10.3f}{n:>8}{100 * ms / total:>7.1f}%")
    return "\n".join(lines)
