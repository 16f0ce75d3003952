"""Arrangements of parts into a block.

"prenorm" (crates/model/src/llama.rs:264-271): x += mixer(norm1(x)); x += feed_forward(norm2(x)).
The residual stream is float32; each addition is fused into the norm that follows it, so a block
takes (resid, pending delta) and returns (resid, its own pending delta).

In steps of a few rows a norm is a kernel that moves a few kilobytes.  Where the parts on both
sides of a norm say that they can (`Part.fuses_norms`) and the norm offers it (`Norm.sink`), the
block hands the norm's sink to the part before it, which adds its result to the residual stream in
its last product, and passes the `ops.ScaledRows` it gets back to the part after it, whose first
product applies the scale; "pending" is then such rows instead of a delta.  The same holds across
blocks: the model names the next block, and `entry_sink` answers for its first norm."""

from __future__ import annotations

from .. import ops
from .base import (build_feed_forward, build_mixer, build_norm, register_arrangement)


class PreNormBlock:
    def __init__(self, spec, dtype, device):
        self.norm1 = build_norm(spec.norm1, dtype, device)
        self.mixer = build_mixer(spec.mixer, dtype, device)
        self.norm2 = build_norm(spec.norm2, dtype, device)
        self.feed_forward = build_feed_forward(spec.feed_forward, dtype, device)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    chains_norms = True      # `forward` takes `next_block`

    def entry_sink(self, resid, step):
        """For the block that runs before this one: the sink of this block's first norm, if its
        mixer takes the rows that come out of it."""
        return self.norm1.sink(resid, step) if self.mixer.fuses_norms(step) else None

    def forward(self, resid, pending, step, cache, state, writes_cache=True, next_block=None):
        h = pending if isinstance(pending, ops.ScaledRows) else self.norm1.forward(resid, pending, step)
        mixer_fuses, ff_fuses = self.mixer.fuses_norms(step), self.feed_forward.fuses_norms(step)
        sink = self.norm2.sink(resid, step) if mixer_fuses and ff_fuses else None
        if sink is not None:
            h = self.mixer.forward(h, step, cache, state, writes_cache, sink=sink)
        else:
            a = self.mixer.forward(h, step, cache, state, writes_cache)
            h = self.norm2.forward(resid, a, step)
        sink = next_block.entry_sink(resid, step) if ff_fuses and next_block is not None else None
        if sink is not None:
            return resid, self.feed_forward.forward(h, step, sink=sink)
        return resid, self.feed_forward.forward(h, step)


register_arrangement("prenorm", PreNormBlock)
