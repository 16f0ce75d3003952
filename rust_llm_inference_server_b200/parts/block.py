"""Arrangements of parts into a block.

"prenorm" (crates/model/src/llama.rs:264-271): x += mixer(norm1(x)); x += feed_forward(norm2(x)).
The residual stream is float32; each addition is fused into the norm that follows it, so a block
takes (resid, pending delta) and returns (resid, its own pending delta)."""

from __future__ import annotations

from .base import (build_feed_forward, build_mixer, build_norm, register_arrangement)


class PreNormBlock:
    def __init__(self, spec, dtype, device):
        self.norm1 = build_norm(spec.norm1, dtype, device)
        self.mixer = build_mixer(spec.mixer, dtype, device)
        self.norm2 = build_norm(spec.norm2, dtype, device)
        self.feed_forward = build_feed_forward(spec.feed_forward, dtype, device)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    def forward(self, resid, delta, step, cache, state, writes_cache=True):
        h = self.norm1.forward(resid, delta, step)
        a = self.mixer.forward(h, step, cache, state, writes_cache)
        h = self.norm2.forward(resid, a, step)
        m = self.feed_forward.forward(h, step)
        return resid, m


register_arrangement("prenorm", PreNormBlock)
