"""Token selection: the key and parameters of the device sampler, and the host sampler for
top-k, top-p and repetition penalty.

Device path (crates/model/src/sampling.rs:11-63, crates/engine/src/sampler.rs:103-113): Gumbel-max
with noise keyed by (request seed, position of the token being generated), so a draw is
reproducible and does not depend on the batch.  Host path (crates/engine/src/sampler.rs:116-221):
repetition penalty, then greedy, or weights exp((l - max)/T) in float64, top-k (ties: lower id
first), nucleus against the whole vocabulary's mass (or the top-k set's), and an inverse-CDF draw.
The reference draws from a ChaCha8 stream per request; here the uniform comes from a counter hash
of (seed, position), which keeps the two properties the reference tests: same seed, same tokens;
and independence of the batch.
"""

from __future__ import annotations

import os
import struct

import numpy as np

from .params import SamplingParams

_M32 = 0xFFFFFFFF
_M64 = 0xFFFFFFFFFFFFFFFF


def lowbias32(x: int) -> int:
    x &= _M32
    x ^= x >> 16
    x = (x * 0x7FEB352D) & _M32
    x ^= x >> 15
    x = (x * 0x846CA68B) & _M32
    x ^= x >> 16
    return x


def row_key(seed: int, position: int) -> int:
    """Noise key of the token at `position` of a request seeded with `seed` (sampling.rs:21-23)."""
    seed &= _M64
    return lowbias32(lowbias32(lowbias32(seed & _M32) ^ (seed >> 32)) ^ (position & _M32))


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def unit_uniform(seed: int, position: int) -> float:
    """Uniform in [0, 1) from the top 53 bits of a hash of (seed, position)."""
    return (_splitmix64(_splitmix64(seed & _M64) ^ (position & _M64)) >> 11) * (1.0 / (1 << 53))


def float_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def random_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")


class Sampler:
    def __init__(self, params: SamplingParams):
        self.params = params
        self.seed = params.seed if params.seed is not None else random_seed()

    def device_mode(self, position: int):
        """(key, bits of 1/T) for the device sampler, or None when the row must go to the host."""
        p = self.params
        if not p.is_device_sampleable():
            return None
        if p.is_greedy():
            return (0, 0)
        inv_t = float(np.float32(1.0) / np.float32(p.temperature))
        return (row_key(self.seed, position), float_bits(inv_t))

    def sample_host(self, logits: np.ndarray, history, position: int) -> int:
        p = self.params
        logits = np.array(logits, dtype=np.float32, copy=True)
        if p.repetition_penalty != 1.0:
            seen = np.unique(np.asarray(list(history), dtype=np.int64))
            seen = seen[(seen >= 0) & (seen < len(logits))]
            vals = logits[seen]
            pen = np.float32(p.repetition_penalty)
            logits[seen] = np.where(vals > 0, vals / pen, vals * pen)
        if p.is_greedy():
            return int(np.argmax(logits))
        n = len(logits)
        w = np.exp((logits.astype(np.float64) - float(logits.max())) / float(p.temperature))
        top_k = 0 if (p.top_k == 0 or p.top_k >= n) else p.top_k
        u = unit_uniform(self.seed, position)
        if top_k == 0 and p.top_p >= 1.0:
            return _draw(np.arange(n), w, u)
        # descending by logit, ties lower id first (sampler.rs:182-195)
        order = np.lexsort((np.arange(n), -logits.astype(np.float64)))
        if top_k:
            order = order[:top_k]
        wk = w[order]
        total = wk.sum() if top_k else w.sum()
        if p.top_p < 1.0:
            acc = np.cumsum(wk / total)
            hit = np.nonzero(acc >= p.top_p)[0]
            keep = int(hit[0]) + 1 if len(hit) else len(order)
            order, wk = order[:keep], wk[:keep]
        return _draw(order, wk, u)


def _draw(ids: np.ndarray, weights: np.ndarray, u: float) -> int:
    """Inverse-CDF draw (sampler.rs:212-221)."""
    c = np.cumsum(weights)
    x = u * c[-1]
    i = int(np.searchsorted(c, x, side="right"))
    if i >= len(ids):
        nz = np.nonzero(weights > 0)[0]
        i = int(nz[-1]) if len(nz) else 0
    return int(ids[i])
