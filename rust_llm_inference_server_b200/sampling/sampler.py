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


def unit_uniform_53(seed: int, position: int) -> int:
    """The 53-bit integer behind `unit_uniform`: u = this / 2^53."""
    return _splitmix64(_splitmix64(seed & _M64) ^ (position & _M64)) >> 11


def order_keys(logits: np.ndarray) -> np.ndarray:
    """Order-preserving 32-bit image of float32 values (as the device kernel forms it)."""
    u = np.asarray(logits, dtype=np.float32).view(np.uint32)
    return np.where(u & np.uint32(0x80000000), ~u, u | np.uint32(0x80000000)).astype(np.uint32)


def filtered_draw(logits: np.ndarray, inv_t: np.float32, top_k: int, top_p: float, u53: int) -> int:
    """Top-k / top-p temperature sampling by the rule of csrc/kernels/sampling_filtered.cu, so that
    host and device pick the same token: fixed-point weights floor(exp((l - max) / T) * 2^40); the
    k highest logits and then the shortest descending prefix whose mass reaches top_p of the mass
    (ties: lower id first, the crossing token included); inverse CDF in vocabulary order with
    r = floor(u * kept mass)."""
    l = np.asarray(logits, dtype=np.float32)
    n = len(l)
    keys = order_keys(l)
    w = (np.exp(((l - l.max()) * np.float32(inv_t)).astype(np.float32)).astype(np.float32)
         * np.float32(2.0 ** 40)).astype(np.uint64)
    order = np.lexsort((np.arange(n), -keys.astype(np.int64)))          # descending logit, then id
    if 0 < top_k < n:
        order = order[:top_k]
    wk = w[order]
    mass = int(wk.sum(dtype=np.uint64))
    if np.float32(top_p) < np.float32(1.0):
        target = int(float(np.float32(top_p)) * float(mass))
        cum = np.cumsum(wk, dtype=np.uint64)                               # exact: the mass stays below 2^63
        hit = np.nonzero(cum >= np.uint64(max(target, 0)))[0]
        keep = int(hit[0]) + 1 if len(hit) else len(order)
        order = order[:max(keep, 1)]
    kept = np.zeros(n, dtype=bool)
    kept[order] = True
    wv = np.where(kept, w, np.uint64(0))
    total = int(wv.sum(dtype=np.uint64))
    if total == 0:
        return 0
    r = ((int(u53) << 11) * total) >> 64
    c = np.cumsum(wv, dtype=np.uint64)
    return int(np.argmax(c > np.uint64(r)))


class Sampler:
    def __init__(self, params: SamplingParams):
        self.params = params
        self.seed = params.seed if params.seed is not None else random_seed()

    def device_mode(self, position: int):
        """(key, bits of 1/T) for the device's greedy / Gumbel-max sampler, or None when the row
        needs filtering (see `filtered_mode`)."""
        p = self.params
        if not p.is_unfiltered():
            return None
        if p.is_greedy():
            return (0, 0)
        inv_t = float(np.float32(1.0) / np.float32(p.temperature))
        return (row_key(self.seed, position), float_bits(inv_t))

    def filtered_mode(self, position: int):
        """(bits of 1/T, top_k, bits of top_p, low, high word of the uniform) for the device's
        top-k / top-p sampler, or None (greedy or unfiltered rows)."""
        p = self.params
        if p.is_unfiltered():
            return None
        inv_t = float(np.float32(1.0) / np.float32(p.temperature))
        u = unit_uniform_53(self.seed, position)
        return (float_bits(inv_t), int(p.top_k), float_bits(float(np.float32(p.top_p))), u & _M32, u >> 32)

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
        if p.top_k == 0 and p.top_p >= 1.0:
            # unfiltered: the device's Gumbel-max rule (sampling.rs:86-100), so that a penalty
            # row draws as its unpenalised neighbours do
            v = np.arange(len(logits), dtype=np.uint64)
            h = (np.uint64(row_key(self.seed, position)) ^ ((v * np.uint64(0x9E3779B9)) & np.uint64(_M32)))
            h ^= h >> np.uint64(16)
            h = (h * np.uint64(0x7FEB352D)) & np.uint64(_M32)
            h ^= h >> np.uint64(15)
            h = (h * np.uint64(0x846CA68B)) & np.uint64(_M32)
            h ^= h >> np.uint64(16)
            u = ((h >> np.uint64(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)
            g = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
            inv_t = np.float32(1.0) / np.float32(p.temperature)
            return int(np.argmax(logits * inv_t + g))
        inv_t = np.float32(1.0) / np.float32(p.temperature)
        return filtered_draw(logits, inv_t, int(p.top_k), float(p.top_p), unit_uniform_53(self.seed, position))
