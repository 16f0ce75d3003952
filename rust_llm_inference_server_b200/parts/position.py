"""Position encodings of the attention mixer.

Rotary encoding with the reference's frequency rules (crates/model/src/rope.rs:19-49): inverse
frequencies in float32, scaled per frequency when rope_type is "llama3".  Angles position * f are
formed in float32 inside the kernel, so no table bounds the position.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from .. import ops
from .base import PositionEncoding, register_position


def rope_inverse_frequencies(head_dim: int, theta: float, scaling=None) -> np.ndarray:
    """float32 [head_dim / 2].  1 / theta^(2j/d); for llama3 scaling a frequency whose wavelength
    is shorter than original/high is kept, longer than original/low is divided by `factor`, and
    between the two is blended linearly in original/wavelength (rope.rs:26-46)."""
    one = np.float32(1.0)
    th = np.float32(theta)
    exps = np.arange(0, head_dim, 2, dtype=np.float32) / np.float32(head_dim)
    freqs = (one / np.power(th, exps, dtype=np.float32)).astype(np.float32)
    if scaling is None or getattr(scaling, "rope_type", None) != "llama3":
        return freqs
    factor = np.float32(scaling.factor)
    low = np.float32(scaling.low_freq_factor)
    high = np.float32(scaling.high_freq_factor)
    orig = np.float32(scaling.original_max_position_embeddings)
    wavelen = (np.float32(2.0) * np.float32(math.pi) / freqs).astype(np.float32)
    smooth = ((orig / wavelen - low) / (high - low)).astype(np.float32)
    blended = ((one - smooth) * freqs / factor + smooth * freqs).astype(np.float32)
    out = np.where(wavelen < orig / high, freqs,
                   np.where(wavelen > orig / low, (freqs / factor).astype(np.float32), blended))
    return out.astype(np.float32)


class Rope(PositionEncoding):
    def __init__(self, spec, dtype, device):
        self.head_dim = spec.head_dim
        inv = rope_inverse_frequencies(spec.head_dim, spec.theta, spec.scaling)
        self.inv_freq = torch.from_numpy(inv).to(device)

    def encode_and_store(self, qkv, q_out, cache, step, n_heads, n_kv_heads, head_dim, store):
        slots = step.slots[cache.group] if (store and cache is not None) else None
        ops.rope_cache(qkv, q_out, cache.k if slots is not None else None,
                       cache.v if slots is not None else None, step.positions, slots,
                       self.inv_freq, n_heads, n_kv_heads, head_dim,
                       cache.page_size if cache is not None else 1)

    def rotate_half_table(self):
        return self.inv_freq


class NoPosition(PositionEncoding):
    """No encoding: q is copied out and k, v are stored as they are."""

    def __init__(self, spec, dtype, device):
        pass

    def encode_and_store(self, qkv, q_out, cache, step, n_heads, n_kv_heads, head_dim, store):
        slots = step.slots[cache.group] if (store and cache is not None) else None
        ops.rope_cache(qkv, q_out, cache.k if slots is not None else None,
                       cache.v if slots is not None else None, step.positions, slots,
                       None, n_heads, n_kv_heads, head_dim,
                       cache.page_size if cache is not None else 1)

    def rotate_half_table(self):
        return None


register_position("rope", Rope)
register_position("none", NoPosition)
