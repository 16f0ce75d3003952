"""Causal grouped-query attention over the paged cache (crates/model/src/attention.rs:11-104)."""

from __future__ import annotations

import math

import torch

from .. import ops
from ..ops.profile import span
from .base import KVCacheSpec, Mixer, build_position, register_mixer


class GQAAttention(Mixer):
    """q, k, v projections (stacked into one matrix at load time; no biases), position encoding of
    q and k, keys and values stored in this call's cache slot, attention of every token over its
    request's cached keys up to its own position, output projection.

    Scores, softmax and the value sum are float32 in every kernel.  Query head h reads key/value
    head h // (n_heads // n_kv_heads) (attention.rs:166-175)."""

    graph_safe = True    # launches depend on the step's device arrays and shapes only

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.position = build_position(spec.position, dtype, device)
        self.scale = float(spec.scale) if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)
        self.window = int(spec.window) if spec.window else 0
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} query heads are not a multiple of {spec.n_kv_heads} key/value heads")
        if spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"attention kernels take head sizes that are multiples of 16 up to 256, got {spec.head_dim}")
        self.w_qkv = None
        self.w_o = None

    def tensors(self) -> dict:
        s = self.spec
        return {s.q_proj: (s.n_heads * s.head_dim, s.hidden),
                s.k_proj: (s.n_kv_heads * s.head_dim, s.hidden),
                s.v_proj: (s.n_kv_heads * s.head_dim, s.hidden),
                s.o_proj: (s.hidden, s.n_heads * s.head_dim)}

    def load(self, src) -> None:
        s = self.spec
        self.w_qkv = torch.cat([src.get(s.q_proj), src.get(s.k_proj), src.get(s.v_proj)], dim=0).contiguous()
        self.w_o = src.get(s.o_proj).contiguous()
        self.position.load(src)

    def cache_spec(self):
        s = self.spec
        return KVCacheSpec(s.n_kv_heads, s.head_dim, s.window)

    @property
    def prefill_tile(self):
        # the flash kernels for prompt portions take one tile of this many tokens a CTA
        return ops.prefill_tile() if self.dtype == torch.bfloat16 and self.spec.head_dim in (64, 128) else None

    def launch_variant(self, step):
        # decode attention cuts the context into pieces by the longest context of the step
        s = self.spec
        return ops.decode_splits(step.n_decode, s.n_kv_heads, step.max_decode_ctx) if step.n_decode else None

    def fuses_norms(self, step) -> bool:
        s = self.spec
        return ops.fuses_norms(step.n_tokens, self.dtype, s.hidden, s.n_heads * s.head_dim)

    def forward(self, x, step, cache, state, writes_cache=True, sink=None):
        s = self.spec
        T = x.shape[0]
        with span("qkv proj"):
            qkv = ops.linear(x, self.w_qkv)
        o = step.buffer("attn_o", (T, s.n_heads * s.head_dim), self.dtype)
        if step.all_decode and ops.decode_attention_takes_qkv(qkv.dtype, s.n_heads, s.n_kv_heads, s.head_dim):
            table = self.position.rotate_half_table()
            if table is not NotImplemented:
                # a step of single tokens: the attention kernel rotates q and the newest key and
                # stores that key itself, one kernel fewer a layer
                with span("rope + kv write + attention"):
                    ops.attention_decode_from_qkv(qkv, cache.k, cache.v, o, step, cache.group, table, writes_cache,
                                                  s.n_heads, s.n_kv_heads, s.head_dim, cache.page_size,
                                                  self.scale, self.window)
                with span("o proj"):
                    return ops.linear(o, self.w_o, sink=sink)
        q = step.buffer("attn_q", (T, s.n_heads * s.head_dim), self.dtype)
        with span("rope + kv write"):
            self.position.encode_and_store(qkv, q, cache, step, s.n_heads, s.n_kv_heads, s.head_dim,
                                           store=writes_cache)
        with span("attention"):
            ops.attention(q, cache.k, cache.v, o, step, cache.group, s.n_heads, s.n_kv_heads,
                          s.head_dim, cache.page_size, self.scale, self.window)
        with span("o proj"):
            return ops.linear(o, self.w_o, sink=sink)


register_mixer("gqa_attention", GQAAttention)
