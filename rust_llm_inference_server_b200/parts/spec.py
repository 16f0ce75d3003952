"""A model as data: which parts each layer is made of, with every size and constant as a
parameter, and the order in which layers run.

Nothing here knows an architecture.  An architecture's `describe(config)` returns a `ModelSpec`;
`parts.build` turns each spec into a part by its `kind` through the part registries.
The reference builds its one model imperatively (crates/model/src/llama.rs:142-170); the specs
carry the same information: tensor names (llama.rs:25-28,144-156; attention.rs:47-51;
layers.rs:171-173) and constants (config.rs:5-26).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class RMSNormSpec:
    dim: int
    eps: float
    weight: str                      # tensor name, shape (dim,)
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    """Rotate-half rotary encoding; `scaling` as in config.RopeScaling (llama3) or None."""
    head_dim: int
    theta: float
    scaling: Any = None
    kind: str = "rope"


@dataclass(frozen=True)
class NoPositionSpec:
    kind: str = "none"


@dataclass(frozen=True)
class GQAAttentionSpec:
    """Causal grouped-query attention.  `window`: keys visible to a query (None = all earlier
    ones).  `scale`: score multiplier (None = 1 / sqrt(head_dim), the reference's fixed choice,
    crates/model/src/attention.rs:147,210)."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    q_proj: str                      # (n_heads * head_dim, hidden)
    k_proj: str                      # (n_kv_heads * head_dim, hidden)
    v_proj: str
    o_proj: str                      # (hidden, n_heads * head_dim)
    position: Any = field(default_factory=NoPositionSpec)
    window: Optional[int] = None
    scale: Optional[float] = None
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden: int
    intermediate: int
    gate_proj: str                   # (intermediate, hidden)
    up_proj: str
    down_proj: str                   # (hidden, intermediate)
    kind: str = "swiglu"


@dataclass(frozen=True)
class EmbeddingSpec:
    """Token table: row `id` of `weight` (vocab, dim) starts the residual stream, multiplied by
    `scale` if one is given (the reference's Llama has none, crates/model/src/llama.rs:256-262)."""
    vocab_size: int
    dim: int
    weight: str
    scale: Optional[float] = None
    kind: str = "embedding"


@dataclass(frozen=True)
class LMHeadSpec:
    """Logits = h · weight^T in float32 (crates/model/src/llama.rs:279-285), then, where given,
    multiplied by `logit_scale` and capped smoothly: cap · tanh(logits / cap).  `weight` may name
    the embedding's tensor (tied)."""
    vocab_size: int
    dim: int
    weight: str
    logit_scale: Optional[float] = None
    soft_cap: Optional[float] = None
    kind: str = "lm_head"


@dataclass(frozen=True)
class LayerSpec:
    """One block.  arrangement "prenorm": x += mixer(norm1(x)); x += feed_forward(norm2(x))
    (crates/model/src/llama.rs:264-271)."""
    norm1: Any
    mixer: Any
    norm2: Any
    feed_forward: Any
    arrangement: str = "prenorm"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run `layer` with cache slot `cache`.  A layer may be named by
    several calls (its weights are shared, each call has a cache slot and state of its own unless
    it names another call's slot).  `writes_cache=False`: the call stores nothing and reads the
    slot that an earlier call of the same step has filled."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden: int
    embedding: Any                   # an EmbeddingSpec, or just the tensor's name (vocab, hidden)
    layers: tuple
    order: tuple                     # of LayerCall
    final_norm: Any
    lm_head: Any                     # an LMHeadSpec, or just the tensor's name (the embedding's when tied)
    max_positions: int
    # names that a checkpoint may hold although the model does not read them
    ignorable: tuple = ()
    eos_token_ids: tuple = ()
