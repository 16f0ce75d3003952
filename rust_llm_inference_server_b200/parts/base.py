"""Interfaces of the parts a layer is made of, and the registries that build them from specs.

A part gets its sizes and constants from its spec, names the checkpoint tensors it needs, and
knows nothing of the model it sits in.  A new kind of part is one class and one `register_*` call.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch


class TensorSource:
    """What a part loads from: `get(name, role)` returns the tensor on the device.

    role "matrix": a matrix-product operand, in the compute type (bfloat16 or float32);
    role "vector": a norm weight or other small float table, widened exactly to float32;
    role "index":  an integer table, as int32;
    role "stored": whatever the checkpoint holds, unchanged (32-bit stays 32-bit).

    `share=True`: parts that ask for the same tensor in the same role get one copy on the device
    (tied embedding and LM head)."""

    def get(self, name: str, role: str = "matrix", share: bool = False) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class Part:
    # True when `forward` reads only device arrays and shapes of the step (never its host-side
    # lists), so that a decode step can be replayed from a captured CUDA graph.
    graph_safe = False

    def launch_variant(self, step):
        """For graph-safe parts: whatever of a decode step, beyond the number of requests and of
        wanted rows, decides a launch configuration (a hashable value; None: nothing does).  Steps
        with equal variants replay the same captured graph."""
        return None

    def fuses_norms(self, step) -> bool:
        """Mixers and feed-forwards: True when, in this step, `forward` takes `ops.ScaledRows` for x
        (rows of the norm before it whose scale its first product applies) and a keyword `sink`
        (an `ops.ResidualSink`: its last product adds the result to the residual stream itself and
        returns the ScaledRows of the norm that follows instead of its output).  The arrangement
        asks before it passes either; a part that says nothing gets and returns plain tensors."""
        return False

    def tensors(self) -> dict:
        """Checkpoint tensors this part reads: {name: shape}."""
        return {}

    def load(self, src: TensorSource) -> None:
        pass


@dataclass(frozen=True)
class KVCacheSpec:
    """What a mixer keeps per token: keys and values of `n_kv_heads` heads of `head_dim`, of all
    earlier tokens (window None) or of the last `window` tokens."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (shape per request, element type)."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """One cache slot's device storage as a mixer sees it."""
    k: torch.Tensor                  # [pages, n_kv_heads, page_size, head_dim]
    v: torch.Tensor
    group: int                       # index into the step's block tables and slot lists
    page_size: int


class TokenEmbedding(Part):
    """Starts the residual stream: `forward(token_ids, out, step)` fills `out`, float32
    [tokens, hidden], from int32 ids on the device."""

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError


class LogitsHead(Part):
    """Ends it: `forward(h, step)` takes the normed rows whose logits are wanted, [rows, hidden] in
    the compute type, and returns float32 logits [rows, vocab]."""

    def forward(self, h: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    """Token mixing over a request's earlier tokens.  `forward` gets the normed activations
    [T, hidden] of all tokens of the step and returns [T, hidden] in the same element type."""

    # Tokens of a request that one CTA of the mixer's kernel for prompt portions takes; the step
    # function then lists every portion of the step in tiles of that many tokens
    # (`step.prefill_tiles`).  None: the mixer needs no such list.
    prefill_tile: Optional[int] = None

    def cache_spec(self) -> Optional[KVCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, step, cache: Optional[LayerCache],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    """`forward(resid, delta)`: adds `delta` (or nothing) into the float32 residual stream in
    place and returns the normed activations in the compute type."""

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], step) -> torch.Tensor:
        raise NotImplementedError

    def forward_rows(self, resid, delta, step, rows: torch.Tensor) -> torch.Tensor:
        """The same for the rows `rows` only (the places whose logits are wanted)."""
        return self.forward(resid, delta, step).index_select(0, rows.long())

    def sink(self, resid: torch.Tensor, step):
        """An `ops.ResidualSink` for this norm over `resid` when, in this step, the product before
        it may do the addition and the product after it the scaling (see `Part.fuses_norms`), or
        None (the default): the norm then runs as a kernel of its own."""
        return None


class PositionEncoding(Part):
    """Belongs to a mixer.  `encode_and_store` splits the fused q|k|v rows, encodes positions into
    q and k, writes q to `q_out` and k, v into the paged cache at the step's slots."""

    def encode_and_store(self, qkv, q_out, cache: Optional[LayerCache], step, n_heads: int,
                         n_kv_heads: int, head_dim: int, store: bool) -> None:
        raise NotImplementedError

    def rotate_half_table(self):
        """For mixers whose decode kernel can encode positions itself: the float32 inverse
        frequencies [head_dim / 2] of a rotate-half encoding, None for "no encoding", or
        NotImplemented (the default) when the encoding is anything else; the mixer then calls
        `encode_and_store` as for every other step."""
        return NotImplemented


_MIXERS: dict[str, Callable] = {}
_FEED_FORWARDS: dict[str, Callable] = {}
_NORMS: dict[str, Callable] = {}
_POSITIONS: dict[str, Callable] = {}
_ARRANGEMENTS: dict[str, Callable] = {}
_EMBEDDINGS: dict[str, Callable] = {}
_LM_HEADS: dict[str, Callable] = {}


def _register(table: dict, what: str):
    def reg(kind: str, factory: Callable, replace: bool = False) -> None:
        if kind in table and not replace:
            raise ValueError(f"{what} kind {kind!r} is already registered")
        table[kind] = factory
    return reg


register_mixer = _register(_MIXERS, "mixer")
register_feed_forward = _register(_FEED_FORWARDS, "feed-forward")
register_norm = _register(_NORMS, "norm")
register_position = _register(_POSITIONS, "position encoding")
register_arrangement = _register(_ARRANGEMENTS, "block arrangement")
register_embedding = _register(_EMBEDDINGS, "embedding")
register_lm_head = _register(_LM_HEADS, "LM head")


def _build(table: dict, what: str, spec, dtype, device):
    kind = getattr(spec, "kind", None)
    if kind not in table:
        raise ValueError(f"no {what} of kind {kind!r} is registered; known: {sorted(table)}")
    return table[kind](spec, dtype, device)


def build_mixer(spec, dtype, device) -> Mixer:
    return _build(_MIXERS, "mixer", spec, dtype, device)


def build_feed_forward(spec, dtype, device) -> FeedForward:
    return _build(_FEED_FORWARDS, "feed-forward", spec, dtype, device)


def build_norm(spec, dtype, device) -> Norm:
    return _build(_NORMS, "norm", spec, dtype, device)


def build_position(spec, dtype, device) -> PositionEncoding:
    return _build(_POSITIONS, "position encoding", spec, dtype, device)


def build_embedding(spec, dtype, device) -> TokenEmbedding:
    return _build(_EMBEDDINGS, "embedding", spec, dtype, device)


def build_lm_head(spec, dtype, device) -> LogitsHead:
    return _build(_LM_HEADS, "LM head", spec, dtype, device)


def build_block(spec, dtype, device):
    kind = getattr(spec, "arrangement", None)
    if kind not in _ARRANGEMENTS:
        raise ValueError(f"no block arrangement {kind!r} is registered; known: {sorted(_ARRANGEMENTS)}")
    return _ARRANGEMENTS[kind](spec, dtype, device)
