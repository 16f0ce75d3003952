"""A model built from a ModelSpec: embedding, blocks in their run order, final norm, LM head.

Role of `Llama::{new, hidden, forward_batch}` (crates/model/src/llama.rs:142-286), with the
architecture taken out: this class reads only the spec.
"""

from __future__ import annotations

import torch

from ..config.model_config import read_config_json
from ..ops import ScaledRows
from ..config.registry import lookup_architecture
from ..parts.base import Part, build_block, build_embedding, build_lm_head, build_norm
from ..parts.spec import EmbeddingSpec, LMHeadSpec, ModelSpec
from ..weights.loader import PlacedSource, check_checkpoint
from ..weights.safetensors_io import Checkpoint, open_model_dir

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "f32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute type must be bfloat16 or float32, got {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"compute type must be bfloat16 or float32, got {name!r}") from None


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        # a spec may name the two ends by their tensors alone: plain lookup, plain product
        emb = spec.embedding if not isinstance(spec.embedding, str) \
            else EmbeddingSpec(spec.vocab_size, spec.hidden, spec.embedding)
        head = spec.lm_head if not isinstance(spec.lm_head, str) \
            else LMHeadSpec(spec.vocab_size, spec.hidden, spec.lm_head)
        self.embedding = build_embedding(emb, dtype, self.device)
        self.blocks = [build_block(ls, dtype, self.device) for ls in spec.layers]
        self.final_norm = build_norm(spec.final_norm, dtype, self.device)
        self.lm_head = build_lm_head(head, dtype, self.device)
        self._tail = _Tail(self.final_norm, self.lm_head)
        self.calls = tuple(spec.order)
        self._plan_caches()
        # parts whose launch configuration depends on more than the step's shape
        self._variant_parts = [p for p in self.parts()
                               if getattr(type(p), "launch_variant", Part.launch_variant) is not Part.launch_variant]
        # whether a step of this model can be captured in a CUDA graph: every part launches the
        # same kernels on the same device buffers whatever the host-side lists of the step hold
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in self.parts())

    @property
    def prefill_tile(self):
        """The tile of prompt tokens the mixers' kernels want listed in a step (None: none does)."""
        tiles = {m.prefill_tile for m in (blk.mixer for blk in self.blocks) if getattr(m, "prefill_tile", None)}
        if len(tiles) > 1:
            raise ValueError(f"the mixers ask for prompt tiles of different sizes: {sorted(tiles)}")
        return tiles.pop() if tiles else None

    def parts(self):
        """Every part of the model, ends included."""
        yield self.embedding
        for blk in self.blocks:
            yield from blk.parts()
        yield self.final_norm
        yield self.lm_head

    def launch_variant(self, step) -> tuple:
        """What of a decode step, beyond its shape, reaches a launch configuration: steps with the
        same value can replay the same captured graph."""
        return tuple(p.launch_variant(step) for p in self._variant_parts)

    # ---- what the cache manager has to provide ----

    def _plan_caches(self) -> None:
        """Per cache slot its KVCacheSpec (from the call that writes it); per call its StateSpec."""
        slots: dict[int, object] = {}
        writer: dict[int, int] = {}
        self.call_state_specs = []
        for ci, call in enumerate(self.calls):
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"run order names layer {call.layer}; the model has {len(self.blocks)}")
            mixer = self.blocks[call.layer].mixer
            cs = mixer.cache_spec()
            if call.writes_cache:
                if call.cache in writer:
                    raise ValueError(f"cache slot {call.cache} is written by calls {writer[call.cache]} and {ci}")
                writer[call.cache] = ci
                slots[call.cache] = cs
            else:
                if call.cache not in writer:
                    raise ValueError(f"call {ci} reads cache slot {call.cache} before any call has written it")
                if slots[call.cache] != cs:
                    raise ValueError(f"call {ci} reads cache slot {call.cache} whose geometry {slots[call.cache]} "
                                     f"differs from its own {cs}")
            self.call_state_specs.append(mixer.state_spec())
        n = (max(slots) + 1) if slots else 0
        self.cache_slot_specs = [slots.get(i) for i in range(n)]

    # ---- weights ----

    def tensors(self) -> dict:
        out: dict = {}
        for part in self.parts():
            for name, shape in part.tensors().items():
                if name in out and tuple(out[name]) != tuple(shape):
                    raise ValueError(f"tensor {name} is expected with shapes {out[name]} and {shape}")
                out[name] = tuple(shape)
        return out

    def load(self, ckpt: Checkpoint) -> None:
        check_checkpoint(self.tensors(), ckpt, self.spec.ignorable)
        src = PlacedSource(ckpt, self.dtype, self.device)
        for part in self.parts():
            part.load(src)

    # ---- forward ----

    def forward(self, step, caches, states):
        """Runs the step's tokens through every call of the run order.  Returns the float32
        residual stream and the last pending delta; `logits` finishes chosen rows."""
        T = step.n_tokens
        resid = step.buffer("resid", (T, self.spec.hidden), torch.float32)
        delta = None
        first = self.blocks[self.calls[0].layer] if self.calls else None
        emb_fuses = getattr(self.embedding, "fuses_norms", None)
        sink = first.entry_sink(resid, step) if (emb_fuses is not None and emb_fuses(step) and
                                                 getattr(first, "chains_norms", False)) else None
        if sink is not None:    # the first block's first norm is left to its first product
            delta = self.embedding.forward(step.token_ids, resid, step, sink=sink)
        else:
            self.embedding.forward(step.token_ids, resid, step)
        for ci, call in enumerate(self.calls):
            blk = self.blocks[call.layer]
            nxt = self.blocks[self.calls[ci + 1].layer] if ci + 1 < len(self.calls) else self._tail
            if getattr(blk, "chains_norms", False) and hasattr(nxt, "entry_sink"):
                # the block may leave its last addition and the next block's first norm to the products around them
                resid, delta = blk.forward(resid, delta, step, caches[call.cache], states[ci], call.writes_cache,
                                           next_block=nxt)
            else:
                resid, delta = blk.forward(resid, delta, step, caches[call.cache], states[ci], call.writes_cache)
        return resid, delta

    def logits(self, resid, delta, step, rows: torch.Tensor):
        """Final norm and LM head on the rows in `rows` (int32 indices into the step's tokens):
        float32 logits [len(rows), vocab] (crates/model/src/llama.rs:272-285)."""
        if isinstance(delta, ScaledRows):       # the last block left the final norm to the head's product
            return self.lm_head.forward(delta, step)
        h = self.final_norm.forward_rows(resid, delta, step, rows)
        return self.lm_head.forward(h, step)


class _Tail:
    """What follows the last block, asked as a block is asked for its `entry_sink`: the final norm's
    sink, when the step wants the logits of all its rows in order (a decode step) and the head's
    product takes the rows that come out of it.  The last block's last product then adds to the
    residual stream itself and the final norm is no kernel of its own."""

    def __init__(self, final_norm, lm_head):
        self.final_norm, self.lm_head = final_norm, lm_head

    def entry_sink(self, resid, step):
        head_fuses = getattr(self.lm_head, "fuses_norms", None)
        if not getattr(step, "wants_every_row", False) or head_fuses is None or not head_fuses(step):
            return None
        sink = getattr(self.final_norm, "sink", None)
        return sink(resid, step) if sink is not None else None


def build_model(config_json: dict, dtype, device="cuda") -> Model:
    arch = lookup_architecture(config_json)
    cfg = arch.parse_config(config_json)
    model = Model(arch.describe(cfg), parse_dtype(dtype), device)
    model.config = cfg
    model.architecture = arch.name
    return model


def load_model(model_dir: str, dtype="bfloat16", device="cuda") -> Model:
    """Reads config.json, picks the architecture through the registry, loads the weights."""
    model = build_model(read_config_json(model_dir), dtype, device)
    model.load(open_model_dir(model_dir))
    return model
