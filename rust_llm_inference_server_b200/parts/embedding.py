"""The two ends of the residual stream: token embedding and LM head
(crates/model/src/layers.rs:191-205, crates/model/src/llama.rs:152-156,256-262,279-285)."""

from __future__ import annotations

import torch

from .. import ops
from ..ops.profile import span
from .base import LogitsHead, TokenEmbedding, register_embedding, register_lm_head


class Embedding(TokenEmbedding):
    """out[t, :] = weight[id_t, :] widened to float32, times `scale` where the spec gives one."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.scale = None if spec.scale is None else float(spec.scale)
        self.weight = None

    def tensors(self) -> dict:
        return {self.spec.weight: (self.spec.vocab_size, self.spec.dim)}

    def load(self, src) -> None:
        self.weight = src.get(self.spec.weight, share=True).contiguous()

    def fuses_norms(self, step) -> bool:
        """True when `forward` takes a keyword `sink` in this step (the first block's first norm,
        an `ops.ResidualSink` over `out`) and returns that norm's `ops.ScaledRows`."""
        return self.weight.dtype == torch.bfloat16 and ops.fuses_norms(step.n_tokens, self.weight.dtype, self.spec.dim)

    def forward(self, token_ids, out, step, sink=None):
        with span("embedding"):
            if sink is not None:
                return ops.embedding_sink(token_ids, self.weight, out, self.scale, sink)
            return ops.embedding(token_ids, self.weight, out, self.scale)


class LMHead(LogitsHead):
    """Float32 logits of the wanted rows; a scale and a smooth cap where the spec gives them."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.logit_scale = None if spec.logit_scale is None else float(spec.logit_scale)
        self.soft_cap = None if spec.soft_cap is None else float(spec.soft_cap)
        self.weight = None

    def tensors(self) -> dict:
        return {self.spec.weight: (self.spec.vocab_size, self.spec.dim)}

    def load(self, src) -> None:
        self.weight = src.get(self.spec.weight, share=True).contiguous()

    def fuses_norms(self, step) -> bool:
        """True when `forward` takes the `ops.ScaledRows` of the final norm in this step."""
        return ops.fuses_norms(step.n_tokens, self.weight.dtype, self.spec.dim)

    def forward(self, h, step):
        with span("lm head"):
            logits = ops.linear(h, self.weight, out_dtype=torch.float32)
            if self.logit_scale is not None or self.soft_cap is not None:
                ops.logit_transform(logits, self.logit_scale, self.soft_cap)
            return logits


register_embedding("embedding", Embedding)
register_lm_head("lm_head", LMHead)
