"""Dense SwiGLU feed-forward (crates/model/src/layers.rs:156-187): down(silu(gate x) * up x)."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, register_feed_forward


class SwiGLU(FeedForward):
    """gate and up are stacked into one (2I, hidden) matrix at load time, so one product feeds the
    gating kernel; a pure change of layout."""

    graph_safe = True    # launches depend on the step's device arrays and shapes only

    def __init__(self, spec, dtype, device):
        self.spec = spec
        self.dtype = dtype
        self.w_gate_up = None
        self.w_down = None

    def tensors(self) -> dict:
        s = self.spec
        return {s.gate_proj: (s.intermediate, s.hidden), s.up_proj: (s.intermediate, s.hidden),
                s.down_proj: (s.hidden, s.intermediate)}

    def load(self, src) -> None:
        s = self.spec
        self.w_gate_up = torch.cat([src.get(s.gate_proj), src.get(s.up_proj)], dim=0).contiguous()
        self.w_down = src.get(s.down_proj).contiguous()

    def forward(self, x, step):
        gu = ops.linear(x, self.w_gate_up)
        act = step.buffer("ffn_act", (x.shape[0], self.spec.intermediate), self.dtype)
        ops.swiglu(gu, act)
        return ops.linear(act, self.w_down)


register_feed_forward("swiglu", SwiGLU)
