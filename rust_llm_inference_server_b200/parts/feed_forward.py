"""Dense SwiGLU feed-forward (crates/model/src/layers.rs:156-187): down(silu(gate x) * up x)."""

from __future__ import annotations

import torch

from .. import ops
from ..ops.profile import span
from .base import FeedForward, register_feed_forward


class SwiGLU(FeedForward):
    """gate and up are stacked into one (2I, hidden) matrix at load time, rows interleaved in
    blocks of 4 (4 gate rows, their 4 up rows, ...), so one product feeds the gating and the
    decode kernel can gate in its epilogue; a pure change of layout."""

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
        g, u = src.get(s.gate_proj), src.get(s.up_proj)
        self.interleave = 4 if s.intermediate % 4 == 0 else 0
        if self.interleave:
            self.w_gate_up = torch.stack([g.view(-1, 4, s.hidden), u.view(-1, 4, s.hidden)], dim=1) \
                .reshape(2 * s.intermediate, s.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = src.get(s.down_proj).contiguous()

    def fuses_norms(self, step) -> bool:
        return ops.fuses_norms(step.n_tokens, self.dtype, self.spec.hidden, self.spec.intermediate)

    def forward(self, x, step, sink=None):
        fusable = self.dtype == torch.bfloat16 and self.interleave == 4 and self.spec.hidden % 8 == 0
        with span("mlp gate+up, silu*up"):
            if fusable and x.shape[0] <= ops.STREAM_GEMM_ROWS:
                act = ops.stream_gemm(x, self.w_gate_up, swiglu4=True)       # product and gating in one kernel
            elif fusable and x.shape[0] >= 128 and self.spec.intermediate % 128 == 0:
                # prefill: the tcgen05 product with the gating in its epilogue (the gate|up activations
                # never reach HBM)
                act = ops.gemm_tcgen05(x, self.w_gate_up, "swiglu4")
            else:
                gu = ops.linear(x, self.w_gate_up)
                act = step.buffer("ffn_act", (x.shape[0], self.spec.intermediate), self.dtype)
                ops.swiglu(gu, act, self.interleave)
        with span("mlp down proj"):
            return ops.linear(act, self.w_down, sink=sink)


register_feed_forward("swiglu", SwiGLU)
