"""RMSNorm over the float32 residual stream (crates/model/src/layers.rs:103-146)."""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..ops.profile import span
from .base import Norm, register_norm


class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * w.  eps is used as a float32 (layers.rs:115); the sum of
    squares and the scale are float32; the weight is held in float32 (an exact widening)."""

    graph_safe = True    # launches depend on the step's device arrays and shapes only

    def __init__(self, spec, dtype, device):
        self.dim = spec.dim
        self.eps = float(np.float32(spec.eps))
        self.weight_name = spec.weight
        self.dtype = dtype
        self.weight = None

    def tensors(self) -> dict:
        return {self.weight_name: (self.dim,)}

    def load(self, src) -> None:
        self.weight = src.get(self.weight_name, "vector")

    def forward(self, resid, delta, step):
        out = step.buffer("norm_out", (resid.shape[0], self.dim), self.dtype)
        with span("residual add + rms norm"):
            return ops.rmsnorm(resid, self.weight, self.eps, out, delta)

    def forward_rows(self, resid, delta, step, rows):
        out = step.buffer("norm_rows_out", (rows.shape[0], self.dim), self.dtype)
        with span("residual add + rms norm"):
            return ops.rmsnorm(resid, self.weight, self.eps, out, delta, rows)

    def sink(self, resid, step):
        if not ops.fuses_norms(resid.shape[0], self.dtype, self.dim):
            return None
        return ops.ResidualSink(resid, self.weight, self.eps)


register_norm("rmsnorm", RMSNorm)
