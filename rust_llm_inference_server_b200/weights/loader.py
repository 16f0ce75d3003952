"""Weights by tensor name: one check of the whole checkpoint against what the model's parts
expect, then placement on the device under a fixed element-type policy.

Policy: a matrix-product operand is kept in bfloat16 for the bfloat16 path (a checkpoint stored in
another float type is rounded once, as the reference casts on load, crates/model/src/llama.rs:59-64)
and widened exactly to float32 for the float32 path; norm weights and other small float vectors
are held in float32 (exact for bfloat16 checkpoints; a tensor stored in 32-bit stays 32-bit);
integer tables become int32.
"""

from __future__ import annotations

import torch

from ..parts.base import TensorSource
from .safetensors_io import Checkpoint


class WeightError(ValueError):
    """The checkpoint does not hold what the model reads; lists every problem at once."""


def check_checkpoint(expected: dict, ckpt: Checkpoint, ignorable=()) -> None:
    have = set(ckpt.names())
    want = set(expected)
    missing = sorted(want - have)
    unexpected = sorted(n for n in have - want if n not in set(ignorable))
    wrong = []
    for n in sorted(want & have):
        es, gs = tuple(expected[n]), tuple(ckpt.shape(n))
        if es != gs:
            wrong.append(f"{n}: expected shape {list(es)}, checkpoint has {list(gs)}")
    if not (missing or unexpected or wrong):
        return
    lines = ["checkpoint does not match the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}):")
        lines.extend("    " + w for w in wrong)
    raise WeightError("\n".join(lines))


class PlacedSource(TensorSource):
    def __init__(self, ckpt: Checkpoint, compute_dtype: torch.dtype, device):
        self.ckpt = ckpt
        self.compute_dtype = compute_dtype
        self.device = device
        self._shared: dict = {}

    def get(self, name: str, role: str = "matrix", share: bool = False) -> torch.Tensor:
        if share:
            key = (name, role)
            if key not in self._shared:
                self._shared[key] = self._place(name, role)
            return self._shared[key]
        return self._place(name, role)

    def _place(self, name: str, role: str) -> torch.Tensor:
        t = self.ckpt.get(name)
        if role == "matrix":
            if not t.dtype.is_floating_point:
                raise WeightError(f"{name}: a matrix operand must be a float tensor, checkpoint has {t.dtype}")
            return t.to(device=self.device, dtype=self.compute_dtype)
        if role == "vector":
            if not t.dtype.is_floating_point:
                raise WeightError(f"{name}: expected a float tensor, checkpoint has {t.dtype}")
            return t.to(device=self.device, dtype=torch.float32)
        if role == "index":
            if t.dtype.is_floating_point:
                raise WeightError(f"{name}: expected an integer table, checkpoint has {t.dtype}")
            return t.to(device=self.device, dtype=torch.int32)
        if role == "stored":
            return t.to(device=self.device)
        raise ValueError(f"unknown tensor role {role!r}")
