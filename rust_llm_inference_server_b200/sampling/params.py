"""Per-request sampling settings, with the reference's names, meanings and defaults
(crates/engine/src/sampler.rs:9-58)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0          # below 1e-5 means greedy
    top_p: float = 1.0                # 1.0 disables nucleus filtering
    top_k: int = 0                    # 0 disables top-k filtering
    repetition_penalty: float = 1.0   # 1.0 disables it; applies to every token of prompt and output
    seed: Optional[int] = None        # none: a random seed per request
    max_tokens: int = 16
    ignore_eos: bool = False          # keep generating through end-of-sequence until max_tokens

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0 or self.temperature < 0 or self.repetition_penalty <= 0:
            raise ValueError("top_k, temperature must be >= 0 and repetition_penalty > 0")

    def is_greedy(self) -> bool:
        return self.temperature < 1e-5

    def is_unfiltered(self) -> bool:
        """Greedy or temperature-only rows: the Gumbel-max kernel picks them (sampler.rs:54-57);
        rows with top-k or top-p go to the filtering kernel.  A repetition penalty is applied to
        the logits on the device before either."""
        return self.is_greedy() or (self.top_k == 0 and self.top_p >= 1.0)
