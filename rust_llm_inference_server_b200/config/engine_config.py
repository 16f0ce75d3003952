"""Engine options, with the reference's names, meanings and defaults.

Parity: `EngineConfig` in crates/engine/src/engine.rs:32-63 and the command-line flags in
crates/server/src/main.rs:106-127.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class EngineConfig:
    max_num_seqs: int = 64            # sequences in one step
    max_batched_tokens: int = 2048    # tokens in one step; longer prompts go in portions
    kv_cache_bytes: int = 1 << 30     # size of the page pool (all groups together)
    block_size: int = 16              # tokens per page
    policy: str = "continuous"        # or "static"
    prefix_caching: bool = True
    max_seq_len: int = 2048           # longest prompt plus completion
    num_blocks: int | None = None     # if given, overrides kv_cache_bytes (pages per group)
    cuda_graphs: bool = True          # replay decode-only steps from captured graphs
    decode_ahead: bool = True         # launch the next decode step before this one's tokens reach the host

    def validate(self) -> None:
        if self.policy not in ("continuous", "static"):
            raise ValueError(f"scheduler policy must be 'continuous' or 'static', got {self.policy!r}")
        if self.block_size <= 0 or self.max_num_seqs <= 0 or self.max_batched_tokens <= 0:
            raise ValueError("block_size, max_num_seqs and max_batched_tokens must be positive")
