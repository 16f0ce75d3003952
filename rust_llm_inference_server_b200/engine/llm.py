"""The Python entry point: `LLM(model_dir, ...).generate(prompt_token_ids, SamplingParams(...))`.

The reference is Rust only and has no Python API; its user-facing call is
`rlis generate` (crates/server/src/main.rs:216-262), whose option names and defaults this class
keeps (`--dtype`, `--max-seq-len`, `--kv-cache-gb`, `--block-size`, `--max-num-seqs`,
`--max-batched-tokens`, `--scheduler`, `--no-prefix-caching`).
"""

from __future__ import annotations

import torch

from ..config.engine_config import EngineConfig
from ..config.model_config import read_config_json
from ..models import build_model, load_model
from ..sampling.params import SamplingParams
from ..weights.random_init import random_tensors, random_tensors_on_device
from ..weights.safetensors_io import Checkpoint
from .engine import LLMEngine, RequestOutput


class LLM:
    def __init__(self, model: str | None = None, dtype: str = "bfloat16", max_seq_len: int = 2048,
                 kv_cache_gb: float = 1.0, block_size: int = 16, max_num_seqs: int = 64,
                 max_batched_tokens: int = 2048, scheduler: str = "continuous",
                 prefix_caching: bool = True, num_blocks: int | None = None, device: str = "cuda",
                 cuda_graphs: bool = True, decode_ahead: bool = True, _model=None):
        if not torch.cuda.is_available():
            raise RuntimeError("this engine runs on a CUDA device only; there is no CPU path")
        self.model = _model if _model is not None else load_model(model, dtype, device)
        cfg = EngineConfig(max_num_seqs=max_num_seqs, max_batched_tokens=max_batched_tokens,
                           kv_cache_bytes=int(kv_cache_gb * (1 << 30)), block_size=block_size,
                           policy=scheduler, prefix_caching=prefix_caching, max_seq_len=max_seq_len,
                           num_blocks=num_blocks, cuda_graphs=cuda_graphs,
                           decode_ahead=decode_ahead)
        self.engine = LLMEngine(self.model, cfg)

    @classmethod
    def from_random(cls, config_json: dict, seed: int, dtype: str = "bfloat16", device: str = "cuda",
                    on_device: bool = False, **engine_options) -> "LLM":
        """Random-weights mode without a folder: the same tensors `write_random_model` would store
        (or, with `on_device`, tensors of the same distributions drawn by the GPU's generator)."""
        model = build_model(config_json, dtype, device)
        store = "bfloat16" if model.dtype == torch.bfloat16 else "float32"
        make = (lambda: random_tensors_on_device(config_json, seed, device, store)) if on_device \
            else (lambda: random_tensors(config_json, seed, store))
        model.load(Checkpoint(tensors=make()))
        return cls(None, dtype=dtype, device=device, _model=model, **engine_options)

    def _submit(self, prompt_token_ids, sampling_params):
        if prompt_token_ids and isinstance(prompt_token_ids[0], int):
            prompt_token_ids = [prompt_token_ids]
        n = len(prompt_token_ids)
        if sampling_params is None:
            sampling_params = SamplingParams()
        plist = sampling_params if isinstance(sampling_params, (list, tuple)) else [sampling_params] * n
        if len(plist) != n:
            raise ValueError(f"{n} prompts but {len(plist)} sampling parameter sets")
        return [self.engine.add_request(p, sp) for p, sp in zip(prompt_token_ids, plist)]

    def stream(self, prompt_token_ids, sampling_params=None):
        """Like `generate`, but yields a StepEvent after every engine step (tokens as they are
        sampled, requests as they finish), as the reference streams events to its caller."""
        self._submit(prompt_token_ids, sampling_params)
        while self.engine.has_work():
            self.engine.step()
            yield self.engine.last_step

    def generate(self, prompt_token_ids, sampling_params=None) -> list:
        """`prompt_token_ids`: a list of token-id lists.  `sampling_params`: one SamplingParams for
        all, or a list.  Returns one RequestOutput per prompt, in the order of the prompts."""
        ids = self._submit(prompt_token_ids, sampling_params)
        done = {o.request_id: o for o in self.engine.run_to_completion()}
        return [done[i] for i in ids]
