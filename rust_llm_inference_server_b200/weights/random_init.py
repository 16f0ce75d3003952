"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

The reference has random weights only in its tests, with its tensor library's default
initialiser (crates/model/src/llama.rs:324-328, crates/engine/src/testing.rs:68-77).  Here:
matrices N(0, 0.02), norm weights N(1, 0.02), each tensor drawn from a counter-based generator
keyed by (seed, tensor name), so a tensor's values do not depend on the order of generation.
"""

from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import torch

from ..config.registry import lookup_architecture
from .safetensors_io import save_file

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _tensor_key(seed: int, name: str) -> list[int]:
    h = hashlib.sha256(name.encode("utf-8")).digest()
    return [int(seed) & 0xFFFFFFFFFFFFFFFF, int.from_bytes(h[:8], "little")]


def random_tensor(seed: int, name: str, shape, kind: str, std: float = 0.02) -> torch.Tensor:
    rng = np.random.Generator(np.random.Philox(key=_tensor_key(seed, name)))
    x = rng.standard_normal(size=tuple(shape), dtype=np.float32) * np.float32(std)
    if kind == "norm":
        x += np.float32(1.0)
    return torch.from_numpy(x)


def random_tensors(config_json: dict, seed: int, store_dtype: str = "bfloat16") -> dict:
    arch = lookup_architecture(config_json)
    cfg = arch.parse_config(config_json)
    kinds = arch.tensor_kinds(cfg)
    if not kinds:
        raise ValueError(f"architecture {arch.name} does not describe its tensors for random weights")
    dt = _STORE[store_dtype]
    return {name: random_tensor(seed, name, shape, kind).to(dt) for name, (shape, kind) in kinds.items()}


def random_tensors_on_device(config_json: dict, seed: int, device, store_dtype: str = "bfloat16") -> dict:
    """The same distributions drawn by the device's generator (other values than
    `random_tensors`): fast enough for benchmark-sized models."""
    arch = lookup_architecture(config_json)
    kinds = arch.tensor_kinds(arch.parse_config(config_json))
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for name, (shape, kind) in kinds.items():
        x = torch.randn(tuple(shape), generator=gen, device=device, dtype=torch.float32) * 0.02
        if kind == "norm":
            x += 1.0
        out[name] = x.to(_STORE[store_dtype])
    return out


def write_random_model(config_json: dict, out_dir: str, seed: int, store_dtype: str = "bfloat16") -> str:
    """Creates `out_dir` with config.json and model.safetensors; returns out_dir."""
    os.makedirs(out_dir, exist_ok=True)
    tensors = random_tensors(config_json, seed, store_dtype)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "random_weights_seed": seed})
    cfg = dict(config_json)
    cfg.setdefault("architectures", [lookup_architecture(config_json).name])
    cfg["torch_dtype"] = store_dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    return out_dir
