"""Typed model configuration read from a checkpoint's `config.json`.

Parity: crates/model/src/config.rs:5-52 of akshajnad/rust_llm_inference_server.  The same keys
are required and optional; nothing the file gives is a constant in code.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Optional


class ConfigError(ValueError):
    """A `config.json` that cannot describe a model of the chosen architecture."""


@dataclass(frozen=True)
class RopeScaling:
    """Frequency-dependent rotary scaling (crates/model/src/config.rs:28-36).

    Only `rope_type == "llama3"` changes the frequencies (crates/model/src/rope.rs:26);
    every other type leaves them as they are, as the reference does.
    """

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: dict) -> "RopeScaling":
        kind = d.get("rope_type", d.get("type"))
        if kind is None:
            raise ConfigError("rope_scaling: missing key 'rope_type'")
        if kind != "llama3":
            # Not scaled by the reference; keep the name so that it shows in errors and dumps.
            return RopeScaling(str(kind), 1.0, 1.0, 1.0, 0)
        missing = [k for k in ("factor", "low_freq_factor", "high_freq_factor",
                               "original_max_position_embeddings") if k not in d]
        if missing:
            raise ConfigError(f"rope_scaling (llama3): missing keys {missing}")
        rs = RopeScaling("llama3", float(d["factor"]), float(d["low_freq_factor"]),
                         float(d["high_freq_factor"]), int(d["original_max_position_embeddings"]))
        if rs.factor <= 0 or rs.high_freq_factor == rs.low_freq_factor or rs.low_freq_factor <= 0 \
                or rs.high_freq_factor <= 0 or rs.original_max_position_embeddings <= 0:
            raise ConfigError(f"rope_scaling (llama3): values out of range: {d}")
        return rs

    def to_dict(self) -> dict:
        if self.rope_type != "llama3":
            return {"rope_type": self.rope_type}
        return {
            "rope_type": self.rope_type, "factor": self.factor,
            "low_freq_factor": self.low_freq_factor, "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass(frozen=True)
class LlamaConfig:
    """The keys of a Llama `config.json` that the forward pass needs.

    Required, as in crates/model/src/config.rs:5-26: hidden_size, intermediate_size,
    num_hidden_layers, num_attention_heads, num_key_value_heads, vocab_size, rms_norm_eps,
    rope_theta, max_position_embeddings.  Optional: head_dim (hidden_size / heads when absent),
    rope_scaling, tie_word_embeddings (false when absent), bos_token_id, eos_token_id.
    """

    architecture = "LlamaForCausalLM"

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: tuple = field(default_factory=tuple)

    REQUIRED = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "vocab_size", "rms_norm_eps", "rope_theta",
                "max_position_embeddings")

    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        missing = [k for k in cls.REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json: missing required keys {missing}")
        for k in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "vocab_size", "max_position_embeddings"):
            if not isinstance(d[k], int) or isinstance(d[k], bool) or d[k] <= 0:
                raise ConfigError(f"config.json: {k} must be a positive integer, got {d[k]!r}")
        nh, nkv = d["num_attention_heads"], d["num_key_value_heads"]
        if nh % nkv != 0:
            raise ConfigError(f"config.json: num_attention_heads {nh} is not a multiple of "
                              f"num_key_value_heads {nkv}")
        hd = d.get("head_dim")
        if hd is None:
            if d["hidden_size"] % nh != 0:
                raise ConfigError(f"config.json: hidden_size {d['hidden_size']} is not a multiple "
                                  f"of num_attention_heads {nh} and head_dim is not given")
            hd = d["hidden_size"] // nh
        if not isinstance(hd, int) or hd <= 0 or hd % 2 != 0:
            raise ConfigError(f"config.json: head_dim must be a positive even integer, got {hd!r}")
        if not float(d["rms_norm_eps"]) > 0 or not float(d["rope_theta"]) > 0:
            raise ConfigError("config.json: rms_norm_eps and rope_theta must be positive")
        rs = d.get("rope_scaling")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        return cls(
            hidden_size=d["hidden_size"], intermediate_size=d["intermediate_size"],
            num_hidden_layers=d["num_hidden_layers"], num_attention_heads=nh,
            num_key_value_heads=nkv, head_dim=hd, vocab_size=d["vocab_size"],
            rms_norm_eps=float(d["rms_norm_eps"]), rope_theta=float(d["rope_theta"]),
            max_position_embeddings=d["max_position_embeddings"],
            rope_scaling=RopeScaling.from_dict(rs) if rs else None,
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            bos_token_id=d.get("bos_token_id"), eos_token_ids=eos_ids,
        )

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"architectures": [self.architecture], "model_type": "llama"}
        for f in fields(self):
            v = getattr(self, f.name)
            if f.name == "rope_scaling":
                out[f.name] = v.to_dict() if v is not None else None
            elif f.name == "eos_token_ids":
                if v:
                    out["eos_token_id"] = list(v) if len(v) > 1 else v[0]
            else:
                out[f.name] = v
        return out

    def kv_bytes_per_token(self, elem_size: int) -> int:
        """Bytes of keys plus values for one token over all layers
        (crates/model/src/config.rs:50-52)."""
        return 2 * self.num_hidden_layers * self.num_key_value_heads * self.head_dim * elem_size


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    # generation_config.json carries the end-of-sequence ids
    # (crates/engine/src/tokenizer.rs:66-85); config.json's own value is the fallback.
    gen = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen):
        try:
            with open(gen, "r", encoding="utf-8") as f:
                g = json.load(f)
            if isinstance(g, dict) and g.get("eos_token_id") is not None:
                d = dict(d)
                d["eos_token_id"] = g["eos_token_id"]
        except (json.JSONDecodeError, OSError):
            pass
    return d
