"""One registry from an architecture's name to its configuration class and model description.

The reference has a single hard-wired model type and tells formats apart only by file extension
(crates/model/src/lib.rs:21-32).  Here the name in `config.json` (`architectures[0]`) picks an
entry; an architecture is added by one `register_architecture` call and no other change.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    # dict from config.json -> typed configuration object
    parse_config: Callable[[dict], Any]
    # typed configuration -> parts.spec.ModelSpec (pure data: which parts, in which order)
    describe: Callable[[Any], Any]
    # typed configuration, numpy Generator-like seed -> {tensor name: (shape, kind)} for the
    # random-weights mode; kind is "matrix" or "norm".
    tensor_kinds: Callable[[Any], dict]


_REGISTRY: dict[str, Architecture] = {}

# The reference reads any config.json as a Llama (it never looks at `architectures`);
# a file without the key is treated the same way.
DEFAULT_ARCHITECTURE = "LlamaForCausalLM"


def register_architecture(name: str, parse_config, describe, tensor_kinds=None) -> None:
    if name in _REGISTRY:
        raise ValueError(f"architecture {name!r} is already registered")
    _REGISTRY[name] = Architecture(name, parse_config, describe, tensor_kinds or (lambda cfg: {}))


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def registered_architectures() -> list[str]:
    return sorted(_REGISTRY)


def architecture_name(config_json: dict) -> str:
    archs = config_json.get("architectures")
    if archs is None:
        return DEFAULT_ARCHITECTURE
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"config.json: 'architectures' must be a list of names, got {archs!r}")
    return archs[0]


def lookup_architecture(config_json: dict) -> Architecture:
    name = architecture_name(config_json)
    if name not in _REGISTRY:
        raise ConfigError(f"config.json names architecture {name!r}; registered: "
                          f"{registered_architectures()}")
    return _REGISTRY[name]
