"""A B200-native inference engine for the Llama decoder, built out of what
akshajnad/rust_llm_inference_server shows: typed configuration and a registry, weights by tensor
name, layers put together from parts, a paged cache manager, one step function, a scheduler,
sampling, and hand-written sm_100a kernels."""

from . import models as _models  # noqa: F401  (registers the architectures)
from . import parts as _parts    # noqa: F401  (registers the built-in parts)

__all__ = ["LLM", "SamplingParams", "EngineConfig"]


def __getattr__(name):
    if name in ("LLM", "RequestOutput"):
        from .engine import llm
        return getattr(llm, name)
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    if name == "EngineConfig":
        from .config.engine_config import EngineConfig
        return EngineConfig
    raise AttributeError(name)
