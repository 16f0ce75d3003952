from .engine_config import EngineConfig
from .model_config import ConfigError, LlamaConfig, RopeScaling, read_config_json
from .registry import (architecture_name, lookup_architecture, register_architecture,
                       registered_architectures, unregister_architecture)
