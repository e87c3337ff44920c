from .model_config import ConfigError, LlamaConfig, RopeScaling, read_config_json
from .engine_config import EngineConfig
from .registry import (Architecture, known_architectures, register_architecture,
                       resolve_architecture)

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "read_config_json", "EngineConfig",
           "Architecture", "known_architectures", "register_architecture",
           "resolve_architecture"]
