from .model_config import ConfigError, DenseDecoderConfig, RopeScaling, read_config_json
from .registry import (Architecture, find_architecture, known_architectures, load_config, register_architecture,
                       resolve_architecture, unregister_architecture)
from .engine_config import EngineConfig

__all__ = ["ConfigError", "DenseDecoderConfig", "RopeScaling", "read_config_json",
           "Architecture", "find_architecture", "known_architectures", "load_config", "register_architecture",
           "resolve_architecture", "unregister_architecture", "EngineConfig"]
