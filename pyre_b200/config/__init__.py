from .engine_config import EngineConfig, parse_dtype
from .model_config import ConfigError, ModelConfig, Qwen2Config
from .registry import (Architecture, architecture, architecture_of, config_from_dict, load_config,
                       register_architecture, registered_architectures)

__all__ = [
    "Architecture", "ConfigError", "EngineConfig", "ModelConfig", "Qwen2Config", "architecture",
    "architecture_of", "config_from_dict", "load_config", "parse_dtype", "register_architecture",
    "registered_architectures",
]
