from .engine_config import EngineConfig
from .model_config import ConfigError, Qwen2Config, read_config_json
from .registry import (architecture_of, known_architectures, register_architecture, resolve,
                       resolve_model_dir)

__all__ = ["EngineConfig", "ConfigError", "Qwen2Config", "read_config_json",
           "architecture_of", "known_architectures", "register_architecture", "resolve", "resolve_model_dir"]
