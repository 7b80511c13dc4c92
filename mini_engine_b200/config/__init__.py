from .model_config import ConfigError, ModelConfig, Qwen3Config, read_config_json, architecture_name
from .registry import (Architecture, register_architecture, get_architecture,
                       registered_architectures, load_model_config)
from .engine_config import EngineConfig

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "read_config_json", "architecture_name",
           "Architecture", "register_architecture", "get_architecture", "registered_architectures",
           "load_model_config", "EngineConfig"]
