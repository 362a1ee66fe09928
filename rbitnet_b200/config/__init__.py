from .base import ModelConfig, ConfigError, read_config_json
from .llama import LlamaConfig
from .registry import (register_architecture, unregister_architecture, known_architectures,
                       get_architecture, architecture_of, config_from_dict, load_config)

__all__ = ["ModelConfig", "ConfigError", "read_config_json", "LlamaConfig",
           "register_architecture", "unregister_architecture", "known_architectures",
           "get_architecture", "architecture_of", "config_from_dict", "load_config"]
