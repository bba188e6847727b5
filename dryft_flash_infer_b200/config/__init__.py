from .base import ConfigError, ModelConfig, read_config_json
from .qwen3 import Qwen3Config
from .registry import (Architecture, architecture_named, architecture_of, config_from_dict,
                       known_architectures, load_config, register_architecture)

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "Architecture", "architecture_named",
           "architecture_of", "config_from_dict", "known_architectures", "load_config",
           "register_architecture", "read_config_json"]
