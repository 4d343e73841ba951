from .base import ConfigError, read_config_json
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, architecture_of, config_from_folder, known_architectures,
                       lookup_architecture, register_architecture)

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "read_config_json", "Architecture",
           "architecture_of", "config_from_folder", "known_architectures", "lookup_architecture",
           "register_architecture"]
