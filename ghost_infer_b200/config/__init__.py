from .errors import ConfigError, UnknownArchitectureError
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, architecture_of, get_architecture, load_config, parse_config,
                       read_config_json, register_architecture, registered_architectures,
                       unregister_architecture)

__all__ = [
    "ConfigError", "UnknownArchitectureError", "LlamaConfig", "RopeScaling", "Architecture",
    "architecture_of", "get_architecture", "load_config", "parse_config", "read_config_json",
    "register_architecture", "registered_architectures", "unregister_architecture",
]
