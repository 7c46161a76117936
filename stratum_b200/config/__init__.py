from .base import ConfigError, KeyReader, ModelConfig, read_config_json
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, architecture_name, find_architecture, register_architecture,
                       registered_architectures)

__all__ = ["ConfigError", "KeyReader", "ModelConfig", "read_config_json", "LlamaConfig", "RopeScaling",
           "Architecture", "architecture_name", "find_architecture", "register_architecture",
           "registered_architectures"]
