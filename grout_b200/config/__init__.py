from .base import ConfigError, ModelConfig, read_json
from .generation import GenerationConfig
from .qwen3 import Qwen3Config
from .registry import (Architecture, known_architectures, load_config, register_architecture,
                       resolve_architecture, unregister_architecture)

__all__ = ["ConfigError", "ModelConfig", "GenerationConfig", "Qwen3Config", "Architecture",
           "known_architectures", "load_config", "register_architecture",
           "resolve_architecture", "unregister_architecture", "read_json"]
