from .base import ConfigError, KeyReader, ModelConfig
from .qwen2 import Qwen2Config
from .registry import (Architecture, config_from_dict, get_architecture, known_architectures, load_config,
                       register_architecture, unregister_architecture)
