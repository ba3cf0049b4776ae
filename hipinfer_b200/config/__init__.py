from .base import (Architecture, ConfigError, ModelConfig, config_from_dict, get_architecture, load_config,
                   register_architecture, registered_architectures, save_config, take)
from .llama import Llama3RopeScaling, LlamaConfig

__all__ = ["Architecture", "ConfigError", "ModelConfig", "config_from_dict", "get_architecture", "load_config",
           "register_architecture", "registered_architectures", "save_config", "take", "Llama3RopeScaling",
           "LlamaConfig"]
