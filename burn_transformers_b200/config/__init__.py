from .base import ModelConfig, detect_model_type, read_json_object
from .gpt2 import Gpt2Config
from .registry import (Architecture, architecture_for, config_from_folder,
                       register_architecture, supported_model_types, unregister_architecture)

__all__ = ["ModelConfig", "Gpt2Config", "Architecture", "architecture_for", "config_from_folder",
           "register_architecture", "supported_model_types", "unregister_architecture",
           "detect_model_type", "read_json_object"]
