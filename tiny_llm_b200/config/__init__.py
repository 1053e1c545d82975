from .errors import ConfigError
from .registry import (config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .llama import LlamaConfig

__all__ = ["ConfigError", "LlamaConfig", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec",
           "config_class_for", "config_from_dict", "load_config", "register_architecture",
           "registered_architectures"]
