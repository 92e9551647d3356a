"""Configuration: typed architecture configs, the model spec they produce, the registry."""

from .qwen2 import ARCHITECTURE as QWEN2_ARCHITECTURE
from .qwen2 import ConfigError, Qwen2Config
from .registry import (config_class_for, load_config, register_architecture,
                       supported_architectures, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, RunSpec

register_architecture(QWEN2_ARCHITECTURE, Qwen2Config)

__all__ = ["ConfigError", "Qwen2Config", "QWEN2_ARCHITECTURE", "LayerSpec", "ModelSpec",
           "PartSpec", "RunSpec", "config_class_for", "load_config",
           "register_architecture", "supported_architectures", "unregister_architecture"]
