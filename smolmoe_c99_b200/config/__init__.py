"""Typed configurations and the registry from an architecture's name to its model."""
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec
from .registry import architectures, config_from_json, load_config, register_architecture
from .qwen2 import Qwen2Config

__all__ = [
    "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config",
    "architectures", "config_from_json", "load_config", "register_architecture",
]
