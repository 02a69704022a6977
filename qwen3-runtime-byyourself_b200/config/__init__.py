"""Configuration: typed per-architecture classes, the registry, and the model plan."""
from .plan import LayerSpec, ModelPlan, PartSpec
from .registry import (ConfigError, config_class_for, config_from_dict, known_architectures,
                       load_config, register_architecture)
from .qwen3 import Qwen3Config

__all__ = ["LayerSpec", "ModelPlan", "PartSpec", "ConfigError", "config_class_for", "config_from_dict",
           "known_architectures", "load_config", "register_architecture", "Qwen3Config"]
