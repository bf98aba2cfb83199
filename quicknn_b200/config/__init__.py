"""Typed configurations and the registry from an architecture's name to its model."""
from .base import (Architecture, ConfigError, ModelConfig, find_architecture, load_config,
                   register_architecture, registered_architectures, unregister_architecture)
from .gemma2 import GEMMA2, Gemma2Config, gemma2_spec

__all__ = ["Architecture", "ConfigError", "ModelConfig", "find_architecture", "load_config",
           "register_architecture", "registered_architectures", "unregister_architecture",
           "GEMMA2", "Gemma2Config", "gemma2_spec"]
