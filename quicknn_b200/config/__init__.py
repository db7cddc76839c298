"""Typed configurations and the registry from an architecture's name to its model."""
from .base import (Architecture, ConfigError, ModelConfig, find_architecture, load_config,
                   register_architecture, registered_architectures, unregister_architecture)
from .gemma2 import GEMMA2, Gemma2Config, gemma2_spec
from .fuposun import FUPOSUN, FuposunConfig, fuposun_spec
from .tumudra import TUMUDRA, TumudraConfig, tumudra_spec
from .mubasun import MUBASUN, MubasunConfig, mubasun_spec
from .gunirax import GUNIRAX, GuniraxConfig, gunirax_spec

__all__ = ["Architecture", "ConfigError", "ModelConfig", "find_architecture", "load_config",
           "register_architecture", "registered_architectures", "unregister_architecture",
           "GEMMA2", "Gemma2Config", "gemma2_spec", "FUPOSUN", "FuposunConfig", "fuposun_spec",
           "TUMUDRA", "TumudraConfig", "tumudra_spec", "MUBASUN", "MubasunConfig", "mubasun_spec",
           "GUNIRAX", "GuniraxConfig", "gunirax_spec"]
