"""Typed configurations and the registry from an architecture's name to its model."""
from .registry import (ConfigError, config_class_for, config_from_dict, load_config,
                       register_architecture, registered_architectures)
from .spec import ArchitectureSpec, LayerSpec, PartSpec, RunEntry
from .llama import LlamaConfig, RopeScaling
from .dedutar import DedutarConfig
from .monolix import MonolixConfig
from .bazurax import BazuraxConfig
from .ragilorn import RagilornConfig

__all__ = [
    "ArchitectureSpec", "BazuraxConfig", "ConfigError", "DedutarConfig", "LayerSpec", "LlamaConfig", "MonolixConfig", "PartSpec", "RagilornConfig", "RopeScaling", "RunEntry",
    "config_class_for", "config_from_dict", "load_config", "register_architecture", "registered_architectures",
]
