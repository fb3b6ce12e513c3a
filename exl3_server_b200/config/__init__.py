"""Typed configurations and the architecture registry."""
from .fields import ConfigError, KeyReader, read_config_json
from .llama import LlamaConfig
from .nibelix import NibelixConfig, NibelixLayer
from .nikodra import NikodraConfig, NikodraLayer
from .potodra import PotodraConfig, PotodraLayer
from .rigitar import RigitarConfig, RigitarLayer
from .registry import (Architecture, register_architecture, registered_names,
                       resolve_architecture, unregister_architecture)

__all__ = ["ConfigError", "KeyReader", "read_config_json", "LlamaConfig", "RigitarConfig", "RigitarLayer", "NikodraConfig", "NikodraLayer", "NibelixConfig", "NibelixLayer", "PotodraConfig", "PotodraLayer", "Architecture",
           "register_architecture", "registered_names", "resolve_architecture",
           "unregister_architecture"]
