"""Typed configurations and the architecture registry."""
from .base import (
    ArchitectureEntry,
    ConfigError,
    ModelConfig,
    known_architectures,
    load_config,
    read_config_json,
    register_architecture,
    resolve_architecture,
    unregister_architecture,
)
from .bubalix import BubalixConfig
from .delunex import DelunexConfig
from .luzitar import LuzitarConfig
from .pilonex import PilonexConfig
from .qwen3 import Qwen3Config

__all__ = [
    "ArchitectureEntry", "BubalixConfig", "ConfigError", "DelunexConfig", "LuzitarConfig", "ModelConfig", "PilonexConfig", "Qwen3Config", "known_architectures",
    "load_config", "read_config_json", "register_architecture", "resolve_architecture",
    "unregister_architecture",
]
