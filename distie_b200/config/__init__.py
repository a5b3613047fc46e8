"""Typed configurations and the architecture registry."""

from .engine_config import EngineConfig, resolve_dtype_name
from .model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .qwen2_config import ConfigError, Qwen2Config
from .registry import (
    Architecture,
    architecture_of,
    get_architecture,
    known_architectures,
    read_config,
    register_architecture,
    unregister_architecture,
)

__all__ = [
    "Architecture",
    "ConfigError",
    "EngineConfig",
    "LayerCall",
    "LayerSpec",
    "ModelSpec",
    "PartSpec",
    "Qwen2Config",
    "architecture_of",
    "get_architecture",
    "known_architectures",
    "read_config",
    "register_architecture",
    "resolve_dtype_name",
    "unregister_architecture",
]
