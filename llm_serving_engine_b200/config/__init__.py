from .model_config import ConfigError, LayerSpec, ModelSpec, PartSpec, Qwen2Config
from .registry import (Architecture, known_architectures, load_config, register_architecture,
                       resolve_architecture)
from .runtime_config import CacheConfig, SchedulerConfig

__all__ = [
    "Architecture", "CacheConfig", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec",
    "Qwen2Config", "SchedulerConfig", "known_architectures", "load_config",
    "register_architecture", "resolve_architecture",
]
