from .base import (ConfigError, ModelConfig, config_from_dict, known_architectures,
                   load_config, register_architecture)
from .engine import EngineConfig
from .spec import LayerSpec, ModelSpec, PartSpec, RunStep

__all__ = [
    "ConfigError", "ModelConfig", "config_from_dict", "known_architectures", "load_config",
    "register_architecture", "EngineConfig", "LayerSpec", "ModelSpec", "PartSpec", "RunStep",
]
