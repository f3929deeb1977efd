from .engine_config import EngineConfig, canonical_dtype
from .model_config import (Architecture, ConfigError, architecture_of, get_architecture,
                           load_model_config, register_architecture,
                           registered_architectures, unregister_architecture)
from .presets import preset, preset_names

__all__ = [
    "Architecture", "ConfigError", "EngineConfig", "architecture_of", "canonical_dtype",
    "get_architecture", "load_model_config", "preset", "preset_names",
    "register_architecture", "registered_architectures", "unregister_architecture",
]
