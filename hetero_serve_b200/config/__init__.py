from .engine_config import EngineConfig, canonical_dtype
from .model_config import (Architecture, ConfigError, GPT2Config, architecture_of,
                           get_architecture, load_model_config, register_architecture,
                           registered_architectures, unregister_architecture)
from .presets import PRESETS, preset

__all__ = [
    "Architecture", "ConfigError", "EngineConfig", "GPT2Config", "PRESETS",
    "architecture_of", "canonical_dtype", "get_architecture", "load_model_config",
    "preset", "register_architecture", "registered_architectures",
    "unregister_architecture",
]
