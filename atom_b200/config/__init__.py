from .engine_config import EngineConfig
from .model_config import (
    ConfigError,
    ModelConfig,
    config_from_dict,
    load_model_config,
    save_model_config,
)

__all__ = [
    "ConfigError", "EngineConfig", "ModelConfig", "config_from_dict", "load_model_config",
    "save_model_config",
]
