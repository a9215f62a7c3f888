from .engine_config import EngineConfig, SchedulerConfig, resolve_dtype
from .model_config import ConfigError, ModelConfig, Qwen2Config, read_config_json
from .registry import (
    Architecture,
    architecture_of,
    get_architecture,
    load_model_config,
    register_architecture,
    supported_architectures,
    unregister_architecture,
)

__all__ = [
    "Architecture",
    "ConfigError",
    "EngineConfig",
    "ModelConfig",
    "Qwen2Config",
    "SchedulerConfig",
    "architecture_of",
    "get_architecture",
    "load_model_config",
    "read_config_json",
    "register_architecture",
    "resolve_dtype",
    "supported_architectures",
    "unregister_architecture",
]
