from .qwen3 import ConfigError, Qwen3Config
from .registry import ARCHITECTURES, config_from_dict, load_config, register_architecture
from .spec import (
    AttentionSpec,
    GatedFeedForwardSpec,
    LayerSpec,
    ModelSpec,
    NormSpec,
    RopeSpec,
    ScheduleEntry,
    default_schedule,
    prenorm_layer,
)

__all__ = [
    "ARCHITECTURES",
    "AttentionSpec",
    "ConfigError",
    "GatedFeedForwardSpec",
    "LayerSpec",
    "ModelSpec",
    "NormSpec",
    "Qwen3Config",
    "RopeSpec",
    "ScheduleEntry",
    "config_from_dict",
    "default_schedule",
    "load_config",
    "prenorm_layer",
    "register_architecture",
]
