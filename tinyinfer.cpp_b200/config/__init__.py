"""Typed configurations, the architecture registry and the architecture-independent plan."""
from .plan import LayerPlan, ModelPlan, PartSpec, ScheduleEntry, default_schedule
from .registry import (Architecture, ConfigError, architecture_of, get_architecture,
                       known_architectures, load_config, read_config_json,
                       register_architecture)
from .qwen3 import Qwen3Config
from .kagorax import KagoraxConfig
from .ruvuvik import RuvuvikConfig
from .feruzen import FeruzenConfig
from .nekorax import NekoraxConfig

__all__ = [
    "Architecture", "ConfigError", "FeruzenConfig", "KagoraxConfig", "LayerPlan", "ModelPlan", "NekoraxConfig", "PartSpec", "Qwen3Config", "RuvuvikConfig",
    "ScheduleEntry", "architecture_of", "default_schedule", "get_architecture",
    "known_architectures", "load_config", "read_config_json", "register_architecture",
]
