from .engine import EngineConfig, ceil_div
from .registry import (
    config_class_for,
    config_from_dict,
    known_architectures,
    load_config,
    register_architecture,
)
from .spec import LayerSpec, ModelSpec, NormSlot, PartSpec, ScheduleEntry
from .qwen2 import Qwen2Config

__all__ = [
    "EngineConfig",
    "LayerSpec",
    "ModelSpec",
    "NormSlot",
    "PartSpec",
    "Qwen2Config",
    "ScheduleEntry",
    "ceil_div",
    "config_class_for",
    "config_from_dict",
    "known_architectures",
    "load_config",
    "register_architecture",
]
