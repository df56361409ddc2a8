from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from .registry import config_class_for, read_config, register_architecture, registered_architectures
from .llama import LlamaConfig

__all__ = ["ConfigError", "LayerSpec", "ModelPlan", "PartSpec", "ScheduleEntry", "config_class_for", "read_config",
           "register_architecture", "registered_architectures", "LlamaConfig"]
