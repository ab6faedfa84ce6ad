from .base import (ArchConfig, ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                   read_config_json, take)
from .llama import LlamaConfig

__all__ = ["ArchConfig", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry",
           "LlamaConfig", "read_config_json", "take"]
