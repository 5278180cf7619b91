from .base import (ArchitectureEntry, ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, architecture,
                   architecture_name, known_architectures, load_config, read_config_dict, register_architecture)
from .gemma2 import Gemma2Config

__all__ = ["ArchitectureEntry", "ConfigError", "Gemma2Config", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry",
           "architecture", "architecture_name", "known_architectures", "load_config", "read_config_dict",
           "register_architecture"]
