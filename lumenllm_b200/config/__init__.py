from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import (config_class_for, config_from_dict, known_architectures, load_config,
                       register_architecture)
from .qwen3 import Qwen3Config
from .params import ParametersFile, SamplingDefaults

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "Qwen3Config",
           "config_class_for", "config_from_dict", "known_architectures", "load_config",
           "register_architecture", "ParametersFile", "SamplingDefaults"]
