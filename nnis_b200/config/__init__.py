from .llama import ConfigError, LlamaConfig
from .registry import (config_from_dict, known_architectures, read_config,
                       register_architecture, spec_from_dir)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = ["ConfigError", "LlamaConfig", "config_from_dict", "known_architectures",
           "read_config", "register_architecture", "spec_from_dir", "LayerSpec", "ModelSpec",
           "PartSpec", "ScheduleEntry"]
