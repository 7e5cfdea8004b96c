from .base import ConfigError, load_config_dict
from .llama import LlamaConfig, RopeScaling
from .registry import (Architecture, config_from_dict, config_from_model_dir, lookup_architecture,
                       register_architecture, registered_architectures, unregister_architecture)
from .spec import (BlockSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule, describe,
                   validate_schedule)

__all__ = [
    "ConfigError", "LlamaConfig", "RopeScaling", "load_config_dict", "Architecture", "config_from_dict",
    "config_from_model_dir", "lookup_architecture", "register_architecture", "registered_architectures",
    "unregister_architecture", "BlockSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule",
    "describe", "validate_schedule",
]
