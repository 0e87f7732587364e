from .spec import PartSpec, LayerSpec, RunSpec, ModelSpec
from .qwen2 import Qwen2Config, ConfigError, preset, PRESETS
from .registry import (Architecture, register_architecture, get_architecture, architectures,
                       architecture_of, architecture_for, find_preset, parameter_count, load_config)

__all__ = ["PartSpec", "LayerSpec", "RunSpec", "ModelSpec", "Qwen2Config", "ConfigError", "preset",
           "PRESETS", "Architecture", "register_architecture", "get_architecture", "architectures",
           "architecture_of", "architecture_for", "find_preset", "parameter_count", "load_config"]
