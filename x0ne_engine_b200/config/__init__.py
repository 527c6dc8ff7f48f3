"""Typed configurations and the architecture registry."""
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry
from .registry import (architectures, config_from_dict, config_from_folder, detect,
                       register_architecture, spec_from_folder, unregister_architecture)
from .qwen3 import ARCHITECTURE as _QWEN3, MODEL_TYPE as _QWEN3_TYPE, Qwen3Config

register_architecture(_QWEN3, _QWEN3_TYPE, Qwen3Config)

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config",
           "architectures", "config_from_dict", "config_from_folder", "detect",
           "register_architecture", "spec_from_folder", "unregister_architecture"]
