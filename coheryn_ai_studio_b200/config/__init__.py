from .qwen2 import ConfigError, Qwen2Config, qwen2_model_spec, read_config_json
from .registry import (Architecture, Capabilities, GgufFace, describe_model, architecture_for, architecture_for_gguf, is_gguf, load_config,
                       register_architecture,
                       registered_architectures, unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, prenorm_layer

__all__ = [
    "ConfigError", "Capabilities", "describe_model", "GgufFace", "architecture_for_gguf", "is_gguf", "Qwen2Config", "qwen2_model_spec", "read_config_json", "Architecture",
    "architecture_for", "load_config", "register_architecture", "registered_architectures",
    "unregister_architecture", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "prenorm_layer",
]
