from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .qwen3 import ConfigError, Qwen3Config
from .registry import (
    config_from_dict,
    load_config,
    load_config_dict,
    load_preset,
    preset_names,
    register_architecture,
    registered_architectures,
)

register_architecture("Qwen3ForCausalLM", Qwen3Config, model_type="qwen3")

__all__ = [
    "ConfigError", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "Qwen3Config",
    "config_from_dict", "load_config", "load_config_dict", "load_preset", "preset_names",
    "register_architecture", "registered_architectures",
]
