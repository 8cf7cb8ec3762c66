from .base import (ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry)
from .qwen3 import Qwen3Config
from .registry import (config_class, config_from_dict, load_config, register_architecture,
                       supported_architectures)

register_architecture("Qwen3ForCausalLM", Qwen3Config)

__all__ = ["ConfigError", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config",
           "config_class", "config_from_dict", "load_config", "register_architecture",
           "supported_architectures"]
