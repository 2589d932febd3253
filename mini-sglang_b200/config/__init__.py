from .registry import ARCHITECTURES, ConfigError, architecture_of, load_config, read_config_json, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, Run
from . import qwen3 as _qwen3  # registers "Qwen3ForCausalLM"
from .qwen3 import Qwen3Config

__all__ = ["ARCHITECTURES", "ConfigError", "architecture_of", "load_config", "read_config_json",
           "register_architecture", "LayerSpec", "ModelSpec", "PartSpec", "Run", "Qwen3Config"]
