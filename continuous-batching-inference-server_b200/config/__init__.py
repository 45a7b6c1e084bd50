from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec
from .registry import (architecture_name, config_from_dict, known_architectures, load_config,
                       register_architecture)
from .gpt2 import GPT2Config

for _name in ("GPT2LMHeadModel", "TinyGPT", "gpt2"):
    register_architecture(_name, GPT2Config)

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "GPT2Config", "architecture_name",
           "config_from_dict", "known_architectures", "load_config", "register_architecture"]
