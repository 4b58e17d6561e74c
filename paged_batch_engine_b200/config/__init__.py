from .specs import BlockSpec, ConfigError, ModelSpec, PartSpec, RunStep
from .registry import (Architecture, architecture_name_of, get_architecture, known_architectures,
                       load_config, register_architecture)
from .qwen2 import Qwen2Config
from .gebadra import GebadraConfig
from .bavetar import BavetarConfig
from .gusorax import GusoraxConfig
from .mobunex import MobunexConfig

register_architecture("Qwen2ForCausalLM", Qwen2Config, replace=True)
register_architecture("Gebadra", GebadraConfig, replace=True)
register_architecture("Bavetar", BavetarConfig, replace=True)
register_architecture("Gusorax", GusoraxConfig, replace=True)
register_architecture("Mobunex", MobunexConfig, replace=True)

__all__ = ["BlockSpec", "ConfigError", "ModelSpec", "PartSpec", "RunStep", "Architecture",
           "architecture_name_of", "get_architecture", "known_architectures", "load_config",
           "register_architecture", "Qwen2Config", "GebadraConfig", "BavetarConfig", "GusoraxConfig", "MobunexConfig"]
