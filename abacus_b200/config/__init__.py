from .registry import (ConfigError, architecture_names, architecture_of, get_architecture, load_config,
                       read_config_json, register_architecture)
from .specs import (AttentionSpec, BlockSpec, GatedMLPSpec, ModelSpec, NormSpec, RotarySpec, ScheduleEntry)
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "architecture_names", "architecture_of", "get_architecture", "load_config",
           "read_config_json", "register_architecture", "AttentionSpec", "BlockSpec", "GatedMLPSpec", "ModelSpec",
           "NormSpec", "RotarySpec", "ScheduleEntry", "Qwen3Config"]
