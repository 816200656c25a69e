"""Configuration: typed per-architecture configs, the part specs, the registry."""
from .registry import (ConfigError, config_class_for, config_from_dict, load_config,
                       register_architecture, registered_architectures, save_config,
                       unregister_architecture)
from .specs import (BlockSpec, FeedForwardSpec, MixerSpec, ModelPlan, NormSpec,
                    PositionSpec, StageSpec)
from .qwen3 import Qwen3Config

__all__ = [
    "ConfigError", "config_class_for", "config_from_dict", "load_config",
    "register_architecture", "registered_architectures", "save_config",
    "unregister_architecture", "BlockSpec", "FeedForwardSpec", "MixerSpec", "ModelPlan",
    "NormSpec", "PositionSpec", "StageSpec", "Qwen3Config",
]
