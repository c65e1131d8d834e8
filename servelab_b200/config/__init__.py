"""Typed configuration: model specs as data, family configs, engine knobs."""

from .engine import CacheConfig, EngineConfig, SchedulerConfig
from .qwen2 import ConfigError, Qwen2Config
from .registry import (config_from_dict, load_config, model_spec_from_config,
                       register_architecture, registered_architectures,
                       resolve_architecture)
from .specs import (AttentionSpec, BlockSpec, GatedMLPSpec, LayerRun, ModelSpec,
                    NoPositionSpec, PartSpec, RMSNormSpec, RotarySpec)

register_architecture(Qwen2Config.architecture, Qwen2Config, model_type=Qwen2Config.model_type)

__all__ = [
    "AttentionSpec", "BlockSpec", "CacheConfig", "ConfigError", "EngineConfig",
    "GatedMLPSpec", "LayerRun", "ModelSpec", "NoPositionSpec", "PartSpec",
    "Qwen2Config", "RMSNormSpec", "RotarySpec", "SchedulerConfig",
    "config_from_dict", "load_config", "model_spec_from_config",
    "register_architecture", "registered_architectures", "resolve_architecture",
]
