"""Typed configuration: part records (``specs``) and the architecture registry."""
from .specs import (AttentionSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, NoPositionSpec, RMSNormSpec, RopeSpec,
                    ScheduleEntry, SwiGLUSpec)
from .registry import (ConfigError, UnsupportedArchitecture, architecture_of, config_from_dict,
                       load_config, register_architecture, registered_architectures)

__all__ = [
    "AttentionSpec", "EmbeddingSpec", "HeadSpec", "LayerSpec", "ModelSpec", "NoPositionSpec", "RMSNormSpec", "RopeSpec",
    "ScheduleEntry", "SwiGLUSpec", "ConfigError", "UnsupportedArchitecture", "architecture_of",
    "config_from_dict", "load_config", "register_architecture", "registered_architectures",
]
