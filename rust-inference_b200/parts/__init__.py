"""The parts a layer is made of, each behind a registry keyed by ``kind``."""
from .base import BuildEnv, CacheRequest, FeedForward, Mixer, Norm, Part, PositionEncoding, StepContext
from .registry import (ParamInfo, build_part, part_class, register_ffn, register_mixer, register_norm,
                       register_position, registered)
from . import attention, mlp, norm, position  # noqa: F401  (registers the built-in parts)
from .block import Block

__all__ = ["BuildEnv", "CacheRequest", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "StepContext",
           "ParamInfo", "build_part", "part_class", "register_ffn", "register_mixer", "register_norm",
           "register_position", "registered", "Block"]
