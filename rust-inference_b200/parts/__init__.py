"""The parts a model is made of, each behind a registry keyed by ``kind``."""
from .base import BuildEnv, CacheRequest, FeedForward, Mixer, Norm, Part, PositionEncoding, StepContext
from .registry import (ParamInfo, build_part, part_class, register_block, register_embedding, register_ffn,
                       register_head, register_mixer, register_norm, register_position, registered)
from . import attention, ends, mlp, norm, position  # noqa: F401  (registers the built-in parts)
from .block import BlockBase, build_block, norm_before

__all__ = ["BuildEnv", "CacheRequest", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "StepContext",
           "ParamInfo", "build_part", "part_class", "register_block", "register_embedding", "register_ffn",
           "register_head", "register_mixer", "register_norm", "register_position", "registered",
           "BlockBase", "build_block", "norm_before"]
