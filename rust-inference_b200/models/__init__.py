"""Architectures.  Importing this package registers them."""
from . import qwen3  # noqa: F401
from .qwen3 import Qwen3Config

__all__ = ["Qwen3Config"]
