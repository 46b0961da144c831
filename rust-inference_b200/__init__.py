"""rust-inference_b200: a small generation library for one B200.

Everything between a request's token ids and its next token, for the Qwen3
dense architecture of thanhauco/rust-inference: typed configuration and an
architecture registry (``config``, ``models``), weights from safetensors or from
a seed (``weights``), layers put together from registered parts (``parts``), a
paged cache with a slot per sequence (``cache``), one step function and a
generation loop (``engine``), sampling (``sampling``), and hand-written CUDA
kernels for sm_100a (``csrc``, ``ops``).
"""
from . import models  # noqa: F401  (registers the architectures)
from .api import LLM, generate
from .config import ConfigError, UnsupportedArchitecture, load_config, register_architecture
from .engine import Engine, Entry, Model
from .sampling import SamplingParams
from .weights import WeightsError, write_random_model

__all__ = ["LLM", "generate", "ConfigError", "UnsupportedArchitecture", "load_config", "register_architecture",
           "Engine", "Entry", "Model", "SamplingParams", "WeightsError", "write_random_model"]
__version__ = "0.1.0"
