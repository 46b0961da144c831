"""Model, step function and generation loop."""
from .engine import Engine, Entry, StepError
from .generate import GenerationResult, GenerationStats, generate, plan_batches
from .model import Model, compute_dtype, expected_tensors

__all__ = ["Engine", "Entry", "StepError", "GenerationResult", "GenerationStats", "generate", "plan_batches",
           "Model", "compute_dtype", "expected_tensors"]
