"""Weights: safetensors by tensor name, checked loading, random-weights mode."""
from .loader import WeightsError, load_checkpoint
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, save_safetensors

__all__ = ["WeightsError", "load_checkpoint", "random_tensor", "random_tensors", "write_random_model",
           "Checkpoint", "SafetensorsError", "SafetensorsFile", "save_safetensors"]
