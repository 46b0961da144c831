"""Sampling: options, random streams, device sampler."""
from .sampler import Sampler, SamplingParams, XorShiftRng, request_seed

__all__ = ["Sampler", "SamplingParams", "XorShiftRng", "request_seed"]
