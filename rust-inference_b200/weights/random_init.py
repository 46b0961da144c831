"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed.

Matrices and the embedding are N(0, 0.02), norm gains (the per-head q/k norms
included) 1 + U(-0.1, 0.1), integer tables zero.  Every tensor has a generator
of its own, seeded from (seed, tensor name), so a tensor's values do not depend
on which other tensors exist.  The tensor list comes from the parts the
architecture is made of, so this works for any registered architecture.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from ..config.registry import config_from_dict
from .safetensors_io import save_safetensors


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(h[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensor(seed: int, name: str, shape, role: str, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    g = _generator(seed, name, device)
    if role == "matrix":
        return (torch.randn(shape, generator=g, dtype=torch.float32, device=device) * 0.02).to(dtype)
    if role == "gain":
        return (1.0 + (torch.rand(shape, generator=g, dtype=torch.float32, device=device) * 0.2 - 0.1)).to(dtype)
    if role == "table":
        return torch.zeros(shape, dtype=torch.int32, device=device)
    raise ValueError(f"unknown parameter role {role!r}")


def random_tensors(expected: Dict[str, object], seed: int, dtype: torch.dtype, device="cpu") -> Dict[str, torch.Tensor]:
    """``expected``: name -> ParamInfo."""
    return {n: random_tensor(seed, n, info.shape, info.role, dtype, device) for n, info in sorted(expected.items())}


def write_random_model(config: dict, seed: int, out_dir: str, dtype: str = "bfloat16") -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns ``out_dir``.

    ``config`` holds config.json keys (it is checked first); ``dtype`` is the
    stored dtype of all float tensors: "bfloat16" or "float32"."""
    from ..engine.model import expected_tensors       # parts -> tensor list
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    cfg = config_from_dict(config)
    spec = cfg.to_spec()
    expected = expected_tensors(spec, for_writing=True)
    os.makedirs(out_dir, exist_ok=True)
    save_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(expected, seed, tdt))
    d = dict(config)
    d.setdefault("torch_dtype", dtype)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(d, f, indent=2)
    return out_dir
