"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed, or the same tensors made on the device without a file.

Matrices and the embedding are N(0, 0.02), norm gains (the per-head q/k norms
included) 1 + U(-0.1, 0.1), integer tables zero.  A value is a function of
(seed, tensor name, element index) and of nothing else (``csrc/random_fill.cuh``):
the host code and the device kernel give the same bits, a tensor's values do not
depend on which other tensors exist, and any part of a tensor (a few rows of an
embedding, say) can be made alone.  So a model of tens of gigabytes can be made on
the device for the engine and, tensor by tensor, on the host for a comparison,
without ever being written.  The tensor list comes from the parts the
architecture is made of, so this works for any registered architecture.
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
from typing import Dict

import torch

from ..config.registry import config_from_dict
from .safetensors_io import save_safetensors

_MASK = (1 << 64) - 1
MATRIX_STD = 0.02          # linears and the embedding (scripts/synthetic_checkpoint.py:135-152 of the reference)
GAIN_SPREAD = 0.2          # norm gains: 1 + U(-0.1, 0.1)


def _mix64(z: int) -> int:
    z &= _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's stream of values."""
    h = int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "little")
    return _mix64((int(seed) & _MASK) ^ _mix64(h))


_U64, _P, _I, _D = ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_int, ctypes.c_double


def _fill(out: torch.Tensor, key: int, first: int, kind: int, a: float, b: float) -> None:
    from ..csrc import build
    code = {torch.float32: 0, torch.bfloat16: 1}[out.dtype]
    if out.is_cuda:
        lib = build.library("random_fill")
        fn = lib.ri_random_fill
        fn.argtypes, fn.restype = [_P, _U64, _U64, _U64, _I, _D, _D, _I, _P], _I
        with torch.cuda.device(out.device):
            rc = fn(out.data_ptr(), key, first, out.numel(), kind, a, b, code, torch.cuda.current_stream().cuda_stream)
    else:
        lib = build.library("host_random")
        fn = lib.ri_random_fill_host
        fn.argtypes, fn.restype = [_P, _U64, _U64, _U64, _I, _D, _D, _I, _I], _I
        rc = fn(out.data_ptr(), key, first, out.numel(), kind, a, b, code, 0)
    if rc:
        raise RuntimeError(f"random fill: {lib.ri_last_error().decode(errors='replace')}")


def random_tensor(seed: int, name: str, shape, role: str, dtype: torch.dtype, device="cpu",
                  first_row: int = 0) -> torch.Tensor:
    """The tensor ``name`` of the random model with this seed, made where ``device`` says.
    ``shape`` with ``first_row`` > 0 gives rows first_row .. first_row + shape[0] - 1 of it."""
    shape = tuple(int(d) for d in shape)
    if role == "table":
        return torch.zeros(shape, dtype=torch.int32, device=device)
    if role not in ("matrix", "gain"):
        raise ValueError(f"unknown parameter role {role!r}")
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"random weights are float32 or bfloat16, not {dtype}")
    out = torch.empty(shape, dtype=dtype, device=device)
    row = 1
    for d in shape[1:]:
        row *= d
    if role == "matrix":
        _fill(out, tensor_key(seed, name), first_row * row, 0, MATRIX_STD, 0.0)
    else:
        _fill(out, tensor_key(seed, name), first_row * row, 1, 1.0, GAIN_SPREAD)
    return out


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
    expected = expected_tensors(spec)
    os.makedirs(out_dir, exist_ok=True)
    save_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(expected, seed, tdt))
    d = dict(config)
    d.setdefault("torch_dtype", dtype)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(d, f, indent=2)
    return out_dir
