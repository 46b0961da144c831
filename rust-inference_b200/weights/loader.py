"""Weights by tensor name, checked against what the model expects.

``load_checkpoint`` opens a model folder, compares the tensors it holds with
the expected names and shapes and raises ONE :class:`WeightsError` that lists
everything wrong: missing tensors, unexpected tensors, wrong shapes.  Tensors
are returned as stored: bfloat16 stays bfloat16, a tensor stored in 32-bit stays
32-bit, float16 is widened to float32, integer tables become int32.  Moving to
the device and to the dtype a part computes in is the model's business.
"""
from __future__ import annotations

from typing import Dict, Iterable, Mapping, Tuple

import torch

from .safetensors_io import Checkpoint, SafetensorsError


class WeightsError(ValueError):
    def __init__(self, model_dir, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"weights in {model_dir} do not fit the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        lines.extend(f"  {o}" for o in other)
        super().__init__("\n".join(lines))


def _as_stored(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype in (torch.float16, torch.float64):
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    raise SafetensorsError(f"dtype {t.dtype} is not supported")


def load_checkpoint(model_dir: str, expected: Mapping[str, Tuple[int, ...]],
                    optional: Iterable[str] = (), ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """``expected``: name -> shape.  ``optional`` names may be absent;
    ``ignorable`` names may be present without being expected."""
    ckpt = Checkpoint(model_dir)
    optional, ignorable = set(optional), set(ignorable)
    have = set(ckpt.names())
    missing = sorted(n for n in expected if n not in have and n not in optional)
    unexpected = sorted(n for n in have if n not in expected and n not in ignorable)
    wrong = []
    for n in sorted(expected):
        if n in have:
            shape, _ = ckpt.shape_dtype(n)
            if tuple(shape) != tuple(expected[n]):
                wrong.append((n, tuple(shape), tuple(expected[n])))
    if missing or unexpected or wrong:
        raise WeightsError(model_dir, missing, unexpected, wrong)
    return {n: _as_stored(ckpt.tensor(n)) for n in expected if n in have}
