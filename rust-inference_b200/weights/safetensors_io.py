"""safetensors files: a memory-mapped reader and a writer.

File layout (thanhauco/rust-inference src/safetensors.rs:3-6, 56-83): a
little-endian u64 header length, a JSON header ``name -> {dtype, shape,
data_offsets:[start,end]}`` with offsets relative to the end of the header,
then raw little-endian data.  ``model.safetensors.index.json`` maps tensor
names to shard files (src/safetensors.rs:157-191).

Tensors come back as torch CPU tensors that view the mapping (no copy) in
their stored dtype.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "U8": (torch.uint8, 1), "F64": (torch.float64, 8),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One ``.safetensors`` file, mapped read-only."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e}") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path} is too small to be a safetensors file")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header runs past the end of the file")
        try:
            header = json.loads(self._map[8:8 + hlen])
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from e
        base = 8 + hlen
        self.info: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, rec in header.items():
            if name == "__metadata__":
                continue
            dt = rec.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: {name} has unsupported dtype {dt!r}")
            shape = tuple(int(s) for s in rec["shape"])
            lo, hi = rec["data_offsets"]
            numel = 1
            for s in shape:
                numel *= s
            if hi - lo != numel * _DTYPES[dt][1] or base + hi > size or lo < 0:
                raise SafetensorsError(f"{path}: bad data offsets for {name}")
            self.info[name] = (dt, shape, base + lo, base + hi)
        self._buf = memoryview(self._map)

    def names(self) -> Iterable[str]:
        return self.info.keys()

    def shape_dtype(self, name: str):
        dt, shape, _, _ = self.info[name]
        return shape, _DTYPES[dt][0]

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, lo, hi = self.info[name]
        tdt = _DTYPES[dt][0]
        if hi == lo:
            return torch.empty(shape, dtype=tdt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # the mapping is read-only; nobody writes to it
            t = torch.frombuffer(self._buf, dtype=torch.uint8, count=hi - lo, offset=lo)
        if lo % _DTYPES[dt][1]:
            t = t.clone()                            # misaligned data: aligned copy
        return t.view(tdt).reshape(shape)


class Checkpoint:
    """All tensors of a model folder: ``model.safetensors`` or an index of shards."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(single):
            f = self._open("model.safetensors")
            for n in f.names():
                self._where[n] = "model.safetensors"
        elif os.path.exists(index):
            with open(index) as fh:
                wm = json.load(fh).get("weight_map")
            if not isinstance(wm, dict):
                raise SafetensorsError(f"{index} has no weight_map")
            for n, shard in wm.items():
                self._where[n] = shard
            for shard in sorted(set(wm.values())):
                f = self._open(shard)
                for n, s in wm.items():
                    if s == shard and n not in f.info:
                        raise SafetensorsError(f"{index} places {n} in {shard}, which does not hold it")
        else:
            raise SafetensorsError(f"{model_dir} holds neither model.safetensors nor model.safetensors.index.json")

    def _open(self, shard: str) -> SafetensorsFile:
        if shard not in self._files:
            self._files[shard] = SafetensorsFile(os.path.join(self.model_dir, shard))
        return self._files[shard]

    def names(self):
        return self._where.keys()

    def __contains__(self, name):
        return name in self._where

    def shape_dtype(self, name):
        return self._open(self._where[name]).shape_dtype(name)

    def tensor(self, name):
        return self._open(self._where[name]).tensor(name)


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    """Write tensors in name order, header padded so that data starts 8-byte aligned
    (as the reference's writers do, src/safetensors.rs:234-257)."""
    header, off = {}, 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"{name}: dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - (8 + len(h)) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
