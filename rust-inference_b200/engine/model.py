"""The model: an embedding, scheduled blocks, a final norm and an output head,
assembled from a :class:`~..config.specs.ModelSpec`.  Nothing here is specific
to an architecture: every one of those five is a registered part named by the
spec, and the order of work is thanhauco/rust-inference's
src/models/qwen3.rs:255-287 (embedding, layers, row selection, final norm,
output projection), with the row selection generalised to any wanted rows.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.registry import load_config
from ..parts import BuildEnv, ParamInfo, build_block, build_part, part_class
from ..profiler import section
from ..weights.loader import load_checkpoint
from ..weights.random_init import random_tensor

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def compute_dtype(name) -> torch.dtype:
    try:
        return _DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}") from None


def _end_name(full_weight_name: str, local: str) -> str:
    """The tensor name of an embedding's or a head's tensor: "weight" carries the given name itself,
    any other tensor the same name with "weight" replaced by its own."""
    if local == "weight":
        return full_weight_name
    stem = full_weight_name[:-len("weight")] if full_weight_name.endswith("weight") else full_weight_name + "."
    return stem + local


def _part_tensors(spec):
    """Yield (full tensor name, ParamInfo, owner key, local name) for every tensor of the model."""
    emb = spec.embedding_record()
    for local, info in part_class("embedding", emb).param_infos(emb).items():
        yield _end_name(spec.embedding_name, local), info, ("embedding",), local
    for local, info in part_class("norm", spec.final_norm).param_infos(spec.final_norm).items():
        yield spec.final_norm_prefix + local, info, ("final_norm",), local
    for i, layer in enumerate(spec.layers):
        for part, family, record in part_class("block", layer).slots(layer):
            for local, info in part_class(family, record).param_infos(record).items():
                yield layer.prefix(part) + local, info, ("layer", i, part), local
    head = spec.head_record()
    for local, info in part_class("head", head).param_infos(head).items():
        if local == "weight" and spec.tie_embeddings:
            continue                                   # the embedding's table
        yield _end_name(spec.head_name, local), info, ("head",), local


def expected_tensors(spec) -> Dict[str, ParamInfo]:
    """name -> ParamInfo of every tensor the checkpoint has to hold."""
    return {name: info for name, info, _, _ in _part_tensors(spec)}


class Model:
    def __init__(self, spec, dtype, device="cuda:0"):
        self.spec = spec
        self.env = BuildEnv(compute_dtype(dtype), torch.device(device))
        self.blocks = [build_block(ls, self.env) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, self.env)
        self.embed_part = build_part("embedding", spec.embedding_record(), self.env)
        self.head_part = build_part("head", spec.head_record(), self.env)
        self.config = None
        self.cache_entry_layers = spec.cache_entries()

    # the two big tables, as the tests and the bench look at them
    @property
    def embedding(self) -> Optional[torch.Tensor]:
        return getattr(self.embed_part, "table", None)

    @property
    def head(self) -> Optional[torch.Tensor]:
        return getattr(self.head_part, "weight", None)

    # ---- weights -------------------------------------------------------------------------
    def _to_role(self, t: torch.Tensor, role: str) -> torch.Tensor:
        want = {"matrix": self.env.dtype, "gain": torch.float32, "table": torch.int32}[role]
        return t.to(device=self.env.device, dtype=want).contiguous()

    def load_tensors(self, get) -> None:
        """``get(name, info)`` returns the tensor (any device, stored dtype) or None
        for an optional one.  Parts are fed one at a time so that the stored and
        the computing copy of the whole model never exist together."""
        spec = self.spec
        groups: Dict[tuple, Dict[str, torch.Tensor]] = {}
        order = []
        for name, info, owner, local in _part_tensors(spec):
            if owner not in groups:
                groups[owner] = {}
                order.append(owner)
            groups[owner][local] = (name, info)
        if ("head",) not in groups:
            groups[("head",)] = {}
            order.append(("head",))
        for owner in order:
            tensors = {}
            for local, (name, info) in groups[owner].items():
                t = get(name, info)
                # a head tensor that is absent means tied embeddings (src/models/qwen3.rs:166-171)
                if t is None and owner == ("head",) and local == "weight" and spec.head_optional:
                    continue
                tensors[local] = self._to_role(t, info.role)
            if owner == ("embedding",):
                self.embed_part.load(tensors)
            elif owner == ("final_norm",):
                self.final_norm.load(tensors)
            elif owner == ("head",):
                if "weight" not in tensors:
                    tensors["weight"] = self.embed_part.table          # tied: the same storage
                self.head_part.load(tensors)
            else:
                _, i, part = owner
                getattr(self.blocks[i], part).load(tensors)

    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", device="cuda:0") -> "Model":
        cfg = load_config(model_dir)
        spec = cfg.to_spec()
        model = cls(spec, dtype, device)
        model.config = cfg
        expected = {n: i.shape for n, i in expected_tensors(spec).items()}
        optional = {spec.head_name} if spec.head_optional else set()
        ignorable = {spec.head_name} if spec.tie_embeddings else set()
        tensors = load_checkpoint(model_dir, expected, optional=optional, ignorable=ignorable)
        model.load_tensors(lambda name, info: tensors.pop(name, None))
        return model

    @classmethod
    def from_random(cls, config, seed: int, dtype="bfloat16", device="cuda:0") -> "Model":
        """Random weights made on the device, tensor by tensor (no folder is written):
        the same distributions as the random-weights mode, for sizes whose file would
        take tens of gigabytes."""
        from ..config.registry import config_from_dict
        cfg = config_from_dict(config) if isinstance(config, dict) else config
        model = cls(cfg.to_spec(), dtype, device)
        model.config = cfg
        dev = model.env.device
        model.load_tensors(lambda name, info: random_tensor(seed, name, info.shape, info.role, model.env.dtype
                                                            if info.role == "matrix" else torch.float32, dev))
        return model

    # ---- what the cache has to hold -----------------------------------------------------------
    def cache_requests(self):
        return [self.blocks[layer].mixer.cache_request() for layer in self.cache_entry_layers]

    @property
    def graph_safe(self) -> bool:
        """Whether one-token steps of this model may be replayed from a CUDA graph."""
        parts = [p for b in self.blocks for _, p, _, _ in b.parts()] + [self.final_norm, self.embed_part, self.head_part]
        parts += [b.mixer.position for b in self.blocks if hasattr(b.mixer, "position")]
        return all(getattr(p, "graph_safe", False) for p in parts)

    def prepare(self, max_positions: int) -> None:
        for b in self.blocks:
            b.mixer.prepare(max_positions)

    def weight_bytes(self, with_embedding: bool = False) -> int:
        """Bytes of the matrices a step reads once each (the head included; the
        embedding only counts when asked, a step reads a few rows of it)."""
        n = sum(p.weight_bytes() for b in self.blocks for _, p, _, _ in b.parts())
        n += self.final_norm.weight_bytes() + self.head_part.weight_bytes()
        if with_embedding and self.head is not self.embedding:
            n += self.embed_part.weight_bytes()
        return n

    # ---- one step ------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, ctx, cache, want_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """float32 logits [wanted rows, vocab] for the packed tokens ``ids``."""
        with section("embedding"):
            resid = self.embed_part(ids, ctx)
        delta = None
        for e in self.spec.schedule:
            resid, delta = self.blocks[e.layer](resid, delta, ctx, cache.layer(e.cache, e.writes))
        if self.final_norm.takes_hint:
            x = self.final_norm(resid, delta, want_rows, self.head_part.reads_first())
        else:
            x = self.final_norm(resid, delta, rows=want_rows)
        with section("lm head"):
            return self.head_part(x)
