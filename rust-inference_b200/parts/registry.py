"""Registries of part classes by kind, and the record every parameter is declared with.

A part class is registered for the ``kind`` of its spec record::

    @register_mixer("attention")
    class Attention(Mixer): ...

and is built by ``build_part("mixer", spec, env)`` wherever a layer's record names that
kind.  The arrangement of a layer's parts (``block``, named by ``LayerSpec.arrangement``), the
embedding and the output head are registered in the same way.  Tests register toy parts like
this; nothing else has to change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple

_REGISTRIES: Dict[str, Dict[str, type]] = {"mixer": {}, "ffn": {}, "norm": {}, "position": {}, "block": {},
                                           "embedding": {}, "head": {}}


@dataclass(frozen=True)
class ParamInfo:
    """A tensor that a part wants from the checkpoint.

    role "matrix": kept in the compute dtype, random init N(0, 0.02);
    role "gain":   kept in float32, random init 1 + U(-0.1, 0.1);
    role "table":  integer table, kept as int32, random init zeros.
    """
    shape: Tuple[int, ...]
    role: str = "matrix"


def _register(family: str, kind: str):
    def deco(cls):
        _REGISTRIES[family][kind] = cls
        cls.kind = kind
        return cls
    return deco


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_ffn(kind: str):
    return _register("ffn", kind)


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_block(kind: str):
    """The arrangement of a layer's parts (``LayerSpec.arrangement`` names it)."""
    return _register("block", kind)


def register_embedding(kind: str):
    """What turns token ids into the residual stream."""
    return _register("embedding", kind)


def register_head(kind: str):
    """What turns the final norm's rows into float32 logits."""
    return _register("head", kind)


def part_class(family: str, spec) -> type:
    kind = getattr(spec, "arrangement", None) if family == "block" else getattr(spec, "kind", None)
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise KeyError(f"no {family} part registered for kind {kind!r} (known: {known})") from None


def build_part(family: str, spec, env):
    return part_class(family, spec)(spec, env)


def registered(family: str):
    return sorted(_REGISTRIES[family])
