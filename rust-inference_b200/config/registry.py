"""One registry from an architecture's name to its configuration class.

A configuration class is built from the keys of ``config.json`` by
``from_dict``, checks itself in ``validate`` and describes the model as parts
in ``to_spec`` (a :class:`~.specs.ModelSpec`).  ``to_dict`` gives back the
``config.json`` keys, which is what the random-weights mode writes.

The architecture is chosen as thanhauco/rust-inference does it
(src/models/config.rs:136-145): the first entry of ``architectures``, else
``model_type``.
"""
from __future__ import annotations

import json
import os
from typing import Dict


class ConfigError(ValueError):
    """A config.json that is malformed or asks for something the model cannot do."""


class UnsupportedArchitecture(ConfigError):
    pass


_BY_NAME: Dict[str, type] = {}


def register_architecture(*names: str):
    """Class decorator: ``@register_architecture("Qwen3ForCausalLM", "qwen3")``."""
    def deco(cls):
        for n in names:
            _BY_NAME[n] = cls
        cls.architecture_names = tuple(names)
        return cls
    return deco


def registered_architectures():
    return sorted(_BY_NAME)


def architecture_of(d: dict) -> str:
    archs = d.get("architectures") or []
    name = archs[0] if archs else d.get("model_type")
    if not name:
        raise UnsupportedArchitecture("config.json names no architecture (architectures / model_type)")
    return name


def config_from_dict(d: dict):
    name = architecture_of(d)
    cls = _BY_NAME.get(name)
    if cls is None:
        # the reference matches by substring (config.rs:140-145)
        for key, c in _BY_NAME.items():
            if key in name:
                cls = c
                break
    if cls is None:
        raise UnsupportedArchitecture(
            f"architecture {name!r} is not registered (known: {', '.join(registered_architectures())})")
    cfg = cls.from_dict(d)
    cfg.validate()
    return cfg


def load_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path) as f:
            d = json.load(f)
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return config_from_dict(d)
