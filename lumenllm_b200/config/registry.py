"""One registry from an architecture's name to its configuration class.

A configuration class has `from_dict(dict)`, `to_dict()` and `model_spec()`.
Adding an architecture is one `register_architecture` call.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict

from .spec import ConfigError

_BY_ARCH: Dict[str, type] = {}
_BY_MODEL_TYPE: Dict[str, type] = {}


def register_architecture(name: str, model_type: str | None = None):
    def deco(cls):
        _BY_ARCH[name] = cls
        if model_type:
            _BY_MODEL_TYPE[model_type] = cls
        return cls
    return deco


def known_architectures():
    return sorted(_BY_ARCH)


def config_class_for(d: dict):
    """`architectures[]` first, then `model_type`
    (crates/aegisllm-base/src/model/mod.rs:136-153, with exact names instead of
    substring matching)."""
    archs = d.get("architectures") or []
    for a in archs:
        if a in _BY_ARCH:
            return _BY_ARCH[a]
    mt = d.get("model_type")
    if mt in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[mt]
    raise ConfigError(f"unknown architecture: architectures={archs!r} model_type={mt!r}; "
                      f"known: {known_architectures()}")


def config_from_dict(d: dict):
    if not isinstance(d, dict):
        raise ConfigError("config.json must hold a JSON object")
    return config_class_for(d).from_dict(d)


def load_config(folder):
    path = Path(folder) / "config.json"
    if not path.exists():
        raise ConfigError(f"missing file: {path}")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    return config_from_dict(d)
