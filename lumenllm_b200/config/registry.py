"""One registry from an architecture's name to its configuration class.

A configuration class has `from_dict(dict)`, `to_dict()` and `model_spec()`.
Adding an architecture is one `register_architecture` call.
"""
from __future__ import annotations

import dataclasses
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


def eos_ids_of(value, where: str) -> tuple:
    """`eos_token_id` as config files write it: absent, one number or a list of numbers."""
    if value is None:
        return ()
    items = [value] if isinstance(value, int) and not isinstance(value, bool) else value
    if not isinstance(items, (list, tuple)) or any(isinstance(x, bool) or not isinstance(x, int)
                                                   for x in items):
        raise ConfigError(f"{where}: 'eos_token_id' must be a number or a list of numbers, "
                          f"got {value!r}")
    return tuple(int(x) for x in items)


def _read_json(path: Path) -> dict:
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d


def load_config(folder):
    """The typed configuration of a model folder. The end-of-sequence ids are the union of
    config.json's and generation_config.json's `eos_token_id` (a number or a list in either
    file: crates/aegisllm-base/src/text.rs:424-452; the second file is optional,
    crates/aegisllm-base/src/artifact.rs:496-523): chat checkpoints name the id that ends a
    turn only in the second file."""
    folder = Path(folder)
    path = folder / "config.json"
    if not path.exists():
        raise ConfigError(f"missing file: {path}")
    config = config_from_dict(_read_json(path))
    gen = folder / "generation_config.json"
    if gen.exists():
        more = eos_ids_of(_read_json(gen).get("eos_token_id"), gen.name)
        have = tuple(getattr(config, "eos_token_ids", ()))
        if set(more) - set(have):
            config = dataclasses.replace(config, eos_token_ids=tuple(sorted(set(have) | set(more))))
    return config
