"""What a model is made of, as data.

A configuration class (one per architecture) turns the keys of config.json into
a ModelSpec: the parts of every layer with their sizes and constants, and the
order in which layers run. Nothing below this level knows which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """config.json (or a parameters file) is missing a key, has a wrong value, or
    asks for something this library does not compute."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: `kind` names the implementation in the parts registry,
    `params` are its sizes and constants, `prefix` is where its tensors live."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """A block: how a mixer and a feed-forward are arranged around the residual
    stream (`block`, e.g. "pre_norm"), and the parts themselves. Each layer has
    its own, so one model can mix kinds."""
    block: str
    mixer: PartSpec
    ffn: PartSpec
    norms: Dict[str, PartSpec]
    prefix: str = ""


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. `layer` indexes ModelSpec.layers (a layer may be named
    by several entries: its weights are shared, each run has a cache of its own).
    `cache_from` names an EARLIER entry whose keys and values this run reads
    instead of writing its own."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, "
                                  f"but there are {len(self.layers)} layers")
            if e.cache_from is not None and not 0 <= e.cache_from < i:
                raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_from}, "
                                  "which does not run before it")
            if e.cache_from is not None and self.schedule[e.cache_from].cache_from is not None:
                raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_from}, "
                                  "which has no cache of its own")
