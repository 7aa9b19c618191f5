"""The parts a model is put together from, their registry and their interfaces.

Categories and what each must offer (all take `(spec: PartSpec, weights, runtime)`
in the constructor and declare their tensors with a classmethod
`tensors(spec) -> {name: (shape, "matrix" | "norm")}`):

  embedding  forward(tokens int32 [N]) -> residual stream float32 [N, H]
  norm       forward(h, delta, out_dtype, rows=None, write_h=True) -> y
             (h float32 [N, H] is the residual stream; `delta`, float32 [S, N, H]
             or None, is added to it first, in float32; y is the normed rows)
  position   a table or rule that a mixer applies to its queries and keys
  mixer      cache_need() -> CacheNeed | None; state_shape() -> (shape, dtype) | None;
             forward(y, ctx, entry) -> delta float32 [S, N, H]
             (y: normed rows in the run dtype; ctx: StepContext; entry: EntryView,
             which hands out this run's cache pages and per-sequence state)
  ffn        forward(y, ctx) -> delta float32 [S, N, H]
  block      forward(h, pending, ctx, entry) -> (h, pending): how mixer, ffn and
             norms are arranged around the residual stream
  head       forward(y) -> logits float32 [W, V]

A delta is a list of S partial sums of one update of the residual stream; the
norm that follows adds them in a fixed order, which keeps split-K products
deterministic and saves a pass over the stream.

No part knows which model it is in: sizes and constants come from spec.params,
tensors from `weights[spec.prefix + ...]`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple

import torch

from ..config.spec import ConfigError, PartSpec

_REGISTRY: Dict[Tuple[str, str], type] = {}
CATEGORIES = ("embedding", "norm", "position", "mixer", "ffn", "block", "head")


def register_part(category: str, kind: str) -> Callable[[type], type]:
    if category not in CATEGORIES:
        raise ConfigError(f"unknown part category '{category}' (known: {CATEGORIES})")

    def deco(cls):
        _REGISTRY[(category, kind)] = cls
        return cls
    return deco


def part_class(category: str, kind: str) -> type:
    try:
        return _REGISTRY[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise ConfigError(f"no {category} part named '{kind}' is registered (known: {known})") from None


def build_part(category: str, spec: PartSpec, weights, runtime):
    return part_class(category, spec.kind)(spec, weights, runtime)


def part_tensors(category: str, spec: PartSpec):
    return part_class(category, spec.kind).tensors(spec)


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision a model runs. `dtype` is the type of the
    activations handed to matrix products and of the cache: torch.bfloat16 (the
    serving kernels) or torch.float32 (everything in true 32-bit)."""
    device: torch.device
    dtype: torch.dtype

    @property
    def is_f32(self) -> bool:
        return self.dtype == torch.float32


def need(params: dict, key: str, what: str):
    if key not in params:
        raise ConfigError(f"{what}: parameter '{key}' is missing")
    return params[key]
