"""Sampling options and the uniform numbers the device sampler draws with.

Options and their defaults are the reference's `SamplingConfig`
(crates/aegisllm-base/src/generation.rs:83-92,166-175); the order temperature ->
top-k -> top-p -> min-p -> draw is that of
crates/aegisllm-base/src/executor/generation.rs:193-273, and as there
(crates/aegisllm-cuda/src/executor/forward.rs:519-544) the host supplies the
uniform number and the device does the rest. The reference draws it unseeded;
here it comes from a counter-based generator keyed by (seed, stream, step); the
generation loop keys it by the request's own seed and step count only, so a
request samples the same tokens alone and in any batch.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

_M64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingConfig:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    seed: Optional[int] = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        if not (self.top_p == self.top_p and self.min_p == self.min_p
                and self.temperature == self.temperature):
            raise ValueError("sampling options must be numbers")


def _mix(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform(seed: int, stream: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits, a pure function of its three keys."""
    x = _mix(seed & _M64)
    x = _mix(x ^ ((stream & _M64) * 0xD1342543DE82EF95 & _M64))
    x = _mix(x ^ ((step & _M64) * 0xA0761D6478BD642F & _M64))
    return (x >> 40) / float(1 << 24)


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")


class DeviceSampler:
    """Picks one token per row of float32 logits on the device."""

    def __init__(self, device):
        self.device = device

    def pick(self, logits: torch.Tensor, configs: Sequence[SamplingConfig],
             us: Sequence[float]) -> torch.Tensor:
        from ..ops import kernels as K
        B = logits.shape[0]
        if len(configs) != B or len(us) != B:
            raise ValueError("one sampling config and one uniform number per row")
        if all(c.greedy for c in configs):
            return K.argmax(logits)
        opts = torch.tensor([[c.temperature, c.top_p, c.min_p, u] for c, u in zip(configs, us)],
                            dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        top_k = torch.tensor([c.top_k for c in configs], dtype=torch.int32) \
            .pin_memory().to(self.device, non_blocking=True)
        return K.sample(logits, opts, top_k)
