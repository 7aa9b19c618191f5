"""Position encodings that a mixer applies to its queries and keys.

"rotary": half-split pairs (i, i + rot/2) rotated by angle = pos * inv_freq_i with
inv_freq_i = 1 / theta^(2i/rot), computed in float32
(norm_rope_kv.cu:437-447,465-492; crates/aegisllm-cpu/src/cpu/rope.rs:34-84).
`rotary_dim` < head_dim rotates only the first dims. A position part offers `rotary_dim` and `angles(ctx)`, the (cos, sin) of every
token of the step as float32 [N, rotary_dim/2, 2]; an encoding with other
frequencies or other positions is another way to fill that table; "none"
rotates nothing.
"""
from __future__ import annotations

import torch

from .base import need, register_part


@register_part("position", "rotary")
class Rotary:
    @classmethod
    def tensors(cls, spec):
        return {}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.head_dim = int(need(p, "head_dim", "rotary"))
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        self.theta = float(need(p, "theta", "rotary"))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim")
        self.inv_freq = self.frequencies().to(runtime.device).contiguous()

    def angles(self, ctx):
        """(cos, sin) for every token of the step, float32 [N, rot/2, 2]; made once per step
        and shared by all layers whose encoding has the same frequencies."""
        shared = ctx.extras.setdefault("per_step", {})   # emptied when the step's forward begins
        key = ("rope", self.rotary_dim, self.theta)
        cs = shared.get(key)
        if cs is None:
            from ..ops import kernels as K
            cs = shared[key] = K.rope_table(ctx.rope_pos, self.inv_freq)
        return cs

    def frequencies(self) -> torch.Tensor:
        i2 = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        return 1.0 / (torch.tensor(self.theta, dtype=torch.float32) ** (i2 / self.rotary_dim))


@register_part("position", "none")
class NoPosition:
    @classmethod
    def tensors(cls, spec):
        return {}

    def __init__(self, spec, weights, runtime):
        self.rotary_dim = 0
        self.inv_freq = None

    def angles(self, ctx):
        return None
