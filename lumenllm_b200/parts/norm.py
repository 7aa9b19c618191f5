"""RMSNorm, with the residual add that precedes it fused in.

y_i = x_i * 1/sqrt(mean(x^2) + eps) * w_i, everything in float32
(crates/aegisllm-cuda/src/cuda/kernels/blackwell/norm_rope_kv.cu:36-62;
crates/aegisllm-cpu/src/cpu/math.rs:4-8). `weight_offset` 1 gives the (1 + w)
form that the reference folds in for other families (executor/loader.rs:189-194);
it is a parameter, 0 for Qwen3 dense.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .base import need, register_part


@register_part("norm", "rmsnorm")
class RMSNorm:
    @classmethod
    def tensors(cls, spec):
        return {f"{spec.prefix}.weight": ((need(spec.params, "size", "rmsnorm"),), "norm")}

    def __init__(self, spec, weights, runtime):
        p = spec.params
        self.size = int(need(p, "size", "rmsnorm"))
        self.eps = float(need(p, "eps", "rmsnorm"))
        w = weights[f"{spec.prefix}.weight"].to(device=runtime.device, dtype=torch.float32)
        off = float(p.get("weight_offset", 0.0))
        self.weight = (w + off).contiguous() if off else w.contiguous()

    def forward(self, h, delta, out_dtype, rows=None, write_h=True):
        return K.add_rmsnorm(h, delta, self.weight, self.eps, out_dtype, rows=rows, write_h=write_h)
