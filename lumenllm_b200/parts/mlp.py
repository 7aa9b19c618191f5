"""Feed-forward parts.

"swiglu": g = y Wg^T, u = y Wu^T, z = g / (1 + exp(-g)) * u, out = z Wd^T
(crates/aegisllm-cuda/src/executor/mlp.rs:271-356; norm_rope_kv.cu:314-325).
Gate and up weights are stacked so that both cost one product. For bfloat16 their rows
are interleaved (gate_0, up_0, gate_1, up_1, ...): then a tile of the product holds both
halves of each pair, and the tensor-core kernel applies SiLU(gate) * up in its epilogue
and writes bfloat16 directly. With few rows the product returns float32 (partial sums)
and a small kernel adds them and applies the activation.
"""
from __future__ import annotations

import torch

from ..ops import gemm as G
from ..ops import kernels as K
from .base import need, register_part
from .linear import Linear


@register_part("ffn", "swiglu")
class SwiGLU:
    graph_safe = True

    @classmethod
    def tensors(cls, spec):
        H = int(need(spec.params, "hidden_size", "swiglu"))
        I = int(need(spec.params, "intermediate_size", "swiglu"))
        return {f"{spec.prefix}.gate_proj.weight": ((I, H), "matrix"),
                f"{spec.prefix}.up_proj.weight": ((I, H), "matrix"),
                f"{spec.prefix}.down_proj.weight": ((H, I), "matrix")}

    def __init__(self, spec, weights, runtime):
        self.runtime = runtime
        pre = spec.prefix
        g, u = weights[f"{pre}.gate_proj.weight"], weights[f"{pre}.up_proj.weight"]
        self.down = Linear(weights[f"{pre}.down_proj.weight"], runtime)
        self.interleaved = (not runtime.is_f32 and g.dtype == torch.bfloat16
                            and u.dtype == torch.bfloat16)
        if self.interleaved:
            I, H = g.shape
            self.gate_up = Linear(torch.stack([g, u], dim=1).reshape(2 * I, H), runtime)
        else:
            self.gate_up = Linear.stacked([g, u], runtime)

    adds_residual = True      # forward takes `residual` and may add its update to it in place

    def forward(self, y, ctx, residual=None):
        if self.interleaved and not self.down.f32:
            z = G.gemm_gate_up_silu(y, self.gate_up.weight)         # many rows: one kernel
            if z is not None:
                return self.down(z, split_ok=True, add_to=residual)
        gu = self.gate_up(y, split_ok=True)        # float32 [N, 2I], possibly S partials
        z = K.silu_mul(gu, self.runtime.dtype, interleaved=self.interleaved)
        return self.down(z, split_ok=True)
