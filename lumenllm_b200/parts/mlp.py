"""Feed-forward parts.

"swiglu": g = y Wg^T, u = y Wu^T, z = g / (1 + exp(-g)) * u, out = z Wd^T
(crates/aegisllm-cuda/src/executor/mlp.rs:271-356; norm_rope_kv.cu:314-325).
Gate and up weights are stacked so that both cost one product.
"""
from __future__ import annotations

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
        self.gate_up = Linear.stacked([weights[f"{pre}.gate_proj.weight"],
                                       weights[f"{pre}.up_proj.weight"]], runtime)
        self.down = Linear(weights[f"{pre}.down_proj.weight"], runtime)

    def forward(self, y, ctx):
        gu = self.gate_up(y, split_ok=True)        # float32 [N, 2I], possibly S partials
        if not self.down.f32:
            out = G.gemm_bf16_silu_gate_up(gu, self.down.weight)   # few rows: one kernel
            if out is not None:
                return out
        z = K.silu_mul(gu, self.runtime.dtype)
        return self.down(z, split_ok=True)
