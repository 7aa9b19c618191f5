"""y = x W^T for a weight stored [out, in] (crates/aegisllm-cuda/src/cuda/kernels/
blackwell/sampling.cu:16-18). The result is float32.

A weight kept in float32 (stored so, or a 32-bit run) is multiplied by the FFMA
kernel in true 32-bit; a bfloat16 weight in a bfloat16 run goes to the tensor
cores with float32 accumulation. Several weights that read the same input are
stacked row-wise at load so that they cost one product.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from ..ops import gemm as G


class Linear:
    def __init__(self, weight: torch.Tensor, runtime):
        if weight.dim() != 2:
            raise ValueError("a linear weight has two dimensions")
        self.runtime = runtime
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.f32 = runtime.is_f32 or weight.dtype == torch.float32

    @classmethod
    def stacked(cls, weights, runtime) -> "Linear":
        dt = torch.float32 if any(w.dtype == torch.float32 for w in weights) else weights[0].dtype
        return cls(torch.cat([w.to(dt) for w in weights], dim=0), runtime)

    def __call__(self, x: torch.Tensor, split_ok: bool = False, add_to=None):
        """x [M, in] in the run dtype -> float32 [M, out]; with split_ok the result may
        come as [S, M, out] partial sums for the next norm to add. With add_to (the float32
        residual stream [M, out]) the product may be added to it in place instead (prompt-sized
        products on the tensor cores do that in their epilogue); the result is None then."""
        if self.f32:
            if x.dtype != torch.float32:
                x = x.float()
            return K.gemm_f32(x, self.weight)
        return G.gemm_bf16(x, self.weight, split_ok=split_ok, add_to=add_to)
