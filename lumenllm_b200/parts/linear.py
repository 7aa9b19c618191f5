"""y = x W^T for a weight stored [out, in] (crates/aegisllm-cuda/src/cuda/kernels/
blackwell/sampling.cu:16-18). The result is float32.

A weight kept in float32 (stored so, or a 32-bit run) is multiplied by the FFMA
kernel in true 32-bit; a bfloat16 weight in a bfloat16 run goes to the tensor
cores with float32 accumulation. Several weights that read the same input are
stacked row-wise at load so that they cost one product.
"""
from __future__ import annotations

import weakref

import torch

from ..ops import kernels as K
from ..ops import gemm as G

# Tiled forms already made, by the tensor they were made from: an embedding table that the
# output head shares is tiled once and held once.
_tiled = {}


def tiled_form(weight: torch.Tensor) -> "K.TiledWeight":
    """The tiled form of a bfloat16 matrix on the device, the same object for the same tensor
    as long as that tensor lives."""
    key = id(weight)
    hit = _tiled.get(key)
    if hit is not None and hit[0]() is weight:
        return hit[1]
    tiled = K.tile_weight(weight)
    _tiled[key] = (weakref.ref(weight, lambda _, key=key: _tiled.pop(key, None)), tiled)
    return tiled


class Linear:
    """`weight` is the matrix as the product reads it: a float32 or bfloat16 tensor [out, in]
    for the 32-bit kernel (and for the library product, where an input row is no multiple of
    16 bytes), else the tiled form the tensor-core kernels stream (ops.kernels.TiledWeight)."""

    def __init__(self, weight, runtime):
        if isinstance(weight, K.TiledWeight):
            self.runtime, self.weight, self.f32 = runtime, weight, False
            self.out_features, self.in_features = weight.shape
            return
        if weight.dim() != 2:
            raise ValueError("a linear weight has two dimensions")
        self.runtime = runtime
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        self.f32 = runtime.is_f32 or weight.dtype == torch.float32
        if not self.f32 and K.can_tile(self.weight):
            self.weight = tiled_form(self.weight)

    @classmethod
    def stacked(cls, weights, runtime) -> "Linear":
        dt = torch.float32 if any(w.dtype == torch.float32 for w in weights) else weights[0].dtype
        return cls(torch.cat([w.to(dt) for w in weights], dim=0), runtime)

    def first_rows(self, n: int) -> "Linear":
        """The product with the first n rows of the weight only, on the same memory."""
        w = self.weight
        return Linear(w.first_rows(n) if isinstance(w, K.TiledWeight) else w[:n], self.runtime)

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
