"""bfloat16 matrix products with float32 accumulation.

The tcgen05 / TMA kernels (csrc/gemm_tc.cu) do the work for every shape: two SMs a tile for
prompts, a weight-streaming orientation with k split for decode and short prompts. A product
may come back as S partial sums [S, M, N] for the consumer to add, or be added to the residual
stream in place. The library product (cuBLAS through torch, as the reference uses cuBLASLt:
crates/aegisllm-cuda/src/cuda/runtime/cublaslt.rs:57-165) stands only where a row of the
operands is not a multiple of 16 bytes, which the TMA cannot address. Weights reach the
tensor-core kernels in tiled form (kernels.tile_weight), made once when the model is built.
"""
from __future__ import annotations

import torch

from . import kernels as K
from .native import KernelError

torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False


def takes_tc(x: torch.Tensor, w) -> bool:
    """A weight in tiled form goes to the tensor-core kernels (it exists only where its rows are
    multiples of 16 bytes); a plain tensor is a weight they cannot address."""
    return isinstance(w, K.TiledWeight) and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, split_ok: bool = False, add_to=None):
    """x bfloat16 [M, K], w bfloat16 [N, K] (tiled, or a plain tensor) -> float32 [M, N]; with split_ok possibly
    [S, M, N] partial sums that the consumer adds. With add_to (float32 [M, N]) the product
    may instead be added to it in place, where the kernel for this shape can do that; None
    is returned then, and the caller has nothing left to add."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_bf16: expected bfloat16 operands, got {x.dtype} and {w.dtype}")
    if not x.is_cuda:
        raise KernelError("gemm_bf16: no CPU path exists")
    if not x.is_contiguous():
        x = x.contiguous()
    if takes_tc(x, w):
        if (add_to is not None and add_to.is_contiguous() and add_to.data_ptr() % 16 == 0
                and K.gemm_tc_adds(x.shape[0], w.shape[0])):
            return K.gemm_tc(x, w, add_to=add_to)
        part = K.gemm_tc(x, w)
    else:
        if isinstance(w, K.TiledWeight):
            raise KernelError(f"gemm_bf16: activations [{x.shape[0]}, {x.shape[1]}] do not fit a tiled weight "
                              f"{w.shape} (rows of 16 bytes, 16-byte aligned)")
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    if part.shape[0] == 1:
        return part[0]
    return part if split_ok else part.sum(dim=0)


def gemm_gate_up_silu(x: torch.Tensor, w_interleaved):
    """silu(gate) * up in bfloat16 [M, I] from x [M, K] and a weight [2I, K] whose rows
    alternate gate_i, up_i, in ONE kernel where that is the faster way; else None, and the
    caller takes the float32 product with the activation kernel behind it. One kernel: from 512
    rows on, and for rows that fill the two-SM kernel's 256-row tiles. Below: up to 128 rows
    the product streams the weights with k split, which the epilogue cannot have (at 100 rows of
    the 8B shape 41 + 6 us against 56 us); from 129 to 511 rows the two-SM kernel works on tiles
    that are part empty, and the split product is the faster again (first token of a prompt of
    160 / 192 / 288 / 384 / 480 tokens at the 8B shape: 4.9 / 5.1 / 7.0 / 7.3 / 8.0 ms against
    5.6 / 5.7 / 7.6 / 7.7 / 8.4; of 256 tokens 5.3 in one kernel against 5.5)."""
    rows = x.shape[0]
    if (rows >= 512 or (rows > 128 and rows % 256 == 0)) and takes_tc(x, w_interleaved):
        return K.gemm_tc(x if x.is_contiguous() else x.contiguous(), w_interleaved,
                         silu_interleaved=True)
    return None
