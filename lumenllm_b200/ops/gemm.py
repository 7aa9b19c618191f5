"""bfloat16 matrix products with float32 accumulation.

Two hand-written kernels do the work: the tcgen05 / TMA kernel (csrc/gemm_tc.cu) for every
shape, in its swapped orientation when there are few rows; and the register-streaming kernel
(csrc/gemm_small.cu) for up to 16 rows against weights of moderate height, where its k-split
over many small blocks and its fused SiLU prologue win. A product may come back as S partial
sums [S, M, N] for the consumer to add. The library product (cuBLAS through torch, as the
reference uses cuBLASLt: crates/aegisllm-cuda/src/cuda/runtime/cublaslt.rs:57-165) stands only
where a row of the operands is not a multiple of 16 bytes, which the TMA cannot address.
"""
from __future__ import annotations

import torch

from . import kernels as K
from .native import KernelError

torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False

SMALL_MAX_N = 8192      # tallest and widest weight the register-streaming kernel is preferred for
SMALL_MAX_K = 8192


def takes_small(M: int, Kdim: int, N: int) -> bool:
    return M <= K.SMALL_M and Kdim % 8 == 0 and N <= SMALL_MAX_N and Kdim <= SMALL_MAX_K


def takes_tc(x: torch.Tensor, w: torch.Tensor) -> bool:
    return x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, split_ok: bool = False, add_to=None):
    """x bfloat16 [M, K], w bfloat16 [N, K] -> float32 [M, N]; with split_ok possibly
    [S, M, N] partial sums that the consumer adds. With add_to (float32 [M, N]) the product
    may instead be added to it in place, where the kernel for this shape can do that; None
    is returned then, and the caller has nothing left to add."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_bf16: expected bfloat16 operands, got {x.dtype} and {w.dtype}")
    if not x.is_cuda:
        raise KernelError("gemm_bf16: no CPU path exists")
    if not x.is_contiguous():
        x = x.contiguous()
    if takes_small(x.shape[0], x.shape[1], w.shape[0]):
        part = K.gemm_small(x, w)
    elif takes_tc(x, w):
        if (add_to is not None and add_to.is_contiguous() and add_to.data_ptr() % 16 == 0
                and K.gemm_tc_adds(x.shape[0], w.shape[0])):
            return K.gemm_tc(x, w, add_to=add_to)
        part = K.gemm_tc(x, w)
    else:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    if part.shape[0] == 1:
        return part[0]
    return part if split_ok else part.sum(dim=0)


def gemm_gate_up_silu(x: torch.Tensor, w_interleaved: torch.Tensor):
    """silu(gate) * up in bfloat16 [M, I] from x [M, K] and a weight [2I, K] whose rows
    alternate gate_i, up_i, in ONE kernel when there are many rows; else None."""
    if x.shape[0] > 64 and takes_tc(x, w_interleaved):
        return K.gemm_tc(x if x.is_contiguous() else x.contiguous(), w_interleaved,
                         silu_interleaved=True)
    return None


def gemm_down_silu(gu: torch.Tensor, w: torch.Tensor, interleaved: bool):
    """(silu(gate) * up) @ w.T for gu float32 [M, 2K] (or [S, M, 2K] partials), M <= 16, with
    the activation applied while the rows are staged. Returns [S2, M, N] partials, or None if
    this shape is not taken (the caller then runs the two steps apart)."""
    M = gu.shape[-2]
    if w.dtype != torch.bfloat16 or not takes_small(M, w.shape[1], w.shape[0]):
        return None
    return K.gemm_small(gu, w, silu_gate_up=True, interleaved=interleaved)
