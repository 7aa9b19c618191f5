"""bfloat16 matrix products with float32 accumulation and float32 output.

Up to 16 rows (decode) go to the hand-written weight-streaming kernel, which returns S
partial results for its consumer to add; more rows go to the library product, as the
reference uses cuBLASLt for its bfloat16 prompt products
(crates/aegisllm-cuda/src/cuda/runtime/cublaslt.rs:57-165).
"""
from __future__ import annotations

import torch

from . import kernels as K
from .native import KernelError

torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False


def takes_small(M: int, Kdim: int, N: int = 0) -> bool:
    """Few rows, and a weight small enough that its row blocks alone do not fill the GPU
    (there the k-split of the streaming kernel pays; very tall weights stream as well
    through the library product)."""
    return M <= K.SMALL_M and Kdim % 8 == 0 and N <= 16384


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, split_ok: bool = False) -> torch.Tensor:
    """x bfloat16 [M, K], w bfloat16 [N, K] -> float32 [M, N]; with split_ok possibly
    [S, M, N] partial sums that the consumer adds."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_bf16: expected bfloat16 operands, got {x.dtype} and {w.dtype}")
    if not x.is_cuda:
        raise KernelError("gemm_bf16: no CPU path exists")
    if takes_small(x.shape[0], x.shape[1], w.shape[0]):
        part = K.gemm_small(x, w)
        if part.shape[0] == 1:
            return part[0]
        return part if split_ok else part.sum(dim=0)
    return torch.mm(x, w.t(), out_dtype=torch.float32)


def gemm_bf16_silu_gate_up(gu: torch.Tensor, w: torch.Tensor):
    """(silu(gate) * up) @ w.T for gu float32 [M, 2K] (or [S, M, 2K] partials), M <= 16, with
    the activation applied while the rows are staged. Returns [S2, M, N] partials, or None if
    this shape is not taken (the caller then runs the two steps apart)."""
    M = gu.shape[-2]
    if w.dtype != torch.bfloat16 or not takes_small(M, w.shape[1], w.shape[0]):
        return None
    return K.gemm_small(gu, w, silu_gate_up=True)
