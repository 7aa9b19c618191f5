"""bfloat16 matrix products with float32 accumulation and float32 output."""
from __future__ import annotations

import torch

from .native import KernelError

torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, split_ok: bool = False) -> torch.Tensor:
    """x bfloat16 [M, K], w bfloat16 [N, K] -> float32 [M, N] (library product, as the
    reference uses cuBLASLt for its bfloat16 prompt products:
    crates/aegisllm-cuda/src/cuda/runtime/cublaslt.rs:57-165)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_bf16: expected bfloat16 operands, got {x.dtype} and {w.dtype}")
    if not x.is_cuda:
        raise KernelError("gemm_bf16: no CPU path exists")
    return torch.mm(x, w.t(), out_dtype=torch.float32)
