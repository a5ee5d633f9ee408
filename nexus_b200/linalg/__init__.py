"""`linalg`: matrix products and reductions; CUDA BF16/FP16 operands use the tcgen05 GEMM."""
from __future__ import annotations

import torch


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a [M, K] @ b [K, N]."""
    if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16) and a.dtype == b.dtype and a.dim() == 2 and \
            b.dim() == 2 and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and a.is_contiguous() and b.is_contiguous():
        from ..ops import _cuda as K
        return K.gemm(a, b, b_mn=True)
    return a @ b


def gemm(a, b, alpha: float = 1.0, beta: float = 0.0, c=None, trans_a=False, trans_b=False):
    """alpha * op(a) @ op(b) + beta * c."""
    x = a.t() if trans_a else a
    y = b.t() if trans_b else b
    out = matmul(x.contiguous(), y.contiguous()) * alpha
    return out if c is None or beta == 0.0 else out + beta * c


def dot(a, b): return (a.reshape(-1).float() * b.reshape(-1).float()).sum()
def norm(a): return a.float().norm()
def transpose(a): return a.t().contiguous()
