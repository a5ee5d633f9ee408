"""Strided-batched linear on the tcgen05 GEMM with autograd: the grouped expert GEMM of the MoE
layer over capacity-padded [E, rows, d] buffers (one launch for all experts).
Parity: tests/cuda/test_phase14_moe_cuda.cpp:1-12 of the reference (padded strided-batched expert GEMMs)."""
from __future__ import annotations

import torch


class _BatchedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        from ..ops import _cuda as K
        ctx.save_for_backward(x, w)
        return K.gemm(x, w)  # [E, rows, in] x [E, out, in]^T -> [E, rows, out]

    @staticmethod
    def backward(ctx, dy):
        from ..ops import _cuda as K
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = K.gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = K.gemm(dy, x, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return dx, dw


def batched_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y[e] = x[e] @ w[e].T for x [E, rows, in], w [E, out, in]."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and w.dtype == x.dtype and \
            x.shape[-1] % 8 == 0 and w.shape[1] % 8 == 0 and x.shape[1] % 8 == 0:
        return _BatchedLinear.apply(x.contiguous(), w.contiguous())
    return torch.einsum("eri,eoi->ero", x, w.to(x.dtype))
