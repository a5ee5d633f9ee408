"""ctypes bindings of the low-precision kernels: FP8 quantisation (per tensor with amax for delayed
scaling, per row with dynamic scales), the FP8 tcgen05 GEMM path and the 8-bit blockwise AdamW."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _cuda as K

_FMT = {torch.float8_e4m3fn: K.E4M3, torch.float8_e5m2: K.E5M2}


def fp8_quantize(x: torch.Tensor, dtype=torch.float8_e4m3fn, scale: Optional[torch.Tensor] = None,
                 amax: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``fp8(x * scale)``; ``amax`` (1-element FP32 tensor) is raised to ``max|x|``."""
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    K._check(K.lib().nx_fp8_quantize(K._p(x), C.c_int(K._DT[x.dtype]), K._p(out), C.c_int(_FMT[dtype]),
                                     C.c_int64(x.numel()), K._p(scale), K._p(amax), K._stream()), "nx_fp8_quantize")
    return out


def fp8_quantize_rows(x: torch.Tensor, dtype=torch.float8_e4m3fn) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row dynamic quantisation of a 2-D tensor.  Returns (codes, scale_inv[rows])."""
    rows, cols = x.shape
    out = torch.empty((rows, cols), dtype=dtype, device=x.device)
    si = torch.empty(rows, dtype=torch.float32, device=x.device)
    K._check(K.lib().nx_fp8_quantize_rows(K._p(x), C.c_int(K._DT[x.dtype]), K._p(out), C.c_int(_FMT[dtype]),
                                          C.c_int(rows), C.c_int(cols), K._p(si), K._stream()), "nx_fp8_quantize_rows")
    return out, si


def fp8_dequantize(q: torch.Tensor, scale_inv: Optional[torch.Tensor] = None, dtype=torch.bfloat16) -> torch.Tensor:
    out = torch.empty(q.shape, dtype=dtype, device=q.device)
    K._check(K.lib().nx_fp8_dequantize(K._p(q), C.c_int(_FMT[q.dtype]), K._p(out), C.c_int(K._DT[dtype]),
                                       C.c_int64(q.numel()), K._p(scale_inv), K._stream()), "nx_fp8_dequantize")
    return out


def fp8_linear(x: torch.Tensor, w_q: torch.Tensor, w_scale_inv: torch.Tensor, bias=None, act=None,
               out_dtype=torch.bfloat16, amax_out=None) -> torch.Tensor:
    """y = act(x W^T + b) with x quantised per row on the fly (E4M3) and W held as FP8 codes with one
    scale per output row; the GEMM runs on the FP8 tensor-core path and dequantises in its epilogue."""
    xq, xs = fp8_quantize_rows(x)
    return K.gemm(xq, w_q, bias=bias, act=act, out_dtype=out_dtype, scale_a=xs, scale_b=w_scale_inv, amax_out=amax_out)


class AdamW8bitState:
    """Moment storage of the 8-bit AdamW for one flat parameter range."""

    def __init__(self, n: int, device):
        blk = int(K.lib().nx_adamw8_block())
        nb = (n + blk - 1) // blk
        self.n = n
        self.qm = torch.zeros(n, dtype=torch.uint8, device=device)
        self.qv = torch.zeros(n, dtype=torch.uint8, device=device)
        self.absmax_m = torch.zeros(nb, dtype=torch.float32, device=device)
        self.absmax_v = torch.zeros(nb, dtype=torch.float32, device=device)

    def nbytes(self) -> int:
        return 2 * self.n + 8 * self.absmax_m.numel()


def adamw8(master, shadow, grad, state: AdamW8bitState, opt_state, *, wd_scale=1.0, lr_scale=1.0, clip=None,
           zero_grad=False) -> None:
    K._check(K.lib().nx_adamw8(K._p(master), K._p(shadow), K._p(grad), K._p(state.qm), K._p(state.qv),
                               K._p(state.absmax_m), K._p(state.absmax_v), C.c_int64(state.n), K._p(opt_state),
                               C.c_float(wd_scale), C.c_float(lr_scale), K._p(clip), C.c_int(int(zero_grad)),
                               K._stream()), "nx_adamw8")


def grad_sq_accumulate(grad, accum) -> None:
    K._check(K.lib().nx_grad_sq_accumulate(K._p(grad), C.c_int64(grad.numel()), K._p(accum), K._stream()),
             "nx_grad_sq_accumulate")


def delayed_clip_finish(clip, accum, max_norm: float, norm_out=None) -> None:
    K._check(K.lib().nx_delayed_clip_finish(K._p(clip), K._p(norm_out), K._p(accum), C.c_double(max_norm), K._stream()),
             "nx_delayed_clip_finish")
