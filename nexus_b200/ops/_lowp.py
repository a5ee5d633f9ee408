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


# ------------------------------------------------------------------------------------------------
# Block-scaled FP8 (MX): FP8 codes plus one E8M0 scale (2^(byte-127)) per 32 elements along K
# ------------------------------------------------------------------------------------------------
class MxGemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("sfa", C.c_void_p), ("sfb", C.c_void_p), ("out", C.c_void_p),
        ("out_scales", C.c_void_p), ("bias", C.c_void_p), ("amax_out", C.c_void_p), ("status", C.c_void_p),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldo", C.c_int64),
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("a_dtype", C.c_int32), ("b_dtype", C.c_int32),
        ("out_dtype", C.c_int32), ("bias_dtype", C.c_int32), ("act", C.c_int32),
        ("alpha", C.c_float), ("max_ctas", C.c_int32),
    ]


def mx_scale_bytes(rows: int, cols: int) -> int:
    """Bytes of the scale atoms of a ``rows x cols`` block-scaled matrix (512 per 128 x 128 elements)."""
    return ((rows + 127) // 128) * ((cols + 127) // 128) * 512


def mx_scale_index(rows: int, cols: int, device="cpu") -> torch.Tensor:
    """``[rows, ceil(cols/32)]`` tensor of byte offsets into the scale atoms (the order the tensor core reads them
    in: atom of (row block of 128, column block of 128), inside it ``(r % 32) * 16 + ((r % 128) // 32) * 4 + j % 4``)."""
    kb128 = (cols + 127) // 128
    r = torch.arange(rows, device=device)[:, None]
    j = torch.arange((cols + 31) // 32, device=device)[None, :]
    return ((r // 128) * kb128 + j // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + j % 4


def mx_quantize_reference(x: torch.Tensor, dtype=torch.float8_e4m3fn, transpose: bool = False
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Plain-torch statement of :func:`mx_quantize` (any device): returns (codes, scale atoms as uint8)."""
    src = (x.t() if transpose else x).float()
    rows, cols = src.shape
    fmax = float(torch.finfo(dtype).max)
    nblk = (cols + 31) // 32
    pad = torch.zeros(rows, nblk * 32, dtype=torch.float32, device=x.device)
    pad[:, :cols] = src
    blocks = pad.view(rows, nblk, 32)
    amax = blocks.abs().amax(dim=2)
    v = (amax * torch.tensor(1.0 / fmax, dtype=torch.float32, device=x.device)).contiguous()
    bits = v.view(torch.int32)
    e = (bits >> 23) & 0xFF
    e = e + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    e = e.clamp(1, 253)
    e = torch.where(amax > 0, e, torch.full_like(e, 127))
    inv = ((254 - e) << 23).to(torch.int32).view(torch.float32)
    codes = (blocks * inv[:, :, None]).clamp(-fmax, fmax).to(dtype).view(rows, nblk * 32)[:, :cols].contiguous()
    scales = torch.full((mx_scale_bytes(rows, cols),), 127, dtype=torch.uint8, device=x.device)
    scales[mx_scale_index(rows, cols, x.device).reshape(-1)] = e.to(torch.uint8).reshape(-1)
    return codes, scales


def mx_dequantize_reference(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """FP32 values of a block-scaled matrix (any device)."""
    rows, cols = codes.shape
    e = scales[mx_scale_index(rows, cols, codes.device)].to(torch.int32)
    s = (e << 23).view(torch.float32)
    return codes.float() * s.repeat_interleave(32, dim=1)[:, :cols]


def mx_quantize(x: torch.Tensor, dtype=torch.float8_e4m3fn, transpose: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise a 2-D tensor to FP8 codes with E8M0 scales per 32 elements along the last axis of the result.
    ``transpose=True`` returns the codes of ``x.T`` (blocks along the rows of ``x``) without materialising ``x.T``."""
    if not x.is_cuda:
        return mx_quantize_reference(x, dtype, transpose)
    assert x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    r, k = (cols, rows) if transpose else (rows, cols)
    codes = torch.empty((r, k), dtype=dtype, device=x.device)
    scales = torch.empty(mx_scale_bytes(r, k), dtype=torch.uint8, device=x.device)
    K._check(K.lib().nx_mx_quantize(K._p(x), C.c_int(K._DT[x.dtype]), C.c_int64(x.stride(0)), C.c_int(rows), C.c_int(cols),
                                    K._p(codes), K._p(scales), C.c_int(_FMT[dtype]), C.c_int(int(transpose)), K._stream()),
             "nx_mx_quantize")
    return codes, scales


def mx_dequantize(codes: torch.Tensor, scales: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    if not codes.is_cuda:
        return mx_dequantize_reference(codes, scales).to(dtype)
    rows, cols = codes.shape
    out = torch.empty((rows, cols), dtype=dtype, device=codes.device)
    K._check(K.lib().nx_mx_dequantize(K._p(codes), K._p(scales), C.c_int(_FMT[codes.dtype]), C.c_int(rows), C.c_int(cols),
                                      K._p(out), C.c_int(K._DT[dtype]), K._stream()), "nx_mx_dequantize")
    return out


def mx_gemm(a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor, sfb: torch.Tensor, bias=None, act=None,
            out_dtype=torch.bfloat16, alpha: float = 1.0, amax_out=None, max_ctas: int = 0):
    """``act(alpha * A B^T + bias)`` of two block-scaled FP8 matrices (``a [M, K]``, ``b [N, K]``).  With an FP8
    ``out_dtype`` the result is itself block-scaled along N and ``(codes, scales)`` is returned: the K-major operand
    of a following :func:`mx_gemm`."""
    m, k = a.shape
    n = b.shape[0]
    assert b.shape[1] == k
    if not a.is_cuda:
        v = alpha * (mx_dequantize_reference(a, sfa) @ mx_dequantize_reference(b, sfb).t())
        if bias is not None:
            v = v + bias.float()
        if act == "gelu":
            v = torch.nn.functional.gelu(v, approximate="tanh")
        elif act == "relu":
            v = torch.relu(v)
        elif act == "silu":
            v = torch.nn.functional.silu(v)
        if amax_out is not None:
            amax_out.copy_(torch.maximum(amax_out, v.abs().max()))
        return mx_quantize_reference(v, out_dtype) if out_dtype in _FMT else v.to(out_dtype)
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    out_scales = torch.empty(mx_scale_bytes(m, n), dtype=torch.uint8, device=a.device) if out_dtype in _FMT else None
    g = MxGemmArgs()
    g.a, g.b, g.sfa, g.sfb = a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr()
    g.out = out.data_ptr()
    g.out_scales = 0 if out_scales is None else out_scales.data_ptr()
    g.bias = 0 if bias is None else bias.data_ptr()
    g.amax_out = 0 if amax_out is None else amax_out.data_ptr()
    g.status = K.status_word(a.device).data_ptr()
    g.lda, g.ldb, g.ldo = a.stride(0), b.stride(0), out.stride(0)
    g.m, g.n, g.k = m, n, k
    g.a_dtype, g.b_dtype = _FMT[a.dtype], _FMT[b.dtype]
    g.out_dtype = K._DT[out_dtype]
    g.bias_dtype = K._DT[bias.dtype] if bias is not None else K.F32
    g.act = K.ACT[act]
    g.alpha = alpha
    g.max_ctas = max_ctas
    K._check(K.lib().nx_gemm_mxf8(C.byref(g), K._stream()), "nx_gemm_mxf8")
    return (out, out_scales) if out_scales is not None else out


class _MxWeightCache:
    """Block-scaled forms of a weight (as stored, and transposed) keyed by the tensor and its version counter: between
    two optimizer steps the micro-batches of an accumulation step quantise each weight once per form.  Entries die
    with their tensor."""

    def __init__(self):
        self._store = {}
        self.hits = self.misses = 0
        # Off by default: an update made through ``w.data`` (or any alias with its own version counter) does not bump
        # ``w._version``.  Turn it on when weights change only through the tensor itself (torch.optim does) or when
        # the training loop calls ``invalidate()`` after each optimizer step (`fused.ops.adamw_multi_tensor` does).
        self.enabled = False

    def invalidate(self) -> None:
        self._store.clear()

    def get(self, w: torch.Tensor, transpose: bool):
        import weakref
        if not self.enabled:
            return mx_quantize(w.detach(), transpose=transpose)
        key = (id(w), transpose)
        ent = self._store.get(key)
        if ent is not None and ent[0]() is w and ent[1] == w._version and ent[2] == w.data_ptr():
            self.hits += 1
            return ent[3]
        self.misses += 1
        val = mx_quantize(w.detach(), transpose=transpose)
        try:
            ref = weakref.ref(w, lambda _r, k=key: self._store.pop(k, None))
        except TypeError:
            return val
        self._store[key] = (ref, w._version, w.data_ptr(), val)
        return val


mx_weight_cache = _MxWeightCache()


class _MxLinearFn(torch.autograd.Function):
    """y = x W^T (+ b) with all three GEMMs of the layer on the block-scaled FP8 path: forward and input gradient use
    E4M3 activations / weights (E5M2 for dy), the weight gradient contracts over the tokens, so dy and x are
    re-quantised with their blocks along the token axis."""

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        xq, xs = mx_quantize(x2)
        wq, ws = mx_weight_cache.get(w, False)
        y = mx_gemm(xq, xs, wq, ws, bias=bias, out_dtype=x.dtype if x.dtype != torch.float32 else torch.float32)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.shape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        gq, gs = mx_quantize(dy2, torch.float8_e5m2)                    # [M, N], blocks along N
        wtq, wts = mx_weight_cache.get(w, True)                         # [K, N], blocks along N
        dx = mx_gemm(gq, gs, wtq, wts, out_dtype=x2.dtype)              # [M, K]
        gtq, gts = mx_quantize(dy2, torch.float8_e5m2, transpose=True)  # [N, M], blocks along M
        xtq, xts = mx_quantize(x2, transpose=True)                      # [K, M], blocks along M
        dw = mx_gemm(gtq, gts, xtq, xts, out_dtype=torch.float32).to(w.dtype)  # [N, K]
        db = dy2.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx.reshape(ctx.shape), dw, db


def mx_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable linear layer whose forward, input-gradient and weight-gradient GEMMs all run block-scaled FP8."""
    return _MxLinearFn.apply(x, w, bias)
