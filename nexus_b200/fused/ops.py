"""Fused training operators with autograd: one node each for forward + backward.

On CUDA tensors (BF16/FP16 activations) every operator runs the hand-written sm_100a kernels of
``lib/libnexus_b200_cuda.so`` (tcgen05 GEMM with fused bias/activation epilogues, flash attention,
fused norms, in-place shifted cross-entropy, Philox dropout).  On CPU tensors, and for FP32 CUDA
tensors, the same math runs as plain PyTorch; that path is also the oracle the GPU tests compare
against.

Parity: include/nexus/fused/fused.hpp:35-53 (fused_linear / fused_layernorm /
fused_residual_layernorm / fused_softmax) and include/nexus/fused/training.hpp:42-117
(cross_entropy_shifted, rms_norm, embedding_pos, dropout_philox, adamw_multi_tensor) of the reference.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from . import philox as _philox

_ACTS = ("identity", "relu", "gelu", "silu")


def _use_kernels(*ts: torch.Tensor) -> bool:
    t = ts[0]
    if not t.is_cuda or t.dtype not in (torch.bfloat16, torch.float16):
        return False
    from ..ops import _cuda as K
    K.lib()  # raises loudly when the library is missing on a GPU machine
    return True


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return F.gelu(x, approximate="tanh")


def _act_fwd(x: torch.Tensor, act: str) -> torch.Tensor:
    if act == "identity":
        return x
    if act == "relu":
        return torch.relu(x)
    if act == "gelu":
        return gelu_tanh(x)
    if act == "silu":
        return F.silu(x)
    raise ValueError(f"unknown activation {act}")


# ------------------------------------------------------------------------------------------- linear
class _FusedLinear(torch.autograd.Function):
    """y = act(x @ W^T + b), W stored [out, in]."""

    @staticmethod
    def forward(ctx, x, w, b, act):
        from ..ops import _cuda as K
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        aux = None
        if act == "gelu":
            aux = torch.empty((x2.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
            y = K.gemm(x2, w, bias=b, act="gelu", aux_out=aux)
        elif act in ("relu", "silu"):
            aux = K.gemm(x2, w, bias=b)
            y = _act_fwd(aux, act)
        else:
            y = K.gemm(x2, w, bias=b)
        ctx.save_for_backward(x2, w, aux if aux is not None else torch.empty(0, device=x.device))
        ctx.act, ctx.has_bias, ctx.x_shape = act, b is not None, x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from ..ops import _cuda as K
        x2, w, aux = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.act == "gelu":
            pre = aux.float().requires_grad_(True)
            with torch.enable_grad():
                gelu_tanh(pre).backward(dy2.float())
            dpre = pre.grad.to(dy2.dtype)
        elif ctx.act in ("relu", "silu"):
            pre = aux.float().requires_grad_(True)
            with torch.enable_grad():
                _act_fwd(pre, ctx.act).backward(dy2.float())
            dpre = pre.grad.to(dy2.dtype)
        else:
            dpre = dy2
        dx = K.gemm(dpre, w, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            rows = x2.shape[0]
            if rows % 8 == 0:
                dw = K.gemm(dpre, x2, a_mn=True, b_mn=True, out_dtype=torch.float32,
                            split_k=max(1, min(8, rows // 2048))).to(w.dtype)
            else:
                dw = (dpre.float().t() @ x2.float()).to(w.dtype)
        db = K.colsum(dpre).to(w.dtype) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None


_LINEAR_PRECISION = ["native"]


class linear_precision:
    """Context manager: ``with linear_precision("mxfp8"):`` runs every :func:`fused_linear` inside it (forward,
    input gradient and weight gradient) on the block-scaled FP8 tensor-core path - FP8 codes with one power-of-two
    scale per 32 elements along the contraction axis, E4M3 for activations and weights, E5M2 for gradients.
    Layers whose sizes the path does not take (K or N not a multiple of 16) keep their native precision."""

    def __init__(self, kind: str = "mxfp8"):
        if kind not in ("native", "mxfp8"):
            raise ValueError("linear_precision: kind must be 'native' or 'mxfp8'")
        self.kind = kind

    def __enter__(self):
        _LINEAR_PRECISION.append(self.kind)
        return self

    def __exit__(self, *exc):
        _LINEAR_PRECISION.pop()
        return False


def fused_linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, act: str = "identity"):
    """``act(x @ w.T + b)`` with ``w`` [out, in]; one autograd node."""
    if act not in _ACTS:
        raise ValueError(f"fused_linear: activation must be one of {_ACTS}")
    if _LINEAR_PRECISION[-1] == "mxfp8" and x.shape[-1] % 16 == 0 and w.shape[0] % 16 == 0 and w.is_contiguous():
        from ..ops import _lowp as L
        return _act_fwd(L.mx_linear(x, w, b), act)
    k_ok = x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0
    if _use_kernels(x) and w.dtype == x.dtype and k_ok and w.is_contiguous():
        return _FusedLinear.apply(x, w, b, act)
    return _act_fwd(F.linear(x, w, b), act)


# ------------------------------------------------------------------------------- gated activations
class _GatedActivation(torch.autograd.Function):
    """y = act(h[:, :F]) * h[:, F:] for h = [gate | up] (SwiGLU / GeGLU): one kernel forward, one backward."""

    @staticmethod
    def forward(ctx, h, kind):
        from ..ops import _infer as I
        h2 = h.reshape(-1, h.shape[-1])
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        ctx.save_for_backward(h2)
        ctx.kind, ctx.shape = kind, h.shape
        return I.gated_fwd(h2, "silu" if kind == "swiglu" else "gelu").view(*h.shape[:-1], h.shape[-1] // 2)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import _infer as I
        (h2,) = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        return I.gated_bwd(h2, dy2, "silu" if ctx.kind == "swiglu" else "gelu").view(ctx.shape), None


def gated_activation(h: torch.Tensor, kind: str = "swiglu") -> torch.Tensor:
    """``silu(gate) * up`` (``kind="swiglu"``) or ``gelu_tanh(gate) * up`` (``"geglu"``) of ``h = [gate | up]`` along
    the last axis.  BF16 tensors on a GPU run the fused kernels; everything else the FP32 formula."""
    if kind not in ("swiglu", "geglu"):
        raise ValueError("gated_activation: kind must be 'swiglu' or 'geglu'")
    if _use_kernels(h) and h.dtype == torch.bfloat16 and h.shape[-1] % 2 == 0:
        return _GatedActivation.apply(h, kind)
    Fd = h.shape[-1] // 2
    a, b = h[..., :Fd], h[..., Fd:]
    g = F.silu(a.float()) if kind == "swiglu" else gelu_tanh(a.float())
    return (g * b.float()).to(h.dtype)


# -------------------------------------------------------------------------------------------- norms
class _FusedNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, residual, eps, rms):
        from ..ops import _cuda as K
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        r2 = residual.reshape(-1, shape[-1]).contiguous() if residual is not None else None
        s_out = torch.empty_like(x2) if r2 is not None else None
        g32 = gamma.float() if gamma.dtype != torch.float32 and gamma.dtype != x.dtype else gamma
        b32 = beta.to(g32.dtype) if beta is not None else None
        y, mean, rstd = K.norm_fwd(x2, g32, b32, rms=rms, eps=eps, residual=r2, sum_out=s_out, out_dtype=x.dtype)
        ctx.save_for_backward(s_out if s_out is not None else x2, g32, mean if mean is not None else rstd, rstd)
        ctx.rms, ctx.shape, ctx.has_res, ctx.has_beta = rms, shape, residual is not None, beta is not None
        ctx.pdtypes = (gamma.dtype, beta.dtype if beta is not None else None)
        y = y.view(shape)
        if residual is not None:
            ctx.mark_non_differentiable()
            return y, s_out.view(shape)
        return y, None

    @staticmethod
    def backward(ctx, dy, dsum):
        from ..ops import _cuda as K
        xs, g, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, ctx.shape[-1]).contiguous()
        add = dsum.reshape(-1, ctx.shape[-1]).contiguous() if dsum is not None else None
        dg = torch.zeros(ctx.shape[-1], dtype=torch.float32, device=dy.device)
        db = torch.zeros(ctx.shape[-1], dtype=torch.float32, device=dy.device) if ctx.has_beta else None
        dx = K.norm_bwd(dy2, xs, g, None if ctx.rms else mean, rstd, rms=ctx.rms, add=add, dx_dtype=xs.dtype,
                        dgamma=dg, dbeta=db).view(ctx.shape)
        dgamma = dg.to(ctx.pdtypes[0])
        dbeta = db.to(ctx.pdtypes[1]) if db is not None else None
        return dx, dgamma, dbeta, (dx if ctx.has_res else None), None, None


def _norm_ref(x, gamma, beta, eps, rms):
    if rms:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()).to(x.dtype)
    return F.layer_norm(x.float(), (x.shape[-1],), gamma.float(), beta.float() if beta is not None else None,
                        eps).to(x.dtype)


def fused_layernorm(x, gamma, beta=None, eps: float = 1e-5):
    if _use_kernels(x) and x.shape[-1] % 4 == 0:
        return _FusedNorm.apply(x, gamma, beta, None, eps, False)[0]
    return _norm_ref(x, gamma, beta, eps, False)


def fused_residual_layernorm(x, residual, gamma, beta=None, eps: float = 1e-5):
    """Returns ``(layernorm(x + residual), x + residual)`` from one pass."""
    if _use_kernels(x) and x.shape[-1] % 4 == 0:
        y, s = _FusedNorm.apply(x, gamma, beta, residual, eps, False)
        return y, s
    s = x + residual
    return _norm_ref(s, gamma, beta, eps, False), s


def rms_norm(x, gamma, eps: float = 1e-5):
    if _use_kernels(x) and x.shape[-1] % 4 == 0:
        return _FusedNorm.apply(x, gamma, None, None, eps, True)[0]
    return _norm_ref(x, gamma, None, eps, True)


def fused_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return torch.softmax(x.float(), dim=dim).to(x.dtype)


# ---------------------------------------------------------------------------------------- attention
class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, window, scale, softcap=0.0, alibi_slopes=None, dropout=(0.0, 0, 0)):
        from ..ops import _cuda as K
        o, lse = K.attention_fwd(q, k, v, causal=causal, window=window, scale=scale, softcap=softcap,
                                 alibi_slopes=alibi_slopes, dropout_p=dropout[0], dropout_seed=dropout[1],
                                 dropout_offset=dropout[2])
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cfg = (causal, window, scale, softcap, alibi_slopes, dropout)
        return o

    @staticmethod
    def backward(ctx, do):
        from ..ops import _cuda as K
        q, k, v, o, lse = ctx.saved_tensors
        causal, window, scale, softcap, alibi_slopes, dropout = ctx.cfg
        dq, dk, dv = K.attention_bwd(q, k, v, o, lse, do.contiguous(), causal=causal, window=window, scale=scale,
                                     softcap=softcap, alibi_slopes=alibi_slopes, dropout_p=dropout[0],
                                     dropout_seed=dropout[1], dropout_offset=dropout[2])
        return dq, dk, dv, None, None, None, None, None, None


def attention_reference(q, k, v, causal=True, window=0, scale=None, softcap=0.0, alibi_slopes=None,
                        dropout_p=0.0, dropout_seed=0, dropout_offset=0):
    """Math attention in FP32 on [B, T, H, D] tensors: the oracle of the tensor-core kernels (which draw the same
    Philox dropout stream), and the path for shapes and types they do not take."""
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    scale = D ** -0.5 if scale is None else scale
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    if Hkv != H:
        kf = kf.repeat_interleave(H // Hkv, 1)
        vf = vf.repeat_interleave(H // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    if softcap > 0.0:
        s = softcap * torch.tanh(s / softcap)
    qi = torch.arange(Tq, device=q.device)[:, None] + (Tk - Tq)
    ki = torch.arange(Tk, device=q.device)[None]
    if alibi_slopes is not None:
        s = s + alibi_slopes.float().view(1, H, 1, 1) * (ki - qi).float()
    mask = torch.zeros(Tq, Tk, dtype=torch.bool, device=q.device)
    if causal:
        mask |= ki > qi
    if window > 0:
        mask |= ki < qi - window + 1
    s = s.masked_fill(mask, float("-inf"))
    p = torch.softmax(s, -1)
    p = torch.nan_to_num(p, nan=0.0)
    if dropout_p > 0.0:
        keep = torch.from_numpy(_philox.dropout_mask(p.numel(), dropout_p, dropout_seed, dropout_offset))
        p = p * keep.view(p.shape).to(p.device) / (1.0 - dropout_p)
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)


def attention(q, k, v, causal=True, window=0, scale=None, softcap=0.0, alibi_slopes=None, dropout_p=0.0,
              dropout_seed=0, dropout_offset=0):
    """Scaled-dot-product attention on [B, T, H, D] (GQA when k/v have fewer heads)."""
    D = q.shape[-1]
    if _use_kernels(q) and D in (64, 128) and q.dtype == torch.bfloat16 and \
            all(t.stride(-1) == 1 and t.stride(1) % 8 == 0 and t.stride(2) % 8 == 0 for t in (q, k, v)):
        slopes = None if alibi_slopes is None else alibi_slopes.detach().float().contiguous().to(q.device)
        return _FlashAttention.apply(q, k, v, causal, window, scale, float(softcap), slopes,
                                     (float(dropout_p), int(dropout_seed), int(dropout_offset)))
    if not q.is_cuda and q.dtype == torch.float32 and dropout_p == 0.0 and \
            not (torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)):
        # CPU inference: the blocked native kernel (no [Tq, Tk] score matrix)
        from .. import cpu as _cpu
        o, _ = _cpu.flash_attention(q.detach().contiguous().numpy(), k.detach().contiguous().numpy(),
                                    v.detach().contiguous().numpy(), causal=causal, window=window, scale=scale,
                                    softcap=softcap, alibi=None if alibi_slopes is None else alibi_slopes.detach().float().numpy())
        return torch.from_numpy(o)
    return attention_reference(q, k, v, causal, window, scale, softcap, alibi_slopes, dropout_p, dropout_seed,
                               dropout_offset)


def attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k=None, causal=True, window=0, scale=None, softcap=0.0,
                     alibi_slopes=None, dropout_p=0.0, dropout_seed=0, dropout_offset=0):
    """Attention over a packed batch of variable-length sequences.

    q [total_q, H, D], k / v [total_k, Hkv, D]; ``cu_seqlens_*`` are the [batch + 1] cumulative lengths
    (``cu_seqlens_k`` defaults to ``cu_seqlens_q``).  Sequence i attends only to itself; the causal mask is
    bottom-right aligned when its query and key lengths differ.  Each sequence is one launch of the tensor-core
    kernels on a strided view of the packed tensors (no copy, no padding), so the gradients flow through the same
    backward kernels.  Parity: the cu_seqlens fields of include/nexus/attention/params.hpp of the reference.
    """
    cq = [int(x) for x in (cu_seqlens_q.tolist() if torch.is_tensor(cu_seqlens_q) else cu_seqlens_q)]
    ck = cq if cu_seqlens_k is None else \
        [int(x) for x in (cu_seqlens_k.tolist() if torch.is_tensor(cu_seqlens_k) else cu_seqlens_k)]
    if len(cq) != len(ck) or len(cq) < 2 or cq[0] != 0 or ck[0] != 0 or cq[-1] != q.shape[0] or ck[-1] != k.shape[0]:
        raise ValueError("attention_varlen: cumulative lengths do not describe the packed tensors")
    outs = []
    for i in range(len(cq) - 1):
        if cq[i + 1] < cq[i] or ck[i + 1] < ck[i]:
            raise ValueError("attention_varlen: cumulative lengths must not decrease")
        if cq[i + 1] == cq[i]:
            continue
        if ck[i + 1] == ck[i]:          # no key at all: the output rows are zero
            outs.append(torch.zeros_like(q[cq[i]:cq[i + 1]]))
            continue
        o = attention(q[None, cq[i]:cq[i + 1]], k[None, ck[i]:ck[i + 1]], v[None, ck[i]:ck[i + 1]], causal, window,
                      scale, softcap, alibi_slopes, dropout_p, dropout_seed, dropout_offset + cq[i])
        outs.append(o[0])
    return torch.cat(outs, 0) if outs else torch.zeros_like(q)


# ------------------------------------------------------------------------------------ cross-entropy
def _ce_reference(logits, targets, ignore_index, smoothing, z_loss):
    """logits [N, V] float, targets [N] long.  Mean over valid targets of
    (1-s)*nll + s*(lse - mean(logits)) + z*lse^2."""
    lf = logits.float()
    lse = torch.logsumexp(lf, -1)
    valid = targets != ignore_index
    nll = lse - lf.gather(1, targets.clamp(min=0)[:, None])[:, 0]
    per = (1.0 - smoothing) * nll + smoothing * (lse - lf.mean(-1)) + z_loss * lse * lse
    n = valid.sum().clamp(min=1)
    return (per * valid).sum() / n


class _FusedCE(torch.autograd.Function):
    """Loss and gradient in one pass: the gradient overwrites a working copy of the logits, on the device through the
    CUDA kernel, on the host through the native threaded kernel (`csrc/host/fused_train_cpu.cpp`)."""

    @staticmethod
    def forward(ctx, logits, tokens, targets, vocab, ignore_index, smoothing, z_loss):
        ctx.shape, ctx.dtype = logits.shape, logits.dtype
        if not logits.is_cuda:
            from .. import _native
            work = logits.detach().reshape(-1, logits.shape[-1]).to(torch.float32).clone()
            tg = (shifted_targets(tokens, ignore_index) if targets is None else targets).reshape(-1)
            tg = tg.to(torch.int32).contiguous()
            loss, _ = _native.cpu_cross_entropy(work.numpy(), tg.numpy(), vocab, ignore_index, smoothing, z_loss, 1.0, True)
            ctx.save_for_backward(work)
            return torch.tensor(loss, dtype=torch.float32)
        from ..ops import _cuda as K
        work = logits.reshape(-1, logits.shape[-1]).clone()  # gradient is produced in place in this copy
        tk = tokens.to(torch.int32).contiguous() if tokens is not None else None
        tg = targets.to(torch.int32).contiguous().reshape(-1) if targets is not None else None
        T = tokens.shape[-1] if tokens is not None else 1
        loss = K.cross_entropy_shifted(work, tk, targets=tg, vocab=vocab, ignore_index=ignore_index,
                                       smoothing=smoothing, z_loss=z_loss, grad_scale=1.0, seq_len=T)
        ctx.save_for_backward(work)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        return (g * dloss.to(g.dtype)).to(ctx.dtype).view(ctx.shape), None, None, None, None, None, None


def _host_fused(logits: torch.Tensor) -> bool:
    """The native host kernel takes 16- and 32-bit floats; FP64 (gradient checks) stays on the torch expression."""
    return not logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16, torch.float16)


def shifted_targets(tokens: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """target[b, t] = tokens[b, t+1]; the last position of every row is ignored."""
    tg = torch.full_like(tokens, ignore_index, dtype=torch.long)
    tg[:, :-1] = tokens[:, 1:].long()
    return tg


def cross_entropy_shifted(logits: torch.Tensor, tokens: torch.Tensor, ignore_index: int = -100,
                          label_smoothing: float = 0.0, z_loss: float = 0.0, vocab: Optional[int] = None):
    """Next-token loss from logits [B, T, V(+pad)] and the input tokens [B, T]."""
    V = vocab or logits.shape[-1]
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and logits.shape[-1] >= V:
        from ..ops import _cuda as K
        K.lib()
        return _FusedCE.apply(logits, tokens, None, V, ignore_index, label_smoothing, z_loss)
    if _host_fused(logits) and logits.shape[-1] >= V:
        return _FusedCE.apply(logits, tokens, None, V, ignore_index, label_smoothing, z_loss)
    tg = shifted_targets(tokens, ignore_index).reshape(-1)
    return _ce_reference(logits.reshape(-1, logits.shape[-1])[:, :V], tg, ignore_index, label_smoothing, z_loss)


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100,
                  label_smoothing: float = 0.0, z_loss: float = 0.0):
    """Unshifted variant: explicit targets [N]."""
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32):
        from ..ops import _cuda as K
        K.lib()
        return _FusedCE.apply(logits, None, targets, logits.shape[-1], ignore_index, label_smoothing, z_loss)
    if _host_fused(logits):
        return _FusedCE.apply(logits, None, targets, logits.shape[-1], ignore_index, label_smoothing, z_loss)
    return _ce_reference(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), ignore_index, label_smoothing,
                         z_loss)


# ---------------------------------------------------------------------------------------- embedding
class _EmbeddingPos(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, wte, wpe, deterministic):
        from ..ops import _cuda as K
        tk = tokens.to(torch.int32).contiguous()
        out = K.embedding_pos_fwd(tk, wte, wpe, out_dtype=wte.dtype, seq_len=tokens.shape[-1])
        ctx.save_for_backward(tk)
        ctx.meta = (wte.shape, wpe.shape if wpe is not None else None, wte.dtype, deterministic)
        return out

    @staticmethod
    def backward(ctx, dy):
        from ..ops import _cuda as K
        (tk,) = ctx.saved_tensors
        wshape, pshape, dt, det = ctx.meta
        B, T = tk.shape
        dwte = torch.zeros(wshape, dtype=torch.float32, device=dy.device)
        dwpe = torch.zeros(pshape, dtype=torch.float32, device=dy.device) if pshape is not None else None
        K.embedding_bwd(tk, dy.contiguous(), dwte, dwpe[:T] if dwpe is not None else None, B, T, deterministic=det)
        return None, dwte.to(dt), dwpe.to(dt) if dwpe is not None else None, None


def embedding_pos(tokens: torch.Tensor, wte: torch.Tensor, wpe: Optional[torch.Tensor] = None,
                  deterministic: bool = True) -> torch.Tensor:
    """``wte[tokens] + wpe[position]`` for tokens [B, T]; deterministic index-sorted backward."""
    if wte.is_cuda and wte.shape[1] % 4 == 0 and wte.dtype in (torch.bfloat16, torch.float32) and tokens.dim() == 2:
        from ..ops import _cuda as K
        K.lib()
        return _EmbeddingPos.apply(tokens, wte, wpe, deterministic)
    out = wte[tokens.long()]
    if wpe is not None:
        out = out + wpe[: tokens.shape[-1]][None]
    return out


# ------------------------------------------------------------------------------------------ dropout
class _DropoutPhilox(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, offset):
        ctx.cfg = (p, seed, offset)
        return _dropout_apply(x, p, seed, offset)

    @staticmethod
    def backward(ctx, dy):
        p, seed, offset = ctx.cfg
        return _dropout_apply(dy.contiguous(), p, seed, offset), None, None, None


def _dropout_apply(x, p, seed, offset):
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32):
        from ..ops import _cuda as K
        return K.dropout(x.contiguous(), p, seed, offset)
    if not x.is_cuda and x.dtype == torch.float32:
        from .. import _native
        return torch.from_numpy(_native.cpu_dropout_philox(x.detach().contiguous().numpy(), p, seed, offset)).view(x.shape)
    keep = torch.from_numpy(_philox.dropout_mask(x.numel(), p, seed, offset)).view(x.shape).to(x.device)
    return torch.where(keep, x * (1.0 / (1.0 - p)), torch.zeros_like(x))


def dropout_philox(x: torch.Tensor, p: float, seed: int, offset: int, training: bool = True) -> torch.Tensor:
    """Counter-based dropout: the mask is a pure function of (seed, offset, element index)."""
    if not training or p <= 0.0:
        return x
    if not (0.0 <= p < 1.0):
        raise ValueError("dropout probability must be in [0, 1)")
    return _DropoutPhilox.apply(x, p, seed, offset)


def philox_uniform(n: int, seed: int, offset: int) -> torch.Tensor:
    return torch.from_numpy(_philox.philox_uniform(n, seed, offset))


# -------------------------------------------------------------------------------------------- AdamW
def adamw_multi_tensor(params: Sequence[torch.Tensor], grads: Sequence[torch.Tensor], m: Sequence[torch.Tensor],
                       v: Sequence[torch.Tensor], step: int, lr: float, beta1: float = 0.9, beta2: float = 0.95,
                       eps: float = 1e-8, weight_decay: float = 0.1, max_grad_norm: float = 0.0,
                       wd_scales: Optional[Sequence[float]] = None, lr_scales: Optional[Sequence[float]] = None,
                       grad_sq_sum: Optional[float] = None) -> float:
    """In-place AdamW over a list of FP32 tensors with one global-norm clip.  ``step`` is 1-based.

    Operation order (kept identical on every backend so results match bit for bit):
    ``clip = min(1, max/(|g|+1e-6)); p -= lr*wd*p; m = b1*m + (1-b1)*g; v = b2*v + (1-b2)*g*g;
    p -= lr*(m*inv1) / (sqrt(v*inv2) + eps)`` with the coefficients computed in double and rounded once.
    Returns the global gradient norm.  ``grad_sq_sum`` overrides the local square sum (sharded callers).
    """
    if grad_sq_sum is None:
        sq = 0.0
        for g in grads:
            sq += float(g.double().pow(2).sum())
    else:
        sq = grad_sq_sum
    norm = math.sqrt(sq)
    if not math.isfinite(norm):
        return norm
    clip = np.float32(1.0)
    if max_grad_norm > 0.0:
        clip = np.float32(min(1.0, max_grad_norm / (norm + 1e-6)))
    inv1 = np.float32(1.0 / (1.0 - beta1 ** step))
    inv2 = np.float32(1.0 / (1.0 - beta2 ** step))
    b1, b2 = np.float32(beta1), np.float32(beta2)
    omb1, omb2 = np.float32(1.0) - b1, np.float32(1.0) - b2
    import sys
    lowp = sys.modules.get("nexus_b200.ops._lowp")
    if lowp is not None:
        lowp.mx_weight_cache.invalidate()   # block-scaled copies of the weights are stale after this update
    with torch.no_grad():
        for i, (p, g, mi, vi) in enumerate(zip(params, grads, m, v)):
            lr_i = np.float32(lr) * np.float32(1.0 if lr_scales is None else lr_scales[i])
            wd_i = np.float32(weight_decay) * np.float32(1.0 if wd_scales is None else wd_scales[i])
            gc = g.float() * float(clip)
            p.sub_(p * float(lr_i * wd_i))
            mi.mul_(float(b1)).add_(gc * float(omb1))
            vi.mul_(float(b2)).add_((gc * gc) * float(omb2))
            denom = (vi * float(inv2)).sqrt_().add_(float(np.float32(eps)))
            p.sub_((mi * float(inv1)) * float(lr_i) / denom)
    return norm
