"""Mixture-of-experts FFN on the GPU kernels: FP32 router, top-k + gate softmax over the selected
experts, capacity assignment in priority order, gather into padded per-expert buffers, expert SwiGLU FFN
as strided-batched tcgen05 GEMMs, gate-weighted combine; full backward (expert weights, router, input).
Parity: src/moe/moe.cpp, include/nexus/lm/moe_layer.hpp:24-37 of the reference (CPU there)."""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _cuda as K
from ..ops import _infer as I


class _Table(C.Structure):
    _fields_ = [("ptr", C.c_void_p * 8)]


def _one(t: torch.Tensor) -> _Table:
    tb = _Table()
    tb.ptr[0] = t.data_ptr()
    return tb


def route(logits: torch.Tensor, k: int, capacity: int):
    """logits FP32 [N, E] -> (expert[N,k] i32, gate[N,k] f32, slot[N,k] i32, counts[E] i32, dropped[1] i32)."""
    N, E = logits.shape
    dev = logits.device
    expert = torch.empty((N, k), dtype=torch.int32, device=dev)
    gate = torch.empty((N, k), dtype=torch.float32, device=dev)
    slot = torch.empty((N, k), dtype=torch.int32, device=dev)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    dropped = torch.zeros(1, dtype=torch.int32, device=dev)
    L = K.lib()
    K._check(L.nx_moe_topk(K._p(logits), C.c_int(N), C.c_int(E), C.c_int(k), K._p(expert), K._p(gate), K._stream()),
             "nx_moe_topk")
    K._check(L.nx_moe_assign(K._p(expert), C.c_int(N), C.c_int(k), C.c_int(E), C.c_int(capacity), K._p(slot),
                             K._p(counts), K._p(dropped), K._stream()), "nx_moe_assign")
    return expert, gate, slot, counts, dropped


def dispatch(x, expert, slot, E: int, capacity: int, row_scale=None) -> torch.Tensor:
    """Rows of x [N, d] (BF16) -> zero-padded buffers [E, capacity, d]."""
    N, d = x.shape
    k = expert.shape[1]
    buf = torch.zeros((E, capacity, d), dtype=torch.bfloat16, device=x.device)
    tb = _one(buf)
    K._check(K.lib().nx_moe_dispatch(K._p(x), K._p(None), K._p(expert), K._p(slot), C.byref(tb), C.c_int(N * k),
                                     C.c_int(d), C.c_int(E), C.c_int(capacity), C.c_int(0), C.c_int(1),
                                     K._p(row_scale), C.c_int(k), K._stream()), "nx_moe_dispatch")
    return buf


def combine(buf, expert, slot, gate, E: int, capacity: int) -> torch.Tensor:
    N, k = expert.shape
    d = buf.shape[-1]
    y = torch.empty((N, d), dtype=torch.bfloat16, device=buf.device)
    tb = _one(buf)
    K._check(K.lib().nx_moe_combine(C.byref(tb), K._p(expert), K._p(slot), K._p(gate), K._p(y), C.c_int(N), C.c_int(k),
                                    C.c_int(d), C.c_int(E), C.c_int(capacity), K._stream()), "nx_moe_combine")
    return y


class _MoeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, router_w, up, down, k, capacity):
        N, d = x.shape
        E, F2, _ = up.shape
        logits = x.float() @ router_w.float().t()
        expert, gate, slot, counts, dropped = route(logits, k, capacity)
        buf = dispatch(x, expert, slot, E, capacity)
        h = K.gemm(buf, up)                                            # [E, C, 2F]
        act = I.gated_fwd(h.view(E * capacity, F2), "silu").view(E, capacity, F2 // 2)
        out = K.gemm(act, down)                                        # [E, C, d]
        y = combine(out, expert, slot, gate, E, capacity)
        ctx.save_for_backward(x, router_w, up, down, expert, gate, slot, buf, h, act, out, logits)
        ctx.k, ctx.capacity = k, capacity
        ctx.mark_non_differentiable(counts, dropped)
        return y, counts, dropped

    @staticmethod
    def backward(ctx, dy, _c, _d):
        x, router_w, up, down, expert, gate, slot, buf, h, act, out, logits = ctx.saved_tensors
        k, cap = ctx.k, ctx.capacity
        N, d = x.shape
        E, F2, _ = up.shape
        dy = dy.contiguous().to(torch.bfloat16)
        dgate = torch.empty((N, k), dtype=torch.float32, device=x.device)
        K._check(K.lib().nx_moe_gate_grad(K._p(dy), K._p(out), K._p(expert), K._p(slot), K._p(dgate), C.c_int(N), C.c_int(k),
                                          C.c_int(d), C.c_int(cap), K._stream()), "nx_moe_gate_grad")
        dout = dispatch(dy, expert, slot, E, cap, row_scale=gate.contiguous().view(-1))
        dact = K.gemm(dout, down, b_mn=True)                           # [E, C, F]
        ddown = K.gemm(dout, act, a_mn=True, b_mn=True, out_dtype=torch.float32)      # [E, d, F]
        dh = I.gated_bwd(h.view(E * cap, F2), dact.view(E * cap, F2 // 2), "silu").view(E, cap, F2)
        dbuf = K.gemm(dh, up, b_mn=True)                               # [E, C, d]
        dup = K.gemm(dh, buf, a_mn=True, b_mn=True, out_dtype=torch.float32)          # [E, 2F, d]
        ones = torch.ones_like(gate)
        dx = combine(dbuf, expert, slot, ones, E, cap).float()
        # router: gate = softmax over the selected logits
        inner = (gate * dgate).sum(-1, keepdim=True)
        dsel = gate * (dgate - inner)
        dlogits = torch.zeros_like(logits).scatter_add_(1, expert.long(), dsel)
        drouter = dlogits.t() @ x.float()
        dx = dx + dlogits @ router_w.float()
        return dx.to(x.dtype), drouter.to(router_w.dtype), dup.to(up.dtype), ddown.to(down.dtype), None, None


def moe_ffn(x: torch.Tensor, router_w: torch.Tensor, up: torch.Tensor, down: torch.Tensor, k: int, capacity: int):
    """x [N, d] BF16, router_w [E, d], up [E, 2F, d] (gate | up rows), down [E, d, F].
    Returns (y [N, d] BF16, counts[E], dropped[1])."""
    if capacity % 8 or x.shape[1] % 8:
        raise ValueError("capacity and model width must be multiples of 8")
    return _MoeFn.apply(x, router_w, up, down, k, capacity)


def reference(x, router_w, up, down, k: int, capacity: int):
    """Plain PyTorch FP32 of the same routing rules (priority: choice, then token)."""
    xf, N = x.float(), x.shape[0]
    E, F2, _ = up.shape
    logits = xf @ router_w.float().t()
    val, idx = torch.sort(logits, dim=-1, descending=True, stable=True)
    val, idx = val[:, :k], idx[:, :k]
    gate = torch.softmax(val, -1)
    y = torch.zeros_like(xf)
    fill = [0] * E
    keep = torch.zeros((N, k), dtype=torch.bool)
    idx_c = idx.cpu()
    for j in range(k):
        for t in range(N):
            e = int(idx_c[t, j])
            if fill[e] < capacity:
                fill[e] += 1
                keep[t, j] = True
    keep = keep.to(x.device)
    for e in range(E):
        m = (idx == e) & keep
        tok, ch = m.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        hh = xf[tok] @ up[e].float().t()
        a = torch.nn.functional.silu(hh[:, : F2 // 2]) * hh[:, F2 // 2:]
        y.index_add_(0, tok, (a @ down[e].float().t()) * gate[tok, ch][:, None])
    return y, idx, gate, keep
