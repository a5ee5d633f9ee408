"""Mixture-of-experts FFN on the GPU kernels: FP32 router, top-k + gate softmax over the selected
experts, capacity assignment in priority order, gather into padded per-expert buffers, expert SwiGLU FFN
as strided-batched tcgen05 GEMMs, gate-weighted combine; full backward (expert weights, router, input).
Parity: src/moe/moe.cpp, include/nexus/lm/moe_layer.hpp:24-37 of the reference (CPU there)."""
from __future__ import annotations

import ctypes as C

from typing import Optional

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


def route_groups(select: torch.Tensor, k: int, capacity: int, groups: int = 1, reroute: bool = False):
    """Routing with a capacity per group of tokens and, optionally, the Reroute overflow policy, on selection scores
    ``select`` FP32 [N, E] (the router logits, or the noisy ones).  Returns (expert_sel [N, k] the top-k before any
    move, expert [N, k] after rerouting, gate [N, k] = softmax over the selected scores, slot [N, k] into buffers of
    ``groups * capacity`` rows per expert, counts [groups, E], dropped [1], rerouted [1]).
    Parity: src/moe/moe.cpp:115-259 of the reference (GShard capacity per group, (choice, token) priority)."""
    N, E = select.shape
    dev = select.device
    order = torch.sort(select.detach(), dim=-1, descending=True, stable=True).indices.to(torch.int32).contiguous()
    expert_sel = order[:, :k].contiguous()
    gate = torch.softmax(select.gather(1, expert_sel.long()), -1)
    expert = expert_sel.clone()
    slot = torch.empty((N, k), dtype=torch.int32, device=dev)
    counts = torch.zeros(groups * E, dtype=torch.int32, device=dev)
    dropped = torch.zeros(1, dtype=torch.int32, device=dev)
    rerouted = torch.zeros(1, dtype=torch.int32, device=dev)
    K._check(K.lib().nx_moe_assign_groups(K._p(expert), K._p(order if reroute else None), C.c_int(N), C.c_int(k),
                                          C.c_int(E), C.c_int(groups), C.c_int(capacity), K._p(slot), K._p(counts),
                                          K._p(dropped), K._p(rerouted), K._stream()), "nx_moe_assign_groups")
    return expert_sel, expert, gate, slot, counts.view(groups, E), dropped, rerouted


class _MoeGroupsFn(torch.autograd.Function):
    """`_MoeFn` with group capacities, Reroute and noisy top-k.  The gate of an assignment is the softmax over the
    scores of the token's ORIGINAL top-k (a rerouted assignment keeps its weight), so the router gradient goes to the
    originally selected logits while rows travel to the final experts."""

    @staticmethod
    def forward(ctx, x, router_w, noise_w, up, down, k, capacity, groups, reroute, eps):
        N, d = x.shape
        E, F2, _ = up.shape
        cap = groups * capacity
        logits = x.float() @ router_w.float().t()
        nl = None
        select = logits
        if noise_w is not None and eps is not None:
            nl = x.float() @ noise_w.float().t()
            select = logits + eps * torch.nn.functional.softplus(nl)
        expert_sel, expert, gate, slot, counts, dropped, rerouted = route_groups(select, k, capacity, groups, reroute)
        buf = dispatch(x, expert, slot, E, cap)
        h = K.gemm(buf, up)
        act = I.gated_fwd(h.view(E * cap, F2), "silu").view(E, cap, F2 // 2)
        out = K.gemm(act, down)
        y = combine(out, expert, slot, gate, E, cap)
        ctx.save_for_backward(x, router_w, noise_w if noise_w is not None else x.new_zeros(0), up, down, expert_sel, expert,
                              gate, slot, buf, h, act, out, nl if nl is not None else x.new_zeros(0),
                              eps if eps is not None else x.new_zeros(0))
        ctx.k, ctx.cap, ctx.noisy = k, cap, nl is not None
        ctx.mark_non_differentiable(counts, dropped, rerouted)
        return y, counts, dropped, rerouted

    @staticmethod
    def backward(ctx, dy, _c, _d, _r):
        x, router_w, noise_w, up, down, expert_sel, expert, gate, slot, buf, h, act, out, nl, eps = ctx.saved_tensors
        k, cap = ctx.k, ctx.cap
        N, d = x.shape
        E, F2, _ = up.shape
        dy = dy.contiguous().to(torch.bfloat16)
        dgate = torch.empty((N, k), dtype=torch.float32, device=x.device)
        K._check(K.lib().nx_moe_gate_grad(K._p(dy), K._p(out), K._p(expert), K._p(slot), K._p(dgate), C.c_int(N), C.c_int(k),
                                          C.c_int(d), C.c_int(cap), K._stream()), "nx_moe_gate_grad")
        dout = dispatch(dy, expert, slot, E, cap, row_scale=gate.contiguous().view(-1))
        dact = K.gemm(dout, down, b_mn=True)
        ddown = K.gemm(dout, act, a_mn=True, b_mn=True, out_dtype=torch.float32)
        dh = I.gated_bwd(h.view(E * cap, F2), dact.view(E * cap, F2 // 2), "silu").view(E, cap, F2)
        dbuf = K.gemm(dh, up, b_mn=True)
        dup = K.gemm(dh, buf, a_mn=True, b_mn=True, out_dtype=torch.float32)
        dx = combine(dbuf, expert, slot, torch.ones_like(gate), E, cap).float()
        inner = (gate * dgate).sum(-1, keepdim=True)
        dsel = gate * (dgate - inner)
        dselect = torch.zeros((N, E), dtype=torch.float32, device=x.device).scatter_add_(1, expert_sel.long(), dsel)
        drouter = dselect.t() @ x.float()
        dx = dx + dselect @ router_w.float()
        dnoise = None
        if ctx.noisy:
            dnl = dselect * eps * torch.sigmoid(nl)
            dnoise = (dnl.t() @ x.float()).to(noise_w.dtype)
            dx = dx + dnl @ noise_w.float()
        return (dx.to(x.dtype), drouter.to(router_w.dtype), dnoise, dup.to(up.dtype), ddown.to(down.dtype),
                None, None, None, None, None)


def noise_sample(tokens: int, experts: int, seed: int, device) -> torch.Tensor:
    """The standard-normal draws of the noisy top-k router: the CPU generator's stream for ``seed`` (the one
    `moe.route` uses), moved to the device, so both paths select the same experts."""
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    return torch.randn((tokens, experts), generator=g).to(device)


def moe_ffn(x: torch.Tensor, router_w: torch.Tensor, up: torch.Tensor, down: torch.Tensor, k: int, capacity: int, *,
            groups: int = 1, overflow: str = "drop", noise_w: Optional[torch.Tensor] = None, noise_seed: int = 0,
            training: bool = False):
    """x [N, d] BF16, router_w [E, d], up [E, 2F, d] (gate | up rows), down [E, d, F]; ``capacity`` rows per expert
    and group.  Returns (y [N, d] BF16, counts, dropped[1]) for the plain policy (one group, drop, no noise), and
    (y, counts [groups, E], dropped[1], rerouted[1]) when ``groups`` > 1, ``overflow`` = "reroute" or a noisy router
    (``noise_w`` [E, d], used in training) is asked for."""
    if capacity % 8 or x.shape[1] % 8:
        raise ValueError("capacity and model width must be multiples of 8")
    if overflow not in ("drop", "reroute"):
        raise ValueError("overflow must be 'drop' or 'reroute'")
    noisy = training and noise_w is not None
    if groups == 1 and overflow == "drop" and not noisy:
        return _MoeFn.apply(x, router_w, up, down, k, capacity)
    if x.shape[0] % groups:
        raise ValueError(f"token count {x.shape[0]} must be divisible by groups {groups}")
    eps = noise_sample(x.shape[0], up.shape[0], noise_seed, x.device) if noisy else None
    return _MoeGroupsFn.apply(x, router_w, noise_w if noisy else None, up, down, k, capacity, groups,
                              overflow == "reroute", eps)


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
