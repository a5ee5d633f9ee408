"""Expert-parallel mixture-of-experts FFN on GPUs: the experts of a layer are split over the ranks of a group, tokens
stay on the rank that holds them (data parallel), and routed rows travel by peer-memory kernels:

  forward   route (FP32 router, top-k, softmax over the selected logits) -> global slot of every assignment (rank-major
            priority, capacity per expert over ALL ranks' tokens) -> `nx_moe_dispatch` stores each kept row straight into
            the owner's capacity buffer over NVLink -> barrier -> the owner runs its experts as strided-batched tcgen05
            GEMMs (gate/up, SwiGLU, down) -> barrier -> `nx_moe_combine` pulls every token's expert rows back from
            their owners, gate-weighted
  backward  the mirror image: gate-scaled d(y) rows dispatched to the owners, expert weight / input gradient GEMMs there,
            input gradients pulled back, router gradient from d(gate) (dot products against the owners' output rows)

The per-expert row counts that fix the global slots are exchanged with one small NCCL all-gather (control data);
every activation byte moves through the dispatch / combine kernels.  With one rank the same code is the single-GPU
layer, which is the oracle of the 2-GPU test.

Parity: include/nexus/dist/moe_ep.hpp:5-65, src/dist/moe_ep.cpp:45-90 (exchange counts, exchange rows, local expert
GEMMs, exchange back, combine) and the routing rules of src/moe/moe.cpp:115-259 (drop policy) of the reference.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch

from ..ops import _cuda as K
from ..ops import _infer as I


class _Table(C.Structure):
    _fields_ = [("ptr", C.c_void_p * 8)]


class EpContext:
    """Buffers of one expert-parallel group for layers of one shape: two peer-mapped capacity buffers per rank
    ([local experts, capacity, d] BF16; one carries rows to the experts, the other their results back) and the group's
    symmetric workspace (barrier).  One context serves every MoE layer of a model (layers run one after the other)."""

    def __init__(self, pg, experts: int, d_model: int, tokens_per_rank: int, top_k: int, capacity_factor: float,
                 device, min_capacity: int = 8, comm: Optional[str] = None):
        self.pg = pg
        # "fused": rows move by the peer-memory dispatch / combine kernels; "nccl": the same routing and slots, rows
        # exchanged with variable-split all-to-alls (the library form, kept as the same-box comparison)
        self.comm = comm or os.environ.get("NEXUS_B200_EP_COMM", "fused")
        if self.comm not in ("fused", "nccl"):
            raise ValueError("EpContext.comm must be 'fused' or 'nccl'")
        self.n = pg.size() if pg is not None else 1
        self.rank = pg.rank() if pg is not None else 0
        if experts % self.n:
            raise ValueError("experts must divide by the expert-parallel degree")
        self.E, self.le, self.d, self.k = experts, experts // self.n, d_model, top_k
        total = tokens_per_rank * self.n
        cap = max(min_capacity, math.ceil(capacity_factor * total * top_k / experts))
        self.capacity = (cap + 7) // 8 * 8
        self.device = torch.device(device)
        numel = self.le * self.capacity * d_model
        if self.n > 1 and self.comm == "nccl":
            from ..parallel.symm import SymmetricWorkspace
            self.ws = SymmetricWorkspace(pg)             # the trainer's gradient reductions still use it
            self.in_local = torch.zeros(numel, dtype=torch.bfloat16, device=self.device)
            self.out_local = torch.zeros(numel, dtype=torch.bfloat16, device=self.device)
            self.in_table = self.out_table = None
        elif self.n > 1:
            from ..parallel.symm import SymmetricWorkspace
            self.ws = SymmetricWorkspace(pg)
            self.inbuf = self.ws.alloc(numel, torch.bfloat16)
            self.outbuf = self.ws.alloc(numel, torch.bfloat16)
            self.in_local, self.out_local = self.inbuf.local, self.outbuf.local
            self.in_table, self.out_table = self.inbuf.table, self.outbuf.table
        else:
            self.ws = None
            self.in_local = torch.zeros(numel, dtype=torch.bfloat16, device=self.device)
            self.out_local = torch.zeros(numel, dtype=torch.bfloat16, device=self.device)
            self.in_table, self.out_table = _Table(), _Table()
            self.in_table.ptr[0], self.out_table.ptr[0] = self.in_local.data_ptr(), self.out_local.data_ptr()

    def barrier(self) -> None:
        if self.ws is not None:
            self.ws.barrier()

    def view(self, flat: torch.Tensor) -> torch.Tensor:
        return flat.view(self.le, self.capacity, self.d)


def _dispatch(ctx: EpContext, x, expert, slot, table, row_scale=None) -> None:
    N, k = expert.shape
    K._check(K.lib().nx_moe_dispatch(K._p(x), K._p(None), K._p(expert), K._p(slot), C.byref(table), C.c_int(N * k),
                                     C.c_int(ctx.d), C.c_int(ctx.le), C.c_int(ctx.capacity), C.c_int(ctx.rank),
                                     C.c_int(ctx.n), K._p(row_scale), C.c_int(k), K._stream()), "nx_moe_dispatch")


def _combine(ctx: EpContext, table, expert, slot, gate) -> torch.Tensor:
    N, k = expert.shape
    y = torch.empty((N, ctx.d), dtype=torch.bfloat16, device=expert.device)
    K._check(K.lib().nx_moe_combine(C.byref(table), K._p(expert), K._p(slot), K._p(gate), K._p(y), C.c_int(N), C.c_int(k),
                                    C.c_int(ctx.d), C.c_int(ctx.le), C.c_int(ctx.capacity), K._stream()), "nx_moe_combine")
    return y


def route_global(ctx: EpContext, logits: torch.Tensor):
    """Top-k routing of this rank's tokens with GLOBAL slots: assignment (t, j) of rank r gets position
    (rows of ranks < r for that expert) + (its position among rank r's rows, priority j then t); positions at or past
    the capacity are dropped (slot -1).  Returns (expert, gate, slot, global counts [E] before the cap)."""
    N, E = logits.shape
    k = ctx.k
    dev = logits.device
    expert = torch.empty((N, k), dtype=torch.int32, device=dev)
    gate = torch.empty((N, k), dtype=torch.float32, device=dev)
    slot = torch.empty((N, k), dtype=torch.int32, device=dev)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    L = K.lib()
    K._check(L.nx_moe_topk(K._p(logits), C.c_int(N), C.c_int(E), C.c_int(k), K._p(expert), K._p(gate), K._stream()),
             "nx_moe_topk")
    # local positions without a cap (capacity = every assignment), then shift by the lower ranks' counts
    K._check(L.nx_moe_assign(K._p(expert), C.c_int(N), C.c_int(k), C.c_int(E), C.c_int(N * k), K._p(slot), K._p(counts),
                             K._p(None), K._stream()), "nx_moe_assign")
    if ctx.n > 1:
        allc = torch.empty(ctx.n * E, dtype=torch.int32, device=dev)
        ctx.pg.all_gather_tensor(allc, counts)
        allc = allc.view(ctx.n, E)
        base = allc[: ctx.rank].sum(0, dtype=torch.int32)
        total = allc.sum(0, dtype=torch.int32)
        slot = slot + base[expert.long()]
    else:
        total = counts
    slot = torch.where(slot < ctx.capacity, slot, torch.full_like(slot, -1))
    return expert, gate, slot.contiguous(), total


class _A2aPlan:
    """Row exchange of one routing decision through NCCL all-to-alls: which (token, choice) rows go to which rank, in
    (destination rank, expert, slot) order, and where the rows this rank receives sit in its capacity buffer."""

    def __init__(self, ep: EpContext, expert: torch.Tensor, slot: torch.Tensor):
        import torch.distributed as dist
        self.ep, self.dist = ep, dist
        n, le, cap = ep.n, ep.le, ep.capacity
        flat_e, flat_s = expert.reshape(-1).long(), slot.reshape(-1).long()
        keep = flat_s >= 0
        key = torch.where(keep, flat_e * cap + flat_s, torch.full_like(flat_e, ep.E * cap))
        order = torch.argsort(key, stable=True)
        self.nkeep = int(keep.sum())
        self.rows = order[: self.nkeep]                               # flat (token * k + choice) indices, sorted
        self.pos = key[self.rows]                                     # global (expert * cap + slot)
        dst = self.pos // (le * cap)
        send = torch.bincount(dst, minlength=n).to(torch.int64)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=ep.pg.group)
        self.send, self.recv = [int(v) for v in send.cpu()], [int(v) for v in recv.cpu()]
        self.nrecv = sum(self.recv)
        meta = (self.pos - dst * (le * cap)).to(torch.int64)          # position inside the owner's buffer
        self.rpos = torch.empty(self.nrecv, dtype=torch.int64, device=expert.device)
        dist.all_to_all_single(self.rpos, meta, self.recv, self.send, group=ep.pg.group)

    def to_owners(self, rows: torch.Tensor, buf: torch.Tensor) -> None:
        """rows [nkeep, d] (in plan order) -> every owner's capacity buffer ``buf`` [le * cap, d] (zeroed first)."""
        got = torch.empty((self.nrecv, rows.shape[1]), dtype=rows.dtype, device=rows.device)
        self.dist.all_to_all_single(got, rows.contiguous(), self.recv, self.send, group=self.ep.pg.group)
        buf.zero_()
        buf.index_copy_(0, self.rpos, got)

    def from_owners(self, buf: torch.Tensor) -> torch.Tensor:
        """The rows of ``buf`` [le * cap, d] that belong to this rank's assignments, back in plan order [nkeep, d]."""
        back = buf.index_select(0, self.rpos)
        out = torch.empty((self.nkeep, buf.shape[1]), dtype=buf.dtype, device=buf.device)
        self.dist.all_to_all_single(out, back, self.send, self.recv, group=self.ep.pg.group)
        return out


class _MoeEpNcclFn(torch.autograd.Function):
    """The layer of `_MoeEpFn` with the row movement done by NCCL all-to-alls (same routing, slots, expert GEMMs)."""

    @staticmethod
    def forward(ctx, x, logits, up, down, ep: EpContext):
        le, cap, d, k = ep.le, ep.capacity, ep.d, ep.k
        F2 = up.shape[1]
        expert, gate, slot, total = route_global(ep, logits.detach())
        plan = _A2aPlan(ep, expert, slot)
        tok = plan.rows // k
        inb = ep.in_local.view(le * cap, d)
        plan.to_owners(x.index_select(0, tok), inb)
        buf = ep.view(ep.in_local).clone()
        h = K.gemm(buf, up)
        act = I.gated_fwd(h.view(le * cap, F2), "silu").view(le, cap, F2 // 2)
        K.gemm(act, down, out=ep.view(ep.out_local))
        rows_out = plan.from_owners(ep.out_local.view(le * cap, d))              # [nkeep, d] expert outputs of my rows
        g = gate.reshape(-1)[plan.rows].to(torch.float32)
        y = torch.zeros((x.shape[0], d), dtype=torch.float32, device=x.device)
        y.index_add_(0, tok, rows_out.float() * g[:, None])
        ctx.ep, ctx.plan = ep, plan
        ctx.save_for_backward(x, up, down, expert, gate, buf, h, act, rows_out)
        ctx.mark_non_differentiable(total)
        return y.to(torch.bfloat16), total

    @staticmethod
    def backward(ctx, dy, _t):
        x, up, down, expert, gate, buf, h, act, rows_out = ctx.saved_tensors
        ep, plan = ctx.ep, ctx.plan
        le, cap, d, k = ep.le, ep.capacity, ep.d, ep.k
        N, F2 = x.shape[0], up.shape[1]
        dy = dy.contiguous().to(torch.bfloat16)
        tok = plan.rows // k
        dyr = dy.index_select(0, tok)
        dgate = torch.zeros(N * k, dtype=torch.float32, device=x.device)
        dgate[plan.rows] = (dyr.float() * rows_out.float()).sum(-1)
        dgate = dgate.view(N, k)
        g = gate.reshape(-1)[plan.rows].to(torch.float32)
        plan.to_owners((dyr.float() * g[:, None]).to(torch.bfloat16), ep.in_local.view(le * cap, d))
        dout = ep.view(ep.in_local)
        dact = K.gemm(dout, down, b_mn=True)
        ddown = K.gemm(dout, act, a_mn=True, b_mn=True, out_dtype=torch.float32)
        dh = I.gated_bwd(h.view(le * cap, F2), dact.view(le * cap, F2 // 2), "silu").view(le, cap, F2)
        K.gemm(dh, up, b_mn=True, out=ep.view(ep.out_local))
        dup = K.gemm(dh, buf, a_mn=True, b_mn=True, out_dtype=torch.float32)
        dxr = plan.from_owners(ep.out_local.view(le * cap, d))
        dx = torch.zeros((N, d), dtype=torch.float32, device=x.device)
        dx.index_add_(0, tok, dxr.float())
        inner = (gate * dgate).sum(-1, keepdim=True)
        dsel = gate * (dgate - inner)
        dlogits = torch.zeros((N, ep.E), dtype=torch.float32, device=x.device).scatter_add_(1, expert.long(), dsel)
        return dx.to(torch.bfloat16), dlogits, dup.to(up.dtype), ddown.to(down.dtype), None


class _MoeEpFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, logits, up, down, ep: EpContext):
        """x [N, d] BF16 (this rank's tokens); logits [N, E] FP32 router scores (differentiable); up [le, 2F, d],
        down [le, d, F] BF16 (this rank's experts)."""
        le, cap, d = ep.le, ep.capacity, ep.d
        F2 = up.shape[1]
        expert, gate, slot, total = route_global(ep, logits.detach())
        ep.in_local.zero_()
        ep.barrier()                                     # every owner's buffer is cleared and no longer read
        _dispatch(ep, x, expert, slot, ep.in_table)
        ep.barrier()                                     # every rank's rows have landed
        buf = ep.view(ep.in_local).clone()               # kept for the weight gradient
        h = K.gemm(buf, up)                              # [le, C, 2F]
        act = I.gated_fwd(h.view(le * cap, F2), "silu").view(le, cap, F2 // 2)
        K.gemm(act, down, out=ep.view(ep.out_local))     # [le, C, d] into the peer-readable result buffer
        ep.barrier()                                     # results complete on every owner
        y = _combine(ep, ep.out_table, expert, slot, gate)
        ctx.ep = ep
        ctx.save_for_backward(x, up, down, expert, gate, slot, buf, h, act)
        ctx.mark_non_differentiable(total)
        return y, total

    @staticmethod
    def backward(ctx, dy, _t):
        x, up, down, expert, gate, slot, buf, h, act = ctx.saved_tensors
        ep = ctx.ep
        le, cap, d, k = ep.le, ep.capacity, ep.d, ep.k
        N = x.shape[0]
        F2 = up.shape[1]
        dy = dy.contiguous().to(torch.bfloat16)
        # d(gate): the owners' output rows are recomputed into the result buffer (the forward's may be gone)
        K.gemm(act, down, out=ep.view(ep.out_local))
        ep.in_local.zero_()
        ep.barrier()
        dgate = torch.empty((N, k), dtype=torch.float32, device=x.device)
        K._check(K.lib().nx_moe_gate_grad_peers(K._p(dy), C.byref(ep.out_table), K._p(expert), K._p(slot), K._p(dgate),
                                                C.c_int(N), C.c_int(k), C.c_int(d), C.c_int(le), C.c_int(cap),
                                                K._stream()), "nx_moe_gate_grad_peers")
        _dispatch(ep, dy, expert, slot, ep.in_table, row_scale=gate.contiguous().view(-1))
        ep.barrier()                                     # gate-scaled d(y) rows are with the owners; outputs were read
        dout = ep.view(ep.in_local)
        dact = K.gemm(dout, down, b_mn=True)                                            # [le, C, F]
        ddown = K.gemm(dout, act, a_mn=True, b_mn=True, out_dtype=torch.float32)        # [le, d, F]
        dh = I.gated_bwd(h.view(le * cap, F2), dact.view(le * cap, F2 // 2), "silu").view(le, cap, F2)
        K.gemm(dh, up, b_mn=True, out=ep.view(ep.out_local))                            # d(buf) [le, C, d]
        dup = K.gemm(dh, buf, a_mn=True, b_mn=True, out_dtype=torch.float32)            # [le, 2F, d]
        ep.barrier()                                     # input gradients complete on every owner
        dx = _combine(ep, ep.out_table, expert, slot, torch.ones_like(gate))
        ep.barrier()                                     # nobody reads the result buffers any more
        # router: gate = softmax over the selected logits
        inner = (gate * dgate).sum(-1, keepdim=True)
        dsel = gate * (dgate - inner)
        dlogits = torch.zeros((N, ep.E), dtype=torch.float32, device=x.device).scatter_add_(1, expert.long(), dsel)
        return dx, dlogits, dup.to(up.dtype), ddown.to(down.dtype), None


class MoeEpLayer(torch.nn.Module):
    """Top-k MoE SwiGLU FFN with the experts split over an expert-parallel group.

    ``forward(x [N, d] BF16) -> (y [N, d] BF16, aux loss)``; the auxiliary loss is ``aux_alpha * E * sum_e f_e P_e``
    with f_e the global fraction of assignments sent to expert e and P_e this rank's mean router probability (its
    gradient, summed over the ranks by the data-parallel reduction, is that of the global statistic)."""

    def __init__(self, ep: EpContext, d_ff: int, aux_alpha: float = 0.01, init_std: float = 0.02, seed: int = 0,
                 dtype=torch.bfloat16):
        super().__init__()
        self.ep, self.F, self.aux_alpha = ep, d_ff, aux_alpha
        g = torch.Generator(device="cpu").manual_seed(seed)
        E, le, d = ep.E, ep.le, ep.d
        self.router = torch.nn.Parameter((torch.randn(E, d, generator=g) * init_std).to(ep.device, dtype))
        # every rank draws all experts from the same stream and keeps its own block: a 1-rank and an n-rank model agree
        up = torch.randn(E, 2 * d_ff, d, generator=g) * init_std
        down = torch.randn(E, d, d_ff, generator=g) * init_std
        sl = slice(ep.rank * le, (ep.rank + 1) * le)
        self.up = torch.nn.Parameter(up[sl].to(ep.device, dtype).contiguous())
        self.down = torch.nn.Parameter(down[sl].to(ep.device, dtype).contiguous())
        self.last_counts: Optional[torch.Tensor] = None

    def forward(self, x: torch.Tensor):
        ep = self.ep
        logits = x.float() @ self.router.float().t()
        fn = _MoeEpNcclFn if (ep.comm == "nccl" and ep.n > 1) else _MoeEpFn
        y, total = fn.apply(x, logits, self.up, self.down, ep)
        self.last_counts = total
        probs = torch.softmax(logits, dim=-1).mean(0)                       # P_e over this rank's tokens
        frac = total.float() / max(float(x.shape[0] * ep.n * ep.k), 1.0)    # f_e over all ranks (no gradient)
        aux = self.aux_alpha * ep.E * (frac * probs).sum()
        return y, aux
