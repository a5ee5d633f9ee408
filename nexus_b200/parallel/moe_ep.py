"""Expert parallelism: experts live in contiguous blocks on the ranks of an EP group.  Per layer:
exchange per-expert row counts (all-to-all), then the routed rows (all-to-all-v) to the expert
owners, run the local grouped expert GEMMs, send results back (all-to-all-v), gate-weighted
combine.  Backward mirrors the exchanges through autograd.  The load-balancing / z losses use
globally all-reduced routing statistics, so a 1-rank run and an ep-rank run over the same tokens
agree (outputs, input gradients and expert gradients).

On NVSwitch machines the same dispatch / combine is also available as fused device kernels that
store rows straight into the expert owner's buffer over peer memory (`parallel.symm`).

Parity: include/nexus/dist/moe_ep.hpp:5-65 and src/dist/moe_ep.cpp:45-90 of the reference.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional

import torch

from ..moe.moe import Routing, Spec, combine, experts_forward, route


@dataclass
class MoeEpStats:
    a2a_ms: float = 0.0
    a2a_bytes: int = 0
    rows_sent: int = 0
    rows_received: int = 0


class _ExchangeRows(torch.autograd.Function):
    """all-to-all-v of row blocks; backward sends the gradients back along the same routes."""

    @staticmethod
    def forward(ctx, x, send_counts, recv_counts, pg):
        ctx.pg, ctx.sc, ctx.rc = pg, send_counts, recv_counts
        d = x.shape[1]
        parts = [p.contiguous().reshape(-1) for p in x.split(send_counts, dim=0)]
        recv = pg.all_to_all_v(parts)
        return torch.cat([r.view(-1, d) for r in recv], dim=0) if recv else x.new_zeros((0, d))

    @staticmethod
    def backward(ctx, dy):
        d = dy.shape[1]
        parts = [p.contiguous().reshape(-1) for p in dy.split(ctx.rc, dim=0)]
        back = ctx.pg.all_to_all_v(parts)
        return torch.cat([b.view(-1, d) for b in back], dim=0), None, None, None


class MoeExpertParallel(torch.nn.Module):
    """MoE layer whose ``E`` experts are split over ``pg`` (rank r owns experts [r*E/ep, (r+1)*E/ep))."""

    def __init__(self, spec: Spec, pg, init_std: float = 0.02, seed: int = 0, full_up=None, full_down=None,
                 router=None):
        super().__init__()
        spec.validate()
        ep = pg.size() if pg is not None else 1
        if spec.experts % ep:
            raise ValueError("experts must be divisible by the expert-parallel size")
        self.spec, self.pg, self.ep = spec, pg, ep
        self.local = spec.experts // ep
        r = pg.rank() if pg is not None else 0
        g = torch.Generator().manual_seed(seed)
        E, d, Fd = spec.experts, spec.d_model, spec.d_ff
        router0 = torch.randn(d, E, generator=g) * init_std
        up0 = torch.randn(E, 2 * Fd, d, generator=g) * init_std
        down0 = torch.randn(E, d, Fd, generator=g) * init_std
        self.router = torch.nn.Parameter(router if router is not None else router0)
        sl = slice(r * self.local, (r + 1) * self.local)
        self.up = torch.nn.Parameter((full_up if full_up is not None else up0)[sl].clone())
        self.down = torch.nn.Parameter((full_down if full_down is not None else down0)[sl].clone())
        self.stats = MoeEpStats()
        self.last_routing: Optional[Routing] = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        spec, pg, E = self.spec, self.pg, self.spec.experts
        # global routing statistics for the losses (counts, probability sums, lse^2, tokens)
        loss_stats = None
        if pg is not None and self.ep > 1:
            with torch.no_grad():
                logits = x2.float() @ self.router.float()
                probs = torch.softmax(logits, -1)
                lse = torch.logsumexp(logits, -1)
                top = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, : spec.top_k]
                routed = torch.bincount(top.reshape(-1), minlength=E).double()
                st = torch.cat([routed, probs.double().sum(0), (lse.double() ** 2).sum()[None],
                                torch.tensor([float(x2.shape[0])], dtype=torch.float64, device=x2.device)])
                pg.all_reduce_tensor(st, "sum")
                loss_stats = {"routed": st[:E], "prob_sum": st[E: 2 * E], "lse_sq_sum": float(st[2 * E]),
                              "tokens": float(st[2 * E + 1])}
        r = route(x2, self.router, None, spec, self.training, 0, loss_stats)
        self.last_routing = r
        xp = x2[r.perm_token]                                   # rows sorted by expert
        counts = (r.offsets[1:] - r.offsets[:-1])               # rows per (global) expert
        if pg is None or self.ep == 1:
            yp = experts_forward(xp, r.offsets, self.up, self.down)
            return combine(yp, r, x2).view(shape)
        t0 = time.perf_counter()
        # 1) counts: every rank learns how many rows each peer sends to each of its local experts
        theirs = pg.all_to_all_v([counts[k * self.local: (k + 1) * self.local].clone() for k in range(self.ep)])
        recv_mat = torch.stack(theirs)                          # [src rank, local expert]
        send_counts = [int(counts[k * self.local: (k + 1) * self.local].sum()) for k in range(self.ep)]
        recv_counts = [int(c.sum()) for c in theirs]
        # 2) rows to the expert owners
        got = _ExchangeRows.apply(xp, send_counts, recv_counts, pg)
        # received rows are ordered (source rank, local expert): regroup by local expert
        src_off = torch.zeros(self.ep + 1, dtype=torch.long)
        src_off[1:] = torch.tensor(recv_counts).cumsum(0)
        order = []
        for e in range(self.local):
            for s in range(self.ep):
                start = int(src_off[s] + recv_mat[s, :e].sum())
                order.append(torch.arange(start, start + int(recv_mat[s, e])))
        order = torch.cat(order) if order else torch.zeros(0, dtype=torch.long)
        order = order.to(got.device)
        local_off = torch.zeros(self.local + 1, dtype=torch.long, device=got.device)
        local_off[1:] = recv_mat.sum(0).cumsum(0).to(got.device)
        ye = experts_forward(got[order], local_off, self.up, self.down)
        back = torch.empty_like(ye)
        back[order] = ye
        # 3) results back to the token owners
        yp = _ExchangeRows.apply(back, recv_counts, send_counts, pg)
        self.stats.a2a_ms += (time.perf_counter() - t0) * 1e3
        self.stats.rows_sent += sum(send_counts)
        self.stats.rows_received += sum(recv_counts)
        self.stats.a2a_bytes += (sum(send_counts) + sum(recv_counts)) * x2.shape[1] * x2.element_size() * 2
        return combine(yp, r, x2).view(shape)

    def losses(self) -> torch.Tensor:
        return self.last_routing.aux + self.last_routing.z
