"""Differentiable collectives: each forward collective is paired with the collective that carries
its gradient (all-gather <-> reduce-scatter, all-reduce <-> identity, all-to-all <-> all-to-all).
These are the region boundaries of tensor / sequence / context / expert parallelism."""
from __future__ import annotations

from typing import List

import torch


class _AllReduce(torch.autograd.Function):
    """Forward all-reduce(sum), backward identity (the "g" operator of Megatron row-parallel layers)."""

    @staticmethod
    def forward(ctx, x, pg):
        y = x.contiguous().clone()
        pg.all_reduce_tensor(y, "sum")
        return y

    @staticmethod
    def backward(ctx, dy):
        return dy, None


class _CopyToGroup(torch.autograd.Function):
    """Forward identity, backward all-reduce(sum) (the "f" operator of column-parallel layers)."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return x

    @staticmethod
    def backward(ctx, dy):
        g = dy.contiguous().clone()
        ctx.pg.all_reduce_tensor(g, "sum")
        return g, None


class _AllGatherRows(torch.autograd.Function):
    """[n/tp, ...] -> [n, ...] along dim 0; backward reduce-scatter (sequence-parallel region entry)."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        x = x.contiguous()
        out = torch.empty((x.shape[0] * pg.size(),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        pg.all_gather_tensor(out, x)
        return out

    @staticmethod
    def backward(ctx, dy):
        pg = ctx.pg
        dy = dy.contiguous()
        out = torch.empty((dy.shape[0] // pg.size(),) + tuple(dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        pg.reduce_scatter_tensor(out, dy, "sum")
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    """[n, ...] -> sum-reduced [n/tp, ...]; backward all-gather (sequence-parallel region exit)."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        x = x.contiguous()
        out = torch.empty((x.shape[0] // pg.size(),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        pg.reduce_scatter_tensor(out, x, "sum")
        return out

    @staticmethod
    def backward(ctx, dy):
        pg = ctx.pg
        dy = dy.contiguous()
        out = torch.empty((dy.shape[0] * pg.size(),) + tuple(dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        pg.all_gather_tensor(out, dy)
        return out, None


class _AllToAll(torch.autograd.Function):
    """Equal-split all-to-all: scatter dim ``sd`` over ranks, gather along dim ``gd``."""

    @staticmethod
    def forward(ctx, x, pg, sd, gd):
        ctx.cfg = (pg, sd, gd)
        return _a2a(x, pg, sd, gd)

    @staticmethod
    def backward(ctx, dy):
        pg, sd, gd = ctx.cfg
        return _a2a(dy, pg, gd, sd), None, None, None


def _a2a(x, pg, sd, gd):
    n = pg.size()
    parts = [p.contiguous() for p in x.chunk(n, dim=sd)]
    shape = parts[0].shape
    recv = pg.all_to_all_v([p.reshape(-1) for p in parts])
    return torch.cat([r.view(shape) for r in recv], dim=gd)


def all_reduce(x, pg): return x if pg is None or pg.size() == 1 else _AllReduce.apply(x, pg)
def copy_to_group(x, pg): return x if pg is None or pg.size() == 1 else _CopyToGroup.apply(x, pg)
def all_gather_rows(x, pg): return x if pg is None or pg.size() == 1 else _AllGatherRows.apply(x, pg)
def reduce_scatter_rows(x, pg): return x if pg is None or pg.size() == 1 else _ReduceScatterRows.apply(x, pg)
def all_to_all(x, pg, scatter_dim, gather_dim):
    return x if pg is None or pg.size() == 1 else _AllToAll.apply(x, pg, scatter_dim, gather_dim)
