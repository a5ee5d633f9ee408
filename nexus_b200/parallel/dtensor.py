"""`DeviceMesh` and `DTensor`: a row-major mesh of ranks with one sub-group per dimension, tensors
annotated with a placement per mesh dimension — ``Shard(d)``, ``Replicate()`` or ``Partial()`` —
redistribution between placements and propagation rules for matmul, element-wise ops, norms,
softmax and embedding.

Redistribute rules: S->R all-gather, P->R all-reduce, P->S reduce-scatter, S(i)->S(j) all-to-all,
R->S local slice, R->P (keep on index 0, zero elsewhere), S->P (gather then as R->P).

Parity: include/nexus/dist/dtensor.hpp:5-120 and src/dist/dtensor.cpp:356-417 of the reference.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class Shard:
    dim: int


@dataclass(frozen=True)
class Replicate:
    pass


@dataclass(frozen=True)
class Partial:
    pass


class DeviceMesh:
    """Row-major mesh: rank = sum(coord[i] * stride[i]); the last dimension varies fastest."""

    def __init__(self, pg, shape: Sequence[int], names: Optional[Sequence[str]] = None):
        self.pg, self.shape = pg, tuple(int(s) for s in shape)
        n = 1
        for s in self.shape:
            n *= s
        if n != pg.size():
            raise ValueError(f"mesh {self.shape} does not cover {pg.size()} ranks")
        self.names = tuple(names) if names else tuple(f"d{i}" for i in range(len(self.shape)))
        self.rank = pg.rank()
        self.strides = []
        st = 1
        for s in reversed(self.shape):
            self.strides.insert(0, st)
            st *= s
        self.coord = tuple((self.rank // self.strides[i]) % self.shape[i] for i in range(len(self.shape)))
        self._groups: Dict[int, object] = {}
        for d in range(len(self.shape)):   # every rank creates every sub-group in the same order
            mine = None
            seen = set()
            for r in range(pg.size()):
                base = r - ((r // self.strides[d]) % self.shape[d]) * self.strides[d]
                if base in seen:
                    continue
                seen.add(base)
                ranks = [base + k * self.strides[d] for k in range(self.shape[d])]
                g = pg.new_group(ranks) if self.shape[d] > 1 else None
                if self.rank in ranks:
                    mine = g
            self._groups[d] = mine

    def group(self, dim) -> Optional[object]:
        d = self.names.index(dim) if isinstance(dim, str) else dim
        return self._groups[d]

    def size(self, dim) -> int:
        d = self.names.index(dim) if isinstance(dim, str) else dim
        return self.shape[d]

    def index(self, dim) -> int:
        d = self.names.index(dim) if isinstance(dim, str) else dim
        return self.coord[d]

    def flatten(self, dims: Sequence) -> Optional[object]:
        """One group over the product of several mesh dimensions (e.g. dp x cp for gradient sync)."""
        ds = [self.names.index(x) if isinstance(x, str) else x for x in dims]
        mine = None
        seen = set()
        for r in range(self.pg.size()):
            c = [(r // self.strides[i]) % self.shape[i] for i in range(len(self.shape))]
            key = tuple(c[i] for i in range(len(self.shape)) if i not in ds)
            if key in seen:
                continue
            seen.add(key)
            ranks = [q for q in range(self.pg.size())
                     if tuple(((q // self.strides[i]) % self.shape[i]) for i in range(len(self.shape)) if i not in ds) == key]
            g = self.pg.new_group(ranks) if len(ranks) > 1 else None
            if self.rank in ranks:
                mine = g
        return mine


class DTensor:
    def __init__(self, local: torch.Tensor, mesh: DeviceMesh, placements: Sequence):
        if len(placements) != len(mesh.shape):
            raise ValueError("one placement per mesh dimension")
        self.local, self.mesh, self.placements = local, mesh, tuple(placements)

    # ----------------------------------------------------------------------------- construction
    @staticmethod
    def from_full(full: torch.Tensor, mesh: DeviceMesh, placements: Sequence) -> "DTensor":
        t = full
        for d, p in enumerate(placements):
            if isinstance(p, Shard):
                t = t.chunk(mesh.shape[d], dim=p.dim)[mesh.coord[d]]
            elif isinstance(p, Partial):
                t = t if mesh.coord[d] == 0 else torch.zeros_like(t)
        return DTensor(t.contiguous(), mesh, placements)

    def full_tensor(self) -> torch.Tensor:
        return self.redistribute([Replicate()] * len(self.placements)).local

    # ----------------------------------------------------------------------------- redistribute
    def redistribute(self, placements: Sequence) -> "DTensor":
        t, cur = self.local, list(self.placements)
        for d, (src, dst) in enumerate(zip(self.placements, placements)):
            if src == dst:
                continue
            g, n, idx = self.mesh.group(d), self.mesh.shape[d], self.mesh.coord[d]
            if n == 1 or g is None:
                cur[d] = dst
                continue
            if isinstance(src, Shard) and isinstance(dst, Replicate):
                t = _all_gather_dim(t, g, src.dim)
            elif isinstance(src, Partial) and isinstance(dst, Replicate):
                t = t.contiguous().clone()
                g.all_reduce_tensor(t, "sum")
            elif isinstance(src, Partial) and isinstance(dst, Shard):
                moved = t.movedim(dst.dim, 0).contiguous()
                out = torch.empty((moved.shape[0] // n,) + tuple(moved.shape[1:]), dtype=t.dtype, device=t.device)
                g.reduce_scatter_tensor(out, moved, "sum")
                t = out.movedim(0, dst.dim).contiguous()
            elif isinstance(src, Shard) and isinstance(dst, Shard):
                parts = [p.contiguous() for p in t.chunk(n, dim=dst.dim)]
                shape = parts[0].shape
                recv = g.all_to_all_v([p.reshape(-1) for p in parts])
                t = torch.cat([r.view(shape) for r in recv], dim=src.dim)
            elif isinstance(src, Replicate) and isinstance(dst, Shard):
                t = t.chunk(n, dim=dst.dim)[idx].contiguous()
            elif isinstance(src, Replicate) and isinstance(dst, Partial):
                t = t if idx == 0 else torch.zeros_like(t)
            elif isinstance(src, Shard) and isinstance(dst, Partial):
                t = _all_gather_dim(t, g, src.dim)
                t = t if idx == 0 else torch.zeros_like(t)
            else:
                raise ValueError(f"unsupported redistribution {src} -> {dst}")
            cur[d] = dst
        return DTensor(t, self.mesh, cur)


def _all_gather_dim(t: torch.Tensor, g, dim: int) -> torch.Tensor:
    moved = t.movedim(dim, 0).contiguous()
    out = torch.empty((moved.shape[0] * g.size(),) + tuple(moved.shape[1:]), dtype=t.dtype, device=t.device)
    g.all_gather_tensor(out, moved)
    return out.movedim(0, dim).contiguous()


# ------------------------------------------------------------------------------- propagation rules
def dt_matmul(a: DTensor, b: DTensor) -> DTensor:
    """a [.., M, K] @ b [K, N].  Per mesh dim: (R,R)->R, (S(row),R)->S(row), (R,S(1))->S(last),
    (S(last),S(0))->Partial; anything else is redistributed to replicated first."""
    nd = a.local.dim()
    out_pl = []
    a2, b2 = a, b
    for d, (pa, pb) in enumerate(zip(a.placements, b.placements)):
        if isinstance(pa, Replicate) and isinstance(pb, Replicate):
            out_pl.append(Replicate())
        elif isinstance(pa, Shard) and pa.dim < nd - 1 and isinstance(pb, Replicate):
            out_pl.append(Shard(pa.dim))
        elif isinstance(pa, Replicate) and isinstance(pb, Shard) and pb.dim == 1:
            out_pl.append(Shard(nd - 1))
        elif isinstance(pa, Shard) and pa.dim == nd - 1 and isinstance(pb, Shard) and pb.dim == 0:
            out_pl.append(Partial())
        else:
            pla, plb = list(a2.placements), list(b2.placements)
            pla[d], plb[d] = Replicate(), Replicate()
            a2, b2 = a2.redistribute(pla), b2.redistribute(plb)
            out_pl.append(Replicate())
    return DTensor(a2.local @ b2.local, a.mesh, out_pl)


def dt_elementwise(fn, *xs: DTensor) -> DTensor:
    """Pointwise op: all inputs must share their placements; Partial inputs are reduced first unless
    the op is linear (``fn.linear = True``)."""
    pl = xs[0].placements
    ys = []
    for x in xs:
        tgt = [Replicate() if (isinstance(p, Partial) and not getattr(fn, "linear", False)) else q
               for p, q in zip(x.placements, pl)]
        tgt = [Replicate() if isinstance(q, Partial) and not getattr(fn, "linear", False) else q for q in tgt]
        ys.append(x.redistribute(tgt))
    return DTensor(fn(*[y.local for y in ys]), xs[0].mesh, ys[0].placements)


def _unshard_dim(x: DTensor, dim: int) -> DTensor:
    d = dim % x.local.dim()
    tgt = [Replicate() if (isinstance(p, Partial) or (isinstance(p, Shard) and p.dim == d)) else p for p in x.placements]
    return x.redistribute(tgt)


def dt_norm(x: DTensor, weight: torch.Tensor, eps: float = 1e-5, rms: bool = True) -> DTensor:
    from ..fused.ops import fused_layernorm, rms_norm
    x = _unshard_dim(x, -1)
    y = rms_norm(x.local, weight, eps) if rms else fused_layernorm(x.local, weight, None, eps)
    return DTensor(y, x.mesh, x.placements)


def dt_softmax(x: DTensor, dim: int = -1) -> DTensor:
    x = _unshard_dim(x, dim)
    return DTensor(torch.softmax(x.local, dim), x.mesh, x.placements)


def dt_embedding(idx: DTensor, table: DTensor) -> DTensor:
    """Vocabulary-sharded table -> Partial output (rows outside the local range contribute zero)."""
    out_pl = []
    local = None
    t = table.local
    for d, (pi, pt) in enumerate(zip(idx.placements, table.placements)):
        if isinstance(pt, Shard) and pt.dim == 0:
            n, r = table.mesh.shape[d], table.mesh.coord[d]
            lo = r * t.shape[0]
            ids = idx.local.long() - lo
            ok = (ids >= 0) & (ids < t.shape[0])
            local = t[ids.clamp(0, t.shape[0] - 1)] * ok[..., None]
            out_pl.append(Partial())
        else:
            out_pl.append(pi if isinstance(pi, Shard) else Replicate())
    if local is None:
        local = t[idx.local.long()]
    return DTensor(local, idx.mesh, out_pl)
