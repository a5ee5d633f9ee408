"""Context parallelism for long sequences: ring attention (contiguous or zigzag layout, K/V blocks
circulate while the local block is processed, partial outputs merged through their log-sum-exp,
causal blocks skipped) and Ulysses (all-to-all heads <-> sequence around a local attention).

Zigzag layout: the sequence is cut into ``2*cp`` chunks and rank r holds chunks ``{r, 2cp-1-r}`` so
that causal work is balanced.  Merge rule: ``lse = log(e^l1 + e^l2)``,
``o = o1*e^(l1-lse) + o2*e^(l2-lse)``.  Backward circulates K/V together with the dK/dV
accumulators, which arrive back at their owner after a full turn.

Parity: include/nexus/dist/context_parallel.hpp:8-75 and src/dist/context_parallel.cpp:73-298 of the reference.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from .collectives import all_to_all


def chunk_ids(cp: int, rank: int, layout: str = "zigzag") -> List[int]:
    """Global chunk ids held by ``rank`` (1 chunk for 'contiguous', 2 for 'zigzag')."""
    if layout == "contiguous":
        return [rank]
    if layout == "zigzag":
        return [rank, 2 * cp - 1 - rank]
    raise ValueError(f"unknown cp layout '{layout}'")


def shard_sequence(x: torch.Tensor, cp: int, rank: int, layout: str = "zigzag", dim: int = 1) -> torch.Tensor:
    n = cp if layout == "contiguous" else 2 * cp
    chunks = x.chunk(n, dim=dim)
    return torch.cat([chunks[i] for i in chunk_ids(cp, rank, layout)], dim=dim)


def unshard_sequence(parts: List[torch.Tensor], cp: int, layout: str = "zigzag", dim: int = 1) -> torch.Tensor:
    """Inverse of `shard_sequence` given every rank's shard (test helper / final gather)."""
    n = cp if layout == "contiguous" else 2 * cp
    out: List[Optional[torch.Tensor]] = [None] * n
    for r, p in enumerate(parts):
        ids = chunk_ids(cp, r, layout)
        for c, piece in zip(ids, p.chunk(len(ids), dim=dim)):
            out[c] = piece
    return torch.cat(out, dim=dim)


def _block_attention(q, k, v, scale, mode: str):
    """q [B,Tq,H,D], k/v [B,Tk,Hkv,D]; mode 'full' | 'causal' (diagonal block).  Returns (o, lse[B,H,Tq]) in FP32."""
    B, Tq, H, D = q.shape
    Hkv = k.shape[2]
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    if Hkv != H:
        kf = kf.repeat_interleave(H // Hkv, 1)
        vf = vf.repeat_interleave(H // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    if mode == "causal":
        Tk = k.shape[1]
        mask = torch.triu(torch.ones(Tq, Tk, dtype=torch.bool, device=q.device), diagonal=1)
        s = s.masked_fill(mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ vf
    return o.permute(0, 2, 1, 3), lse


def merge_partial(o1, l1, o2, l2):
    """Combine two partial attention results over disjoint key sets."""
    lse = torch.logaddexp(l1, l2)
    w1 = torch.exp(l1 - lse).permute(0, 2, 1)[..., None]
    w2 = torch.exp(l2 - lse).permute(0, 2, 1)[..., None]
    return o1 * w1 + o2 * w2, lse


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, pg, layout, scale):
        cp, r = pg.size(), pg.rank()
        my = chunk_ids(cp, r, layout)
        nch = len(my)
        qs, B = q.chunk(nch, dim=1), q.shape[0]
        out = [None] * nch
        lses = [None] * nch
        kv = torch.stack([k, v]).contiguous()
        for step in range(cp):
            owner = (r - step) % cp
            their = chunk_ids(cp, owner, layout)
            ks, vs = kv[0].chunk(nch, dim=1), kv[1].chunk(nch, dim=1)
            nxt = torch.empty_like(kv)
            work = None
            if step + 1 < cp:  # pass the block on while computing with it
                pg.send_recv(kv, (r + 1) % cp, nxt, (r - 1) % cp, tag=step)
            for i, gi in enumerate(my):
                for j, gj in enumerate(their):
                    if gj > gi:
                        continue  # entirely in the future
                    o, l = _block_attention(qs[i], ks[j], vs[j], scale, "causal" if gj == gi else "full")
                    if out[i] is None:
                        out[i], lses[i] = o, l
                    else:
                        out[i], lses[i] = merge_partial(out[i], lses[i], o, l)
            if step + 1 < cp:
                kv = nxt
        o = torch.cat(out, dim=1)
        lse = torch.cat(lses, dim=2)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cfg = (pg, layout, scale)
        return o.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        pg, layout, scale = ctx.cfg
        cp, r = pg.size(), pg.rank()
        my = chunk_ids(cp, r, layout)
        nch = len(my)
        dof = do.float()
        dsum = (dof * o).sum(-1).permute(0, 2, 1)  # [B,H,T]
        qs, dos = q.chunk(nch, dim=1), dof.chunk(nch, dim=1)
        lss, dss = lse.chunk(nch, dim=2), dsum.chunk(nch, dim=2)
        dq = [torch.zeros_like(x, dtype=torch.float32) for x in qs]
        H, Hkv = q.shape[2], k.shape[2]
        # the travelling packet: K, V and their gradient accumulators
        pack = torch.stack([k.float(), v.float(), torch.zeros_like(k, dtype=torch.float32),
                            torch.zeros_like(v, dtype=torch.float32)]).contiguous()
        for step in range(cp):
            owner = (r - step) % cp
            their = chunk_ids(cp, owner, layout)
            ks, vs = pack[0].chunk(nch, dim=1), pack[1].chunk(nch, dim=1)
            dks, dvs = list(pack[2].chunk(nch, dim=1)), list(pack[3].chunk(nch, dim=1))
            for i, gi in enumerate(my):
                for j, gj in enumerate(their):
                    if gj > gi:
                        continue
                    qf = qs[i].float().permute(0, 2, 1, 3)
                    kf, vf = ks[j].permute(0, 2, 1, 3), vs[j].permute(0, 2, 1, 3)
                    if Hkv != H:
                        kf, vf = kf.repeat_interleave(H // Hkv, 1), vf.repeat_interleave(H // Hkv, 1)
                    s = qf @ kf.transpose(-1, -2) * scale
                    if gj == gi:
                        T = s.shape[-1]
                        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=s.device), 1), float("-inf"))
                    p = torch.exp(s - lss[i][..., None])
                    dof_i = dos[i].permute(0, 2, 1, 3)
                    dv_full = p.transpose(-1, -2) @ dof_i
                    dp = dof_i @ vf.transpose(-1, -2)
                    ds = p * (dp - dss[i][..., None]) * scale
                    dq[i] += (ds @ kf).permute(0, 2, 1, 3)
                    dk_full = ds.transpose(-1, -2) @ qf
                    if Hkv != H:
                        g = H // Hkv
                        dk_full = dk_full.view(dk_full.shape[0], Hkv, g, *dk_full.shape[2:]).sum(2)
                        dv_full = dv_full.view(dv_full.shape[0], Hkv, g, *dv_full.shape[2:]).sum(2)
                    dks[j] += dk_full.permute(0, 2, 1, 3)
                    dvs[j] += dv_full.permute(0, 2, 1, 3)
            # forward the packet; after cp hops every packet is back at its owner
            nxt = torch.empty_like(pack)
            pg.send_recv(pack, (r + 1) % cp, nxt, (r - 1) % cp, tag=100 + step)
            pack = nxt
        return (torch.cat(dq, dim=1).to(q.dtype), pack[2].to(k.dtype), pack[3].to(v.dtype), None, None, None)


def ring_attention(q, k, v, pg, layout: str = "zigzag", scale: Optional[float] = None):
    """Causal attention over a sequence sharded across ``pg`` (each rank passes its local shard)."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    if pg is None or pg.size() == 1:
        from ..fused.ops import attention
        return attention(q, k, v, causal=True, scale=scale)
    return _RingAttention.apply(q, k, v, pg, layout, scale)


def ulysses_attention(q, k, v, pg, scale: Optional[float] = None):
    """[B, T/cp, H, D] -> all-to-all -> [B, T, H/cp, D] -> local causal attention -> all-to-all back.
    Needs a contiguous sequence layout and ``H % cp == 0 and Hkv % cp == 0``."""
    from ..fused.ops import attention
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    if pg is None or pg.size() == 1:
        return attention(q, k, v, causal=True, scale=scale)
    cp = pg.size()
    if q.shape[2] % cp or k.shape[2] % cp:
        raise ValueError("ulysses_attention: heads and kv heads must be divisible by cp")
    qa, ka, va = (all_to_all(t, pg, 2, 1) for t in (q, k, v))
    o = attention(qa.contiguous(), ka.contiguous(), va.contiguous(), causal=True, scale=scale)
    return all_to_all(o, pg, 1, 2)
