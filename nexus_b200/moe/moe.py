"""Mixture-of-experts core: FP32 router, (noisy) top-k, gate = softmax over the selected k, GShard
capacity per group with (choice, token) priority, Drop / Reroute overflow, counting-sort
permutation, grouped SwiGLU expert GEMMs over capacity-padded buffers, gate-weighted combine,
load-balancing (aux) and router z losses, BF16 / FP8 expert storage, FP64 token-by-token oracle.
The capacity assignment walk and the oracle run in the native host module (`csrc/host/moe_route.cpp`,
`csrc/host/moe_ref.cpp`).

``MoEFFN(x) = sum_j g_j Expert_{e_j}(x)`` with ``Expert(x) = (silu(x W1) * (x W3)) W2``;
``up[e] = [W1 | W3]`` is stored [2F, d] and ``down[e]`` [d, F] (out-major, like every weight here).

On CUDA BF16 inputs the expert GEMMs run as one strided-batched tcgen05 GEMM over the padded
[E, capacity, d] buffers; routing statistics are always FP32.

Parity: include/nexus/moe/moe.hpp:8-138 and src/moe/moe.cpp:94-502 of the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np
import torch
import torch.nn.functional as F


@dataclass
class Spec:
    experts: int = 8
    top_k: int = 2
    d_model: int = 0
    d_ff: int = 0
    capacity_factor: float = 1.25
    min_capacity: int = 4
    overflow: str = "drop"  # "drop" | "reroute"
    groups: int = 1
    noisy: bool = False
    aux_alpha: float = 0.01
    z_alpha: float = 1.0e-3

    def validate(self) -> None:
        if self.experts < 1 or not (1 <= self.top_k <= self.experts) or self.d_model < 1 or self.d_ff < 1:
            raise ValueError("moe.Spec: experts >= 1, 1 <= top_k <= experts, d_model, d_ff >= 1")
        if self.capacity_factor <= 0 or self.groups < 1 or self.min_capacity < 0:
            raise ValueError("moe.Spec: capacity_factor > 0, groups >= 1, min_capacity >= 0")
        if self.overflow not in ("drop", "reroute"):
            raise ValueError("moe.Spec: overflow must be 'drop' or 'reroute'")


@dataclass
class Routing:
    N: int = 0
    capacity: int = 0
    expert: torch.Tensor = None      # [N, k] long (after rerouting)
    gate: torch.Tensor = None        # [N, k] float (differentiable)
    row: torch.Tensor = None         # [N, k] long: row in the permuted buffer, -1 when dropped
    offsets: torch.Tensor = None     # [E + 1] long
    perm_token: torch.Tensor = None  # [rows] long: token of every permuted row
    routed: torch.Tensor = None      # [E] long: assignments per expert before capacity
    prob_sum: torch.Tensor = None    # [E] float64: sum of router probabilities
    lse_sq_sum: float = 0.0
    aux: torch.Tensor = None         # scalar tensors (differentiable)
    z: torch.Tensor = None
    dropped: int = 0
    rerouted: int = 0


def _round_half_away(x: float) -> int:
    return int(math.floor(x + 0.5)) if x >= 0 else -int(math.floor(-x + 0.5))


def capacity_of(spec: Spec, tokens_per_group: int) -> int:
    return max(spec.min_capacity, _round_half_away(spec.top_k * tokens_per_group / spec.experts * spec.capacity_factor))


def route(x: torch.Tensor, router_w: torch.Tensor, noise_w: Optional[torch.Tensor], spec: Spec,
          training: bool = False, seed: int = 0, loss_stats: Optional[dict] = None) -> Routing:
    """x [N, d]; router_w [d, E].  ``loss_stats`` (expert-parallel callers) supplies globally reduced
    ``routed``, ``prob_sum``, ``lse_sq_sum`` and ``tokens`` for the aux / z losses."""
    spec.validate()
    N, E, k = x.shape[0], spec.experts, spec.top_k
    if N % spec.groups != 0:
        raise ValueError(f"token count {N} must be divisible by groups {spec.groups}")
    logits = x.float() @ router_w.float()
    lse = torch.logsumexp(logits, -1)
    probs = torch.softmax(logits, -1)
    select = logits
    if training and spec.noisy and noise_w is not None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        eps = torch.randn(logits.shape, generator=g).to(logits.device)
        select = logits + eps * F.softplus(x.float() @ noise_w.float())
    order = torch.sort(select.detach(), dim=-1, descending=True, stable=True).indices
    expert = order[:, :k].contiguous()
    topv = select.gather(1, expert)
    gate = torch.softmax(topv, -1)
    routed = torch.bincount(expert.reshape(-1), minlength=E)
    r = Routing(N=N, expert=expert, gate=gate, routed=routed)
    r.prob_sum = probs.double().sum(0)
    r.lse_sq_sum = float((lse.detach().double() ** 2).sum())
    # losses on the clean logits; f before capacity
    if loss_stats is None:
        Nl = float(N)
        f = routed.double() / (Nl * k)
        P = probs.double().sum(0) / Nl
        r.aux = (spec.aux_alpha * E * (f.detach() * P).sum()).float()
        r.z = (spec.z_alpha * (lse.double() ** 2).sum() / Nl).float()
    else:
        Nl = float(loss_stats["tokens"])
        f = loss_stats["routed"].double().to(x.device) / (Nl * k)
        # gradient flows through the local probabilities only; the value uses the global sums
        P_local = probs.double().sum(0) / Nl
        P_glob = loss_stats["prob_sum"].double().to(x.device) / Nl
        r.aux = (spec.aux_alpha * E * (f * (P_local + (P_glob - P_local).detach())).sum()).float()
        z_local = (lse.double() ** 2).sum() / Nl
        r.z = (spec.z_alpha * (z_local + (loss_stats["lse_sq_sum"] / Nl - z_local).detach())).float()
    # capacity and acceptance: per group, every first choice before any second choice
    Ng = N // spec.groups
    C = capacity_of(spec, Ng)
    r.capacity = C
    dev = x.device
    # the sequential walk (acceptance in (choice, token) order, reroute search, counting sort) runs in the native module
    from .. import _native
    reroute = spec.overflow != "drop"
    ex, row, offsets, perm, r.dropped, r.rerouted = _native.moe_assign(
        expert.cpu().numpy(), order.cpu().numpy() if reroute else np.zeros((0, 0), dtype=np.int64), E, spec.groups, C, reroute)
    if reroute:
        r.expert = torch.from_numpy(ex).to(dev)
    r.row, r.offsets = torch.from_numpy(row).to(dev), torch.from_numpy(offsets).to(dev)
    perm = torch.from_numpy(perm).to(dev)
    r.perm_token = perm
    return r


def _swiglu(h: torch.Tensor, Fdim: int) -> torch.Tensor:
    return F.silu(h[..., :Fdim]) * h[..., Fdim:]


def experts_forward(xp: torch.Tensor, offsets: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """Grouped expert MLP over the permuted rows xp [rows, d]; up [E, 2F, d], down [E, d, F]."""
    E, twoF, d = up.shape
    Fd = twoF // 2
    counts = (offsets[1:] - offsets[:-1])
    if xp.is_cuda and xp.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and d % 8 == 0 and Fd % 8 == 0:
        from ..fused.batched import batched_linear
        cap = int(counts.max().item()) if counts.numel() else 0
        cap = max(8, (cap + 7) // 8 * 8)
        # scatter the contiguous expert slices into a capacity-padded [E, cap, d] buffer
        idx = torch.arange(xp.shape[0], device=xp.device)
        e_of = torch.bucketize(idx, offsets[1:], right=True)
        slot = idx - offsets[e_of]
        buf = xp.new_zeros((E, cap, d))
        buf[e_of, slot] = xp
        h = batched_linear(buf, up)
        a = _swiglu(h.float(), Fd).to(xp.dtype)
        y = batched_linear(a, down)
        return y[e_of, slot]
    out = xp.new_empty((xp.shape[0], d))
    offs = offsets.tolist()
    for e in range(E):
        lo, hi = offs[e], offs[e + 1]
        if hi > lo:
            h = xp[lo:hi] @ up[e].to(xp.dtype).t()
            out[lo:hi] = _swiglu(h, Fd) @ down[e].to(xp.dtype).t()
    return out


def moe_forward(x: torch.Tensor, router_w, noise_w, up, down, spec: Spec, training: bool = False, seed: int = 0):
    """x [N, d] -> (y [N, d], Routing).  Differentiable w.r.t. x, router, experts."""
    r = route(x, router_w, noise_w, spec, training, seed)
    xp = x[r.perm_token]
    yp = experts_forward(xp, r.offsets, up, down)
    return combine(yp, r, x), r


def combine(yp: torch.Tensor, r: Routing, like: torch.Tensor) -> torch.Tensor:
    """y[t] = sum_j gate[t, j] * yp[row[t, j]] over accepted assignments."""
    N, k = r.row.shape
    ok = r.row >= 0
    rows = r.row.clamp(min=0)
    picked = yp[rows.reshape(-1)].view(N, k, -1)
    w = (r.gate * ok).to(picked.dtype)
    return (picked * w[..., None]).sum(1).to(like.dtype)


def reference(x, router_w, up, down, spec: Spec):
    """FP64 token-by-token oracle (no noise): returns (y, aux, z).  Native and independent of the tensor code above
    (`csrc/host/moe_ref.cpp`: its own router, top-k, capacity / Drop / Reroute walk and expert MLPs)."""
    y, aux, z, _dropped, _rerouted = reference_full(x, router_w, up, down, spec)
    return y, aux, z


def reference_full(x, router_w, up, down, spec: Spec):
    """The oracle with its routing statistics: (y [N, d] FP64, aux, z, dropped, rerouted)."""
    from .. import _native
    spec.validate()
    N = x.shape[0]
    if N % spec.groups:
        raise ValueError(f"token count {N} must be divisible by groups {spec.groups}")
    cap = capacity_of(spec, N // spec.groups)
    np64 = lambda t: t.detach().double().cpu().contiguous().numpy()
    y, aux, z, dropped, rerouted = _native.moe_reference(np64(x), np64(router_w), np64(up), np64(down), spec.top_k,
                                                         spec.groups, cap, spec.overflow == "reroute",
                                                         float(spec.aux_alpha), float(spec.z_alpha))
    return torch.from_numpy(y), float(aux), float(z), int(dropped), int(rerouted)


def quantize_experts(w: torch.Tensor, kind: str):
    """Expert weight storage for inference: 'bf16', 'fp8' (E4M3, one scale = amax/448 per expert) or 'mxfp8'
    (E4M3 with one E8M0 scale per 32 elements along the contraction axis).
    Returns (stored, scales or None); ``dequantize_experts`` restores FP32."""
    if kind == "bf16":
        return w.to(torch.bfloat16), None
    if kind == "fp8":
        amax = w.abs().flatten(1).amax(1).clamp(min=1e-12)
        scale = amax / 448.0
        q = (w / scale.view(-1, *([1] * (w.dim() - 1)))).to(torch.float8_e4m3fn)
        return q, scale
    if kind == "mxfp8":
        # block-scaled: one power-of-two scale per 32 elements of each weight row (the contraction axis), stored per
        # expert in the atom order the block-scaled tensor-core GEMM reads (ops._lowp.mx_gemm takes them as they are)
        from ..ops import _lowp as L
        pairs = [L.mx_quantize(w[e].reshape(-1, w.shape[-1]).contiguous()) for e in range(w.shape[0])]
        q = torch.stack([c for c, _ in pairs]).view(w.shape)
        return q, torch.stack([sc for _, sc in pairs])
    raise ValueError("quantize_experts: kind must be 'bf16', 'fp8' or 'mxfp8'")


def dequantize_experts(q: torch.Tensor, scale: Optional[torch.Tensor]) -> torch.Tensor:
    if scale is not None and scale.dtype == torch.uint8:   # block-scaled storage
        from ..ops import _lowp as L
        rows = q[0].numel() // q.shape[-1]
        return torch.stack([L.mx_dequantize(q[e].reshape(rows, q.shape[-1]), scale[e]) for e in range(q.shape[0])]).view(q.shape)
    w = q.float()
    return w if scale is None else w * scale.view(-1, *([1] * (w.dim() - 1)))


class MoEFFN(torch.nn.Module):
    """Drop-in MoE feed-forward layer; ``forward`` returns y and stores ``last_routing`` (aux, z, stats)."""

    def __init__(self, spec: Spec, init_std: float = 0.02, seed: int = 0, dtype=torch.float32):
        super().__init__()
        spec.validate()
        self.spec = spec
        g = torch.Generator().manual_seed(seed)
        E, d, Fd = spec.experts, spec.d_model, spec.d_ff
        self.router = torch.nn.Parameter(torch.randn(d, E, generator=g) * init_std)
        self.noise = torch.nn.Parameter(torch.zeros(d, E)) if spec.noisy else None
        self.up = torch.nn.Parameter((torch.randn(E, 2 * Fd, d, generator=g) * init_std).to(dtype))
        self.down = torch.nn.Parameter((torch.randn(E, d, Fd, generator=g) * init_std).to(dtype))
        self.last_routing: Optional[Routing] = None
        self.seed = seed
        self.calls = 0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        self.calls += 1
        y, r = moe_forward(x2, self.router, self.noise, self.up, self.down, self.spec, self.training,
                           self.seed + self.calls)
        self.last_routing = r
        return y.view(shape)

    def losses(self) -> torch.Tensor:
        r = self.last_routing
        return r.aux + r.z
