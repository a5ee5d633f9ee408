"""Data parallelism: gradient buckets in backward-ready order, reduced while backward still runs.

Buckets (25 MiB by default) are planned from the order in which gradients became ready in the first
step and rebuilt once after it; each bucket is flattened, optionally compressed to BF16, SUM-reduced
asynchronously (hierarchically when asked) as soon as its last gradient arrives, and copied back
before the optimizer step.  ``no_sync`` (``backward_context(False)``) skips communication during
accumulation; ``find_unused_parameters`` reduces zeros for parameters that produced no gradient.
`DdpStepStats` records when the first bucket started relative to backward — the overlap evidence.

Parity: include/nexus/dist/ddp.hpp:36-110 and src/dist/ddp.cpp of the reference.
"""
from __future__ import annotations

import contextlib
import math
import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class DdpOptions:
    bucket_bytes: int = 25 * 1024 * 1024
    overlap: bool = True
    bf16_compress: bool = False
    find_unused_parameters: bool = False
    hierarchical_local_size: int = 0
    lr_scaling: str = "none"  # "none" | "linear" | "sqrt"


@dataclass
class DdpStepStats:
    buckets: int = 0
    bytes: int = 0
    backward_ms: float = 0.0
    first_comm_start_ms: float = float("nan")
    comm_wait_ms: float = 0.0


def scaled_lr(base_lr: float, world: int, rule: str) -> float:
    if rule == "linear":
        return base_lr * world
    if rule == "sqrt":
        return base_lr * math.sqrt(world)
    return base_lr


def plan_buckets(sizes_bytes: List[int], order: List[int], bucket_bytes: int) -> List[List[int]]:
    """Groups parameter indices (visited in ``order``) into buckets of at most ``bucket_bytes``."""
    buckets, cur, cur_b = [], [], 0
    for i in order:
        if cur and cur_b + sizes_bytes[i] > bucket_bytes:
            buckets.append(cur)
            cur, cur_b = [], 0
        cur.append(i)
        cur_b += sizes_bytes[i]
    if cur:
        buckets.append(cur)
    return buckets


class DdpEngine:
    def __init__(self, params: List[torch.Tensor], group, options: Optional[DdpOptions] = None):
        self.params, self.pg, self.o = list(params), group, options or DdpOptions()
        self.sizes = [p.numel() * 4 for p in self.params]
        self.order = list(reversed(range(len(self.params))))  # first guess: reverse registration order
        self.buckets = plan_buckets(self.sizes, self.order, self.o.bucket_bytes)
        self._rebuilt = False
        self._ready_order: List[int] = []
        self._sync = True
        self._pending = []
        self._bucket_left: List[int] = []
        self._bucket_of = {}
        self._t0 = 0.0
        self.stats = DdpStepStats()
        self._index_buckets()
        for i, p in enumerate(self.params):
            if p.requires_grad:
                p.register_post_accumulate_grad_hook(lambda t, i=i: self._on_grad(i))

    def _index_buckets(self):
        self._bucket_of = {i: b for b, idxs in enumerate(self.buckets) for i in idxs}

    @contextlib.contextmanager
    def backward_context(self, sync: bool):
        """Wrap ``loss.backward()``; ``sync=False`` is the ``no_sync`` accumulation mode."""
        self._sync = sync
        self._ready_order = []
        self._bucket_left = [len(b) for b in self.buckets]
        self._pending = []
        self._t0 = time.perf_counter()
        self.stats = DdpStepStats(buckets=len(self.buckets), bytes=sum(self.sizes))
        try:
            yield
        finally:
            self.stats.backward_ms = (time.perf_counter() - self._t0) * 1e3
            if sync:
                seen = set(self._ready_order)
                for i, p in enumerate(self.params):  # parameters that produced no gradient
                    if i not in seen and p.requires_grad:
                        if self.o.find_unused_parameters and p.grad is None:
                            p.grad = torch.zeros_like(p)
                        if p.grad is not None:
                            self._on_grad(i, late=True)

    def _on_grad(self, i: int, late: bool = False) -> None:
        if not self._sync or (i in self._ready_order):
            return
        self._ready_order.append(i)
        b = self._bucket_of[i]
        self._bucket_left[b] -= 1
        if self._bucket_left[b] == 0 and (self.o.overlap or late):
            self._launch(b)

    def _launch(self, b: int) -> None:
        idxs = [i for i in self.buckets[b] if self.params[i].grad is not None]
        if not idxs:
            return
        dt = torch.bfloat16 if self.o.bf16_compress else torch.float32
        flat = torch.cat([self.params[i].grad.reshape(-1).to(dt) for i in idxs])
        if math.isnan(self.stats.first_comm_start_ms):
            self.stats.first_comm_start_ms = (time.perf_counter() - self._t0) * 1e3
        if self.o.hierarchical_local_size > 1:
            self.pg.all_reduce_hierarchical(flat, self.o.hierarchical_local_size, "sum")
            work = None
        elif hasattr(self.pg, "all_reduce_async"):
            work = self.pg.all_reduce_async(flat, "sum")
        else:
            self.pg.all_reduce_tensor(flat, "sum")
            work = None
        self._pending.append((idxs, flat, work))

    def finish(self) -> None:
        """Waits for every bucket and writes the reduced gradients back (called before the optimizer)."""
        t = time.perf_counter()
        for b, left in enumerate(self._bucket_left):
            if self._sync and left == 0 and not any(set(self.buckets[b]) & set(p[0]) for p in self._pending):
                self._launch(b)
        for idxs, flat, work in self._pending:
            if work is not None:
                work.wait()
            off = 0
            for i in idxs:
                g = self.params[i].grad
                g.copy_(flat[off: off + g.numel()].view(g.shape).to(g.dtype))
                off += g.numel()
        self._pending = []
        self.stats.comm_wait_ms = (time.perf_counter() - t) * 1e3
        if not self._rebuilt and self._ready_order:
            # rebuild once from the observed ready order (every rank observes the same order)
            rest = [i for i in range(len(self.params)) if i not in self._ready_order]
            self.order = self._ready_order + rest
            self.buckets = plan_buckets(self.sizes, self.order, self.o.bucket_bytes)
            self._index_buckets()
            self._rebuilt = True
