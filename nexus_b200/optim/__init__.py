"""Optimizers and schedulers of the facade: `AdamW`, `SGD`, `CosineAnnealing`, `LinearWarmup`,
`OneCycle`.  AdamW uses the shared no-FMA op order of `fused.ops.adamw_multi_tensor`.
Parity: include/nexus/optim of the reference."""
from __future__ import annotations

import math
from typing import List

import numpy as np
import torch

from ..fused.ops import adamw_multi_tensor


class AdamW:
    algorithm = "adamw"

    def __init__(self, params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        self.params = [p for p in params]
        self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = lr, beta1, beta2, eps, weight_decay
        self.m = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.v = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.steps = 0

    def zero_grad(self):
        for p in self.params:
            p.grad = None

    def step(self):
        idx = [i for i, p in enumerate(self.params) if p.grad is not None]
        if not idx:
            return
        self.steps += 1
        adamw_multi_tensor([self.params[i].data for i in idx], [self.params[i].grad for i in idx],
                           [self.m[i] for i in idx], [self.v[i] for i in idx], self.steps, self.lr, self.beta1,
                           self.beta2, self.eps, self.weight_decay, 0.0)

    def state_tensors(self) -> List[torch.Tensor]:
        return list(self.m) + list(self.v)

    def scalars(self) -> List[float]:
        return [self.beta1, self.beta2, self.eps, self.weight_decay]

    def load_state(self, step, lr, blobs, scalars):
        self.steps, self.lr = int(step), float(lr)
        n = len(self.params)
        for t, b in zip(self.m + self.v, blobs[: 2 * n]):
            t.copy_(torch.from_numpy(np.frombuffer(b, dtype=np.float32).copy()).view(t.shape))
        if len(scalars) >= 4:
            self.beta1, self.beta2, self.eps, self.weight_decay = scalars[:4]


class SGD:
    algorithm = "sgd"

    def __init__(self, params, lr=1e-2, momentum=0.0, weight_decay=0.0):
        self.params = [p for p in params]
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.buf = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.steps = 0

    def zero_grad(self):
        for p in self.params:
            p.grad = None

    def step(self):
        self.steps += 1
        with torch.no_grad():
            for p, b in zip(self.params, self.buf):
                if p.grad is None:
                    continue
                g = p.grad.float() + self.weight_decay * p.float()
                if self.momentum > 0:
                    b.mul_(self.momentum).add_(g)
                    g = b
                p.sub_((self.lr * g).to(p.dtype))

    def state_tensors(self): return list(self.buf)
    def scalars(self): return [self.momentum, self.weight_decay]

    def load_state(self, step, lr, blobs, scalars):
        self.steps, self.lr = int(step), float(lr)
        for t, b in zip(self.buf, blobs):
            t.copy_(torch.from_numpy(np.frombuffer(b, dtype=np.float32).copy()).view(t.shape))


class CosineAnnealing:
    def __init__(self, total: int, min_ratio: float = 0.0):
        self.total, self.min_ratio = max(1, total), min_ratio

    def factor(self, step: int) -> float:
        r = min(1.0, step / self.total)
        return self.min_ratio + 0.5 * (1 + math.cos(math.pi * r)) * (1 - self.min_ratio)


class LinearWarmup:
    def __init__(self, warmup: int):
        self.warmup = max(1, warmup)

    def factor(self, step: int) -> float:
        return min(1.0, (step + 1) / self.warmup)


class OneCycle:
    def __init__(self, total: int, pct_start: float = 0.3, div: float = 25.0, final_div: float = 1e4):
        self.total, self.pct, self.div, self.final = max(2, total), pct_start, div, final_div

    def factor(self, step: int) -> float:
        up = self.pct * self.total
        if step < up:
            return 1 / self.div + (1 - 1 / self.div) * step / up
        r = min(1.0, (step - up) / max(1.0, self.total - up))
        lo = 1 / (self.div * self.final)
        return lo + 0.5 * (1 + math.cos(math.pi * r)) * (1 - lo)
