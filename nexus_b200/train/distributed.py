"""Single-process data parallelism over model replicas and the loop profile of the training library:
`allreduce_mean_gradients`, `broadcast_parameters`, `DataParallelStep`, `DataParallelTrainer`, `LoopProfile`,
`all_reduce_mean`.

Replicas are ordinary modules (one per device, or several on the CPU); a step splits the batch into contiguous row
blocks (the first ``rows % replicas`` blocks one row longer), runs forward / loss / backward of every replica on its
own thread, averages the gradients into replica 0, steps the optimizer there and copies the parameters back.  On
CUDA replicas the gradient sum uses NCCL-free device copies (peer access) - the multi-process trainers use
`parallel.ddp` / the fused peer-memory paths instead.

Parity: lib/NexusTrain/include/nexus_train/distributed/{gradient_sync,data_parallel_trainer}.hpp,
lib/NexusTrain/include/nexus_train/core/loop_profile.hpp:18 and include/nexus/train/distributed.hpp:17 of the reference.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch


def _params(replica) -> List[torch.nn.Parameter]:
    return [p for p in replica.parameters()]


def allreduce_mean_gradients(replicas: Sequence[Sequence[torch.nn.Parameter]]) -> None:
    """Mean of the replicas' gradients, written into every replica (parameters without a gradient are skipped)."""
    if not replicas:
        return
    width = len(replicas[0])
    for r in replicas:
        if len(r) != width:
            raise ValueError("replica parameter counts differ")
    inv = 1.0 / len(replicas)
    with torch.no_grad():
        for i in range(width):
            root = replicas[0][i]
            if not root.requires_grad or root.grad is None:
                continue
            acc = root.grad
            for r in replicas[1:]:
                g = r[i].grad
                if g is None or g.numel() != acc.numel():
                    raise ValueError("replica gradient shapes differ")
                acc.add_(g.to(acc.device))
            acc.mul_(inv)
            for r in replicas[1:]:
                r[i].grad.copy_(acc)


def broadcast_parameters(source: Sequence[torch.nn.Parameter], replicas: Sequence[Sequence[torch.nn.Parameter]]) -> None:
    """Copies ``source`` into every replica but the first (which is the source's own replica)."""
    with torch.no_grad():
        for i, s in enumerate(source):
            for r in replicas[1:]:
                if r[i].numel() != s.numel():
                    raise ValueError("replica parameter shapes differ")
                r[i].copy_(s)


def all_reduce_mean(ranks: List[List[float]]) -> List[List[float]]:
    """Element-wise mean over equally long per-rank vectors, written back into every rank (and returned)."""
    if not ranks:
        raise ValueError("all_reduce_mean requires a rank")
    n = len(ranks[0])
    for r in ranks:
        if len(r) != n:
            raise ValueError("all_reduce_mean rank lengths differ")
    mean = torch.tensor(ranks, dtype=torch.float64).mean(0).tolist()
    for r in ranks:
        r[:] = mean
    return ranks


@dataclass
class LoopProfile:
    """Where a training loop's wall time went; `report()` prints seconds and shares of the wall time."""
    data_wait_s: float = 0.0
    forward_s: float = 0.0
    loss_s: float = 0.0
    backward_s: float = 0.0
    optimizer_s: float = 0.0
    callback_s: float = 0.0
    wall_s: float = 0.0
    batches: int = 0
    steps: int = 0

    def report(self) -> str:
        wall = self.wall_s if self.wall_s > 0 else 1e-12
        parts = [f"batches={self.batches} steps={self.steps} wall_s={self.wall_s:.4f}"]
        for name in ("data_wait_s", "forward_s", "loss_s", "backward_s", "optimizer_s", "callback_s"):
            v = getattr(self, name)
            parts.append(f"{name}={v:.4f} ({100.0 * v / wall:.1f}%)")
        return " ".join(parts)


class DataParallelStep:
    """One synchronous data-parallel step over in-process replicas.

    ``loss_fn(prediction, labels) -> (loss value, d loss / d prediction)`` (e.g. ``loss.CrossEntropy().forward_backward``);
    ``optimizer`` steps the parameters of replica 0."""

    def __init__(self, replicas: Sequence[torch.nn.Module], loss_fn: Callable, optimizer):
        if not replicas or loss_fn is None or optimizer is None:
            raise ValueError("data parallel step needs replicas, a loss and an optimizer")
        self.replicas = list(replicas)
        self.loss_fn, self.optimizer = loss_fn, optimizer
        self.parameters = [_params(r) for r in self.replicas]
        broadcast_parameters(self.parameters[0], self.parameters)
        self.profile = LoopProfile()

    def step(self, inputs: torch.Tensor, labels: torch.Tensor) -> float:
        if inputs.dim() < 1 or labels.dim() < 1 or inputs.shape[0] != labels.shape[0]:
            raise ValueError("data parallel batch rows must match")
        t_start = time.perf_counter()
        for r in self.replicas:
            r.zero_grad(set_to_none=False)
        rows, width = inputs.shape[0], len(self.replicas)
        base, extra = divmod(rows, width)
        losses, counts, errors = [0.0] * width, [0] * width, [None] * width
        times = [[0.0, 0.0, 0.0] for _ in range(width)]
        threads, cursor = [], 0

        def work(i, row, count):
            try:
                dev = next(self.replicas[i].parameters()).device
                x, y = inputs[row: row + count].to(dev), labels[row: row + count].to(dev)
                t0 = time.perf_counter()
                pred = self.replicas[i](x)
                t1 = time.perf_counter()
                loss, grad = self.loss_fn(pred, y)
                t2 = time.perf_counter()
                pred.backward(grad.to(pred.dtype))
                t3 = time.perf_counter()
                losses[i] = float(loss)
                times[i] = [t1 - t0, t2 - t1, t3 - t2]
            except BaseException as e:  # re-raised on the caller's thread
                errors[i] = e

        for i in range(width):
            count = base + (1 if i < extra else 0)
            counts[i] = count
            if count:
                th = threading.Thread(target=work, args=(i, cursor, count))
                th.start()
                threads.append(th)
            cursor += count
        for th in threads:
            th.join()
        for e in errors:
            if e is not None:
                raise e
        for p in self.parameters:   # an idle replica contributes zero gradients
            for q in p:
                if q.requires_grad and q.grad is None:
                    q.grad = torch.zeros_like(q)
        t_opt = time.perf_counter()
        allreduce_mean_gradients(self.parameters)
        self.optimizer.step()
        broadcast_parameters(self.parameters[0], self.parameters)
        for r in self.replicas:
            r.zero_grad(set_to_none=False)
        t_end = time.perf_counter()
        pr = self.profile
        pr.forward_s += max(t[0] for t in times)
        pr.loss_s += max(t[1] for t in times)
        pr.backward_s += max(t[2] for t in times)
        pr.optimizer_s += t_end - t_opt
        pr.wall_s += t_end - t_start
        pr.batches += 1
        pr.steps += 1
        seen = sum(counts)
        return sum(l * c for l, c in zip(losses, counts)) / max(seen, 1)


class DataParallelTrainer:
    """Epoch loop around `DataParallelStep`: ``fit(loader, epochs)`` returns the mean loss per epoch; ``profile``
    accumulates the loop's time split (data wait, forward, loss, backward, optimizer, callbacks)."""

    def __init__(self, replicas: Sequence[torch.nn.Module], loss_fn: Callable, optimizer, callbacks: Optional[list] = None):
        self.step_fn = DataParallelStep(replicas, loss_fn, optimizer)
        self.callbacks = list(callbacks or [])
        self.history: List[float] = []

    @property
    def profile(self) -> LoopProfile:
        return self.step_fn.profile

    def fit(self, loader, epochs: int = 1) -> List[float]:
        pr = self.profile
        for epoch in range(epochs):
            total, count = 0.0, 0
            it = iter(loader)
            while True:
                t0 = time.perf_counter()
                try:
                    x, y = next(it)
                except StopIteration:
                    break
                waited = time.perf_counter() - t0
                pr.data_wait_s += waited
                pr.wall_s += waited
                x, y = torch.as_tensor(x), torch.as_tensor(y)
                total += self.step_fn.step(x, y) * len(y)
                count += len(y)
            self.history.append(total / max(count, 1))
            t0 = time.perf_counter()
            stop = False
            for cb in self.callbacks:
                if cb(epoch, self.history[-1]) is False:
                    stop = True
            dt = time.perf_counter() - t0
            pr.callback_s += dt
            pr.wall_s += dt
            if stop:
                break
        return self.history
