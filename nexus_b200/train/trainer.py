"""Classification trainer: ``TrainerBuilder(model).adamw(...).loss(...).metric(...).build().fit(train, val, epochs)``.

Per batch: zero_grad -> forward -> loss forward+backward (label smoothing) -> (loss scale) -> every
``gradient_accumulation`` batches: scale 1/window -> unscale + finite check -> global-norm clip ->
step schedule -> optimizer step.  Mixed precision uses a simple loss scaler (initial 128, halved on
overflow, the step is skipped).  ``save_nxs`` writes layers + weights + optimizer state + trainer
record (history, early-stopping state) into one NXS2 file.

Parity: include/nexus/train/trainer.hpp:86-466 and lib/NexusTrain (callbacks, metrics) of the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..loss import CrossEntropy
from ..metrics import Accuracy
from ..optim import SGD, AdamW


@dataclass
class EpochStats:
    epoch: int
    train_loss: float
    val_loss: float
    metrics: Dict[str, float] = field(default_factory=dict)
    skipped_steps: int = 0
    lr: float = 0.0


class LossScaler:
    def __init__(self, init: float = 128.0, backoff: float = 0.5, min_scale: float = 1.0):
        self.scale, self.backoff, self.min_scale = init, backoff, min_scale
        self.overflows = 0

    def on_overflow(self) -> None:
        self.scale = max(self.min_scale, self.scale * self.backoff)
        self.overflows += 1


class TrainerBuilder:
    def __init__(self, model):
        self._model = model
        self._opt_factory = lambda params: AdamW(params, lr=1e-3)
        self._loss = CrossEntropy(0.0)
        self._device = "cpu"
        self._mixed = False
        self._clip = 0.0
        self._metrics: List = []
        self._callbacks: List = []
        self._accum = 1
        self._step_schedule = None
        self._epoch_schedule = None

    def optimizer(self, factory: Callable): self._opt_factory = factory; return self
    def adamw(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        self._opt_factory = lambda p: AdamW(p, lr, beta1, beta2, eps, weight_decay)
        return self
    def sgd(self, lr=1e-2, momentum=0.0, weight_decay=0.0):
        self._opt_factory = lambda p: SGD(p, lr, momentum, weight_decay)
        return self
    def loss(self, loss_or_smoothing=0.0):
        self._loss = CrossEntropy(float(loss_or_smoothing)) if isinstance(loss_or_smoothing, (int, float)) else loss_or_smoothing
        return self
    def execution_policy(self, device: str): self._device = device; return self
    def mixed_precision(self, on: bool = True): self._mixed = on; return self
    def gradient_clip_norm(self, c: float): self._clip = c; return self
    def metric(self, m): self._metrics.append(m() if isinstance(m, type) else m); return self
    def callback(self, c): self._callbacks.append(c() if isinstance(c, type) else c); return self
    def gradient_accumulation(self, n: int): self._accum = max(1, int(n)); return self
    def step_schedule(self, s): self._step_schedule = s; return self
    def learning_rate_schedule(self, s): self._epoch_schedule = s; return self
    def build(self) -> "Trainer": return Trainer(self)


class Trainer:
    def __init__(self, b: TrainerBuilder):
        self.model = b._model.to(b._device)
        self.device = torch.device(b._device)
        self.optimizer = b._opt_factory(list(self.model.parameters()))
        self.loss_fn, self.metrics, self.callbacks = b._loss, b._metrics or [Accuracy()], b._callbacks
        self.clip, self.accum = b._clip, b._accum
        self.step_schedule, self.epoch_schedule = b._step_schedule, b._epoch_schedule
        self.mixed = b._mixed
        self.scaler = LossScaler() if b._mixed else None
        self.history: List[EpochStats] = []
        self.epoch = 0
        self.global_step = 0
        self.best = float("inf")
        self.should_stop = False
        self.skipped_steps = 0
        self.base_lr = self.optimizer.lr

    # ---------------------------------------------------------------------------------- epochs
    def _run_epoch(self, loader, train: bool) -> Tuple[float, Dict[str, float]]:
        self.model.train(train)
        for m in self.metrics:
            m.reset()
        total, count, window = 0.0, 0, 0
        if train:
            self.optimizer.zero_grad()
        for x, y in loader:
            x = torch.as_tensor(x).to(self.device)
            y = torch.as_tensor(y).to(self.device)
            with torch.set_grad_enabled(train):
                if self.mixed and self.device.type == "cuda":
                    with torch.autocast("cuda", dtype=torch.bfloat16):
                        out = self.model(x)
                else:
                    out = self.model(x)
                loss, grad = self.loss_fn.forward_backward(out.float(), y) if train else (self.loss_fn.forward(out.float(), y), None)
            if train:
                scale = self.scaler.scale if self.scaler else 1.0
                self.model.backward(grad.to(out.dtype) * scale) if hasattr(self.model, "backward") and \
                    getattr(self.model, "_last_out", None) is not None else out.backward(grad.to(out.dtype) * scale)
                window += 1
                if window == self.accum:
                    self._apply_step(window)
                    window = 0
            total += float(loss) * len(y)
            count += len(y)
            for m in self.metrics:
                m.update(out.detach().float(), y)
        if train and window:
            self._apply_step(window)
        return total / max(count, 1), {m.name: m.value() for m in self.metrics}

    def _apply_step(self, window: int) -> None:
        params = [p for p in self.model.parameters() if p.grad is not None]
        inv = 1.0 / (window * (self.scaler.scale if self.scaler else 1.0))
        for p in params:
            p.grad.mul_(inv)
        sq = sum(float(p.grad.double().pow(2).sum()) for p in params)
        if not math.isfinite(sq):
            if self.scaler:
                self.scaler.on_overflow()
            self.skipped_steps += 1
            self.optimizer.zero_grad()
            return
        if self.clip > 0:
            coef = min(1.0, self.clip / (math.sqrt(sq) + 1e-6))
            if coef < 1.0:
                for p in params:
                    p.grad.mul_(coef)
        if self.step_schedule is not None:
            self.optimizer.lr = self.base_lr * self.step_schedule.factor(self.global_step)
        self.optimizer.step()
        self.optimizer.zero_grad()
        self.global_step += 1

    def fit(self, train, val=None, epochs: int = 1) -> List[EpochStats]:
        for _ in range(epochs):
            if self.should_stop:
                break
            tl, _ = self._run_epoch(train, True)
            vl, mets = self._run_epoch(val, False) if val is not None else (float("nan"), {})
            st = EpochStats(self.epoch, tl, vl, mets, self.skipped_steps, self.optimizer.lr)
            self.history.append(st)
            self.epoch += 1
            if self.epoch_schedule is not None:
                self.optimizer.lr = self.base_lr * self.epoch_schedule.factor(self.epoch)
            monitored = vl if val is not None else tl
            self.best = min(self.best, monitored)
            for cb in self.callbacks:
                if cb.on_epoch_end(self, st) is False:
                    self.should_stop = True
        return self.history

    def evaluate(self, loader) -> Tuple[float, Dict[str, float]]:
        return self._run_epoch(loader, False)

    # ------------------------------------------------------------------------------ persistence
    def save_nxs(self, path: str) -> None:
        from ..nxs.archive import optim_record, save_model, trainer_record
        o = self.optimizer
        optim = optim_record(o.algorithm, o.steps, [o.lr], o.state_tensors(), o.scalars())
        last = self.history[-1] if self.history else None
        mets = dict(last.metrics) if last else {}
        for i, h in enumerate(self.history):
            mets[f"history.{i}.train_loss"] = h.train_loss
            mets[f"history.{i}.val_loss"] = h.val_loss
        for cb in self.callbacks:
            mets.update({f"callback.{type(cb).__name__}.{k}": v for k, v in cb.state().items()})
        tr = trainer_record(self.epoch, self.global_step, last.train_loss if last else float("nan"), self.best,
                            self.should_stop, mets)
        save_model(self.model, path, optim=optim, trainer=tr)

    def load_nxs(self, path: str) -> None:
        from ..nxs.archive import _load_weights, load_archive
        a = load_archive(path)
        _load_weights(self.model, a["weights"])
        if a.get("optim"):
            o = a["optim"]
            self.optimizer.load_state(o["step"], o["lr"][0], o["blobs"], o["scalars"])
        if a.get("trainer"):
            t = a["trainer"]
            self.epoch, self.global_step, self.best, self.should_stop = t["epoch"], t["global_step"], t["best"], t["stop"]
            mets = dict(t["metrics"])
            for cb in self.callbacks:
                pre = f"callback.{type(cb).__name__}."
                cb.load_state({k[len(pre):]: v for k, v in mets.items() if k.startswith(pre)})
