"""Trainer callbacks: `EarlyStopping`, `ProgressLogger`, `ModelCheckpoint`, `LRScheduler`.
``on_epoch_end`` returning ``False`` stops training.  Parity: lib/NexusTrain callbacks of the reference."""
from __future__ import annotations

import math


class Callback:
    def on_epoch_end(self, trainer, stats): return True
    def state(self) -> dict: return {}
    def load_state(self, d: dict) -> None: pass


class EarlyStopping(Callback):
    def __init__(self, patience: int = 3, min_delta: float = 0.0):
        self.patience, self.min_delta = patience, min_delta
        self.best, self.bad = float("inf"), 0

    def on_epoch_end(self, trainer, stats):
        v = stats.val_loss if not math.isnan(stats.val_loss) else stats.train_loss
        if v < self.best - self.min_delta:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
        return self.bad < self.patience

    def state(self): return {"best": self.best, "bad": float(self.bad)}

    def load_state(self, d):
        self.best, self.bad = d.get("best", self.best), int(d.get("bad", self.bad))


class ProgressLogger(Callback):
    def __init__(self, every: int = 1): self.every = every

    def on_epoch_end(self, trainer, stats):
        if stats.epoch % self.every == 0:
            print(f"epoch {stats.epoch}: train {stats.train_loss:.4f} val {stats.val_loss:.4f} {stats.metrics}", flush=True)
        return True


class ModelCheckpoint(Callback):
    def __init__(self, path: str, best_only: bool = True):
        self.path, self.best_only, self.best = path, best_only, float("inf")

    def on_epoch_end(self, trainer, stats):
        v = stats.val_loss if not math.isnan(stats.val_loss) else stats.train_loss
        if not self.best_only or v < self.best:
            self.best = min(self.best, v)
            trainer.save_nxs(self.path)
        return True


class LRScheduler(Callback):
    def __init__(self, schedule): self.schedule = schedule

    def on_epoch_end(self, trainer, stats):
        trainer.optimizer.lr = trainer.base_lr * self.schedule.factor(stats.epoch + 1)
        return True
