"""Streaming metrics: `Accuracy`, `F1Score`, `ConfusionMatrix`, `PrecisionRecallF1`.
Parity: include/nexus/metrics and lib/NexusTrain metrics of the reference."""
from __future__ import annotations

import torch


class Accuracy:
    name = "accuracy"

    def __init__(self): self.reset()
    def reset(self): self.correct, self.total = 0, 0

    def update(self, logits: torch.Tensor, target: torch.Tensor):
        pred = logits.argmax(-1) if logits.dim() > 1 else (logits > 0).long()
        self.correct += int((pred == target.long()).sum())
        self.total += int(target.numel())

    def value(self) -> float: return self.correct / max(self.total, 1)


class ConfusionMatrix:
    name = "confusion"

    def __init__(self, classes: int):
        self.classes = classes
        self.reset()

    def reset(self): self.m = torch.zeros(self.classes, self.classes, dtype=torch.long)

    def update(self, logits, target):
        pred = logits.argmax(-1).cpu()
        for t, p in zip(target.long().cpu().tolist(), pred.tolist()):
            self.m[t, p] += 1

    def value(self): return self.m.clone()


class PrecisionRecallF1(ConfusionMatrix):
    name = "prf1"

    def value(self):
        tp = self.m.diag().float()
        prec = tp / self.m.sum(0).clamp(min=1)
        rec = tp / self.m.sum(1).clamp(min=1)
        f1 = 2 * prec * rec / (prec + rec).clamp(min=1e-12)
        return {"precision": float(prec.mean()), "recall": float(rec.mean()), "f1": float(f1.mean())}


class F1Score(PrecisionRecallF1):
    name = "f1"

    def value(self) -> float: return super().value()["f1"]
