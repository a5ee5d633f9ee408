"""Tabular "pixel" classifier: 8 x 8 samples whose class is marked by one of the first three pixels.

An MLP from the nn catalog, trained through ``TrainerBuilder`` with AdamW, label-smoothed cross-entropy, gradient
clipping, accuracy / F1 metrics and early stopping.  Exits non-zero when validation accuracy stays below 0.75.
Counterpart of apps/dl_vision_classifier of the reference.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nexus_b200 import nn  # noqa: E402
from nexus_b200.data import DataLoader  # noqa: E402
from nexus_b200.metrics import Accuracy, F1Score  # noqa: E402
from nexus_b200.train import TrainerBuilder  # noqa: E402
from nexus_b200.train.callbacks import EarlyStopping  # noqa: E402


def samples(count: int, salt: int):
    x = np.zeros((count, 64), dtype=np.float32)
    y = np.zeros(count, dtype=np.int64)
    for i in range(count):
        label = (i + salt) % 3
        y[i] = label
        x[i, label] = 1.0
        x[i, 8 + i % 8] = 0.1
    return x, y


def main(device: str = "cpu") -> int:
    train = DataLoader(*samples(96, 0), batch_size=32, shuffle=True, seed=1)
    val = DataLoader(*samples(32, 2), batch_size=32)
    model = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 3))
    trainer = (TrainerBuilder(model).adamw(lr=0.05, weight_decay=1e-4).loss(0.05).execution_policy(device)
               .gradient_clip_norm(1.0).metric(Accuracy).metric(F1Score(3)).callback(EarlyStopping(8)).build())
    history = trainer.fit(train, val, 8)
    last = history[-1]
    print(f"val_acc={last.metrics.get('accuracy', float('nan')):.3f} val_f1={last.metrics.get('f1', float('nan')):.3f} "
          f"train_loss={last.train_loss:.4f}")
    return 0 if last.metrics.get("accuracy", 0.0) >= 0.75 else 1


if __name__ == "__main__":
    sys.exit(main(sys.argv[1] if len(sys.argv) > 1 else "cpu"))
