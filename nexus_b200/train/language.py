"""Legacy `LanguageTrainer`: ``fit(TokenRows{values, batch, time}, epochs)`` on top of the LM trainer
with fixed rows, AdamW(lr, 0.9, 0.999, 1e-8, wd) decaying every parameter, constant LR, no clipping.
Parity: include/nexus/train/language.hpp:36-93 of the reference."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch

from .lm_trainer import AdamW, ArrayTokens, LanguageTrainerBuilder, ParamGroupPolicy


@dataclass
class TokenRows:
    values: Sequence[int]
    batch: int
    time: int


class SequenceLm(torch.nn.Module):
    """Gives a plain layer stack (token ids -> logits, e.g. ``Sequential(Embedding, PositionalEncoding,
    CausalTransformerBlock, Linear)``) the interface the LM trainer drives: `logits(tokens)` and the shifted
    next-token `loss(tokens)`.  The wrapped stack's parameters are trained in place."""

    def __init__(self, net: torch.nn.Module):
        super().__init__()
        self.net = net

    def logits(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.net(tokens.long())

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.logits(tokens)

    def loss(self, tokens: torch.Tensor) -> torch.Tensor:
        lg = self.logits(tokens).float()
        return torch.nn.functional.cross_entropy(lg[:, :-1].reshape(-1, lg.shape[-1]), tokens[:, 1:].reshape(-1).long())


class LanguageTrainer:
    def __init__(self, model, lr: float = 3e-4, weight_decay: float = 0.0, device: str = "cpu"):
        if not hasattr(model, "loss"):
            model = SequenceLm(model)
        self.model, self.lr, self.wd, self.device = model, lr, weight_decay, device
        self.losses: List[float] = []
        self._trainer = None

    def fit(self, rows: TokenRows, epochs: int = 1) -> List[float]:
        vals = np.asarray(rows.values, dtype=np.int32)
        per = rows.batch * rows.time
        if len(vals) < per:
            raise ValueError("LanguageTrainer: fewer tokens than one batch")
        steps = max(1, len(vals) // per)
        if self._trainer is None:
            self._trainer = (LanguageTrainerBuilder(self.model).data(ArrayTokens(vals))
                             .optimizer(AdamW(self.lr, 0.9, 0.999, 1e-8, self.wd), ParamGroupPolicy(decay="all"))
                             .micro_batch(rows.batch).seq_len(rows.time).global_batch_tokens(per).grad_clip(0.0)
                             .precision("f32").execution_policy(self.device).log_every(0).build())
        for _ in range(epochs):
            n0 = len(self._trainer.history)
            self._trainer.train(steps)
            ep = self._trainer.history[n0:]
            self.losses.append(float(np.mean([r.loss for r in ep])))
        return self.losses
