"""`ParallelLm` behind the `LmBackend` interface: the trainer's micro-steps become the pipeline's
micro-batches (collected and run on the last one).
Parity: src/train/parallel_backend.cpp of the reference."""
from __future__ import annotations

from typing import List

import numpy as np
import torch

from ..train.lm_trainer import AdamW, LmBackend, LmParamInfo, LmStepResult
from .parallel_lm import ParallelConfig, ParallelLm


class ParallelLmBackend(LmBackend):
    def __init__(self, model, pg, cfg: ParallelConfig, micro_batch: int, seq_len: int, device="cpu"):
        from ..lm.config import LmConfig
        from ..lm.model import LanguageModel
        if isinstance(model, LmConfig):
            model = LanguageModel(model)
        self.pl = ParallelLm(model, pg, cfg)
        self.B, self.T = micro_batch, seq_len
        self._micro: List[torch.Tensor] = []
        self._weights: List[float] = []
        self._loss = float("nan")
        self._norm = float("nan")

    def device(self) -> str: return "cpu"
    def micro_batch(self) -> int: return self.B
    def seq_len(self) -> int: return self.T
    def vocab(self) -> int: return self.pl.mc.vocab_size
    def reshape(self, micro_batch, seq_len): self.B, self.T = micro_batch, seq_len

    def parameters(self) -> List[LmParamInfo]:
        return [LmParamInfo(n, p.numel(), p.dim(), n in ("wte", "wpe")) for n, p in self.pl.params.items()]

    def set_param_scales(self, weight_decay, lr) -> None:
        self._wd = dict(zip(self.pl.names, weight_decay))

    def micro_step(self, tokens: np.ndarray, grad_weight: float, index: int, count: int) -> None:
        if index == 0:
            self._micro, self._weights = [], []
        self._micro.append(torch.from_numpy(np.ascontiguousarray(tokens, dtype=np.int64)))
        self._weights.append(float(grad_weight))
        if index == count - 1:
            self.pl.forward_backward(self._micro, self._weights)
            self._loss = self.pl.local_loss

    def optimizer_step(self, optimizer: AdamW, lr: float, clip: float) -> None:
        wd = getattr(self, "_wd", None)
        self._norm = self.pl.step(optimizer, lr, clip, (lambda n, p: wd[n]) if wd else None)

    def finish_step(self) -> LmStepResult:
        import math
        return LmStepResult(loss=self._loss, grad_norm=self._norm, skipped=not math.isfinite(self._norm))

    def eval_loss(self, tokens: np.ndarray) -> float:
        return self.pl.eval_loss(torch.from_numpy(np.ascontiguousarray(tokens, dtype=np.int64)))

    def token_losses(self, tokens): raise RuntimeError("token_losses is not available on the 4-D backend")
    def save_state(self) -> bytes: return self.pl.save_state()
    def load_state(self, blob: bytes) -> None: self.pl.load_state(blob)
    def data_parallel_group(self): return self.pl.dp_g
    def parallel_model(self): return self.pl
    def state_layout(self) -> str:
        c = self.pl.cfg
        return f"4d:dp{c.dp}:pp{c.pp}:cp{c.cp}:tp{c.tp}"
