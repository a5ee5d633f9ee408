"""Global configuration: seed and execution policy.  Parity: include/nexus/core/config.hpp:15-47."""
from __future__ import annotations

from dataclasses import dataclass

import torch

_SEED = 1234


def global_seed(seed: int = None) -> int:
    global _SEED
    if seed is not None:
        _SEED = int(seed)
        torch.manual_seed(_SEED)
    return _SEED


@dataclass
class ExecutionPolicy:
    kind: str = "cpu"     # "cpu" | "cuda" | "hybrid"
    device_index: int = 0
    devices: tuple = ()

    @staticmethod
    def cpu(): return ExecutionPolicy("cpu")
    @staticmethod
    def cuda(i: int = 0): return ExecutionPolicy("cuda", i)
    @staticmethod
    def hybrid_cpu_multi_gpu(devices=()): return ExecutionPolicy("hybrid", 0, tuple(devices))

    def device(self) -> str:
        return "cpu" if self.kind == "cpu" else f"cuda:{self.device_index}"
