"""Stateless learning-rate schedules: ``factor(step)`` multiplies the base LR.

Parity: include/nexus/train/schedule.hpp:37-165 of the reference (ConstantLr, LinearLr,
WarmupCosine, WSD with linear or 1-sqrt decay, InverseSqrt; nanoGPT warm-up ``(s+1)/(w+1)``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass


def _warm(step: int, warmup: int) -> float:
    return (step + 1) / (warmup + 1)


def _check_warmup(w: int) -> None:
    if w < 0:
        raise ValueError("LrSchedule: warmup >= 0")


def _check_range(w: int, m: int, r: float) -> None:
    if m <= w or not (0.0 <= r <= 1.0):
        raise ValueError("LrSchedule: max_steps > warmup and 0 <= min_lr_ratio <= 1")


@dataclass
class ConstantLr:
    warmup_steps: int = 0
    name = "constant"

    def __post_init__(self):
        _check_warmup(self.warmup_steps)

    def factor(self, step: int) -> float:
        return _warm(step, self.warmup_steps) if step < self.warmup_steps else 1.0


@dataclass
class LinearLr:
    warmup_steps: int = 0
    max_steps: int = 1
    min_lr_ratio: float = 0.0
    name = "linear"

    def __post_init__(self):
        _check_warmup(self.warmup_steps)
        _check_range(self.warmup_steps, self.max_steps, self.min_lr_ratio)

    def factor(self, step: int) -> float:
        if step < self.warmup_steps:
            return _warm(step, self.warmup_steps)
        if step > self.max_steps:
            return self.min_lr_ratio
        r = (step - self.warmup_steps) / (self.max_steps - self.warmup_steps)
        return self.min_lr_ratio + (1.0 - r) * (1.0 - self.min_lr_ratio)


@dataclass
class WarmupCosine:
    warmup_steps: int = 0
    max_steps: int = 1
    min_lr_ratio: float = 0.1
    name = "warmup_cosine"

    def __post_init__(self):
        _check_warmup(self.warmup_steps)
        _check_range(self.warmup_steps, self.max_steps, self.min_lr_ratio)

    def factor(self, step: int) -> float:
        if step < self.warmup_steps:
            return _warm(step, self.warmup_steps)
        if step > self.max_steps:
            return self.min_lr_ratio
        r = (step - self.warmup_steps) / (self.max_steps - self.warmup_steps)
        return self.min_lr_ratio + 0.5 * (1.0 + math.cos(math.pi * r)) * (1.0 - self.min_lr_ratio)


@dataclass
class WSD:
    warmup: int = 0
    stable: int = 0
    decay: int = 1
    min_lr_ratio: float = 0.0
    sqrt_decay: bool = False
    name = "wsd"

    def __post_init__(self):
        _check_warmup(self.warmup)
        if self.stable < 0 or self.decay < 1 or not (0.0 <= self.min_lr_ratio <= 1.0):
            raise ValueError("WSD: stable >= 0, decay >= 1, 0 <= min_lr_ratio <= 1")

    def factor(self, step: int) -> float:
        if step < self.warmup:
            return _warm(step, self.warmup)
        begin = self.warmup + self.stable
        if step < begin:
            return 1.0
        r = min(1.0, (step - begin + 1) / self.decay)
        shape = 1.0 - math.sqrt(r) if self.sqrt_decay else 1.0 - r
        return self.min_lr_ratio + shape * (1.0 - self.min_lr_ratio)


@dataclass
class InverseSqrt:
    warmup_steps: int = 1
    name = "inverse_sqrt"

    def __post_init__(self):
        if self.warmup_steps < 1:
            raise ValueError("InverseSqrt: warmup_steps >= 1")

    def factor(self, step: int) -> float:
        if step < self.warmup_steps:
            return _warm(step, self.warmup_steps)
        return math.sqrt((self.warmup_steps + 1) / (step + 1))


class LrSchedule:
    """Wraps one of the specs above; ``LrSchedule()`` is a constant schedule."""

    def __init__(self, spec=None):
        self.spec = spec if spec is not None else ConstantLr()

    def factor(self, step: int) -> float:
        if step < 0:
            raise ValueError("LrSchedule: step >= 0")
        return self.spec.factor(step)

    def describe(self) -> str:
        return self.spec.name
