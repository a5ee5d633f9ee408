"""Profiling: interval timers with per-name totals, op counters (FLOPs / bytes / calls), Chrome trace export,
optional NVTX ranges, and the memory ledger (7 labels x 3 memory spaces with peaks).  The recorders live in
the native runtime; this module is their Python face.
Parity: include/nexus/prof/{timer,counters,trace,ledger}.hpp of the reference."""
from __future__ import annotations

import contextlib
import enum
from typing import Dict

import torch

from .. import _native as N


class Label(enum.IntEnum):
    Parameter = 0
    Gradient = 1
    OptimizerState = 2
    Activation = 3
    Temporary = 4
    CommBuffer = 5
    KvCache = 6


class Space(enum.IntEnum):
    Host = 0
    PinnedHost = 1
    Device = 2


_nvtx = [False]


def enable(on: bool = True, nvtx: bool = False) -> None:
    N.prof_enable(bool(on))
    _nvtx[0] = bool(nvtx) and torch.cuda.is_available()


def enabled() -> bool:
    return bool(N.prof_enabled())


def clear() -> None:
    N.prof_clear()


class ScopedTimer:
    """Context manager / decorator: records [enter, exit) under ``name`` (category for the trace)."""

    def __init__(self, name: str, category: str = "host", sync_cuda: bool = False):
        self.name, self.cat, self.sync = name, category, sync_cuda

    def __enter__(self):
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        if _nvtx[0]:
            torch.cuda.nvtx.range_push(self.name)
        self.t0 = N.prof_now_ns()
        return self

    def __exit__(self, *a):
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        t1 = N.prof_now_ns()
        if _nvtx[0]:
            torch.cuda.nvtx.range_pop()
        N.prof_record(self.name, self.cat, self.t0, t1 - self.t0)
        return False

    def __call__(self, fn):
        def wrapped(*a, **k):
            with ScopedTimer(self.name, self.cat, self.sync):
                return fn(*a, **k)
        return wrapped


def record(name: str, category: str, start_ns: int, duration_ns: int) -> None:
    N.prof_record(name, category, int(start_ns), int(duration_ns))


def now_ns() -> int:
    return int(N.prof_now_ns())


def totals() -> Dict[str, dict]:
    """name -> {calls, total_ns, ...} as the native profiler reports it."""
    return dict(N.prof_totals())


def count(op: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
    N.prof_count(op, float(flops), float(nbytes))


def counters() -> Dict[str, dict]:
    return dict(N.prof_counters())


def dump_chrome_trace(path: str) -> int:
    """Writes the recorded intervals as Chrome trace JSON; returns the number of events."""
    return int(N.prof_dump_chrome_trace(path))


class MemoryLedger:
    @staticmethod
    def add(label: Label, space: Space, nbytes: int) -> None:
        N.ledger_add(int(label), int(space), int(nbytes))

    @staticmethod
    def current(label: Label, space: Space) -> int:
        return int(N.ledger_current(int(label), int(space)))

    @staticmethod
    def peak(label: Label, space: Space) -> int:
        return int(N.ledger_peak(int(label), int(space)))

    @staticmethod
    def reset() -> None:
        N.ledger_reset()

    @staticmethod
    @contextlib.contextmanager
    def track(label: Label, space: Space, nbytes: int):
        N.ledger_add(int(label), int(space), int(nbytes))
        try:
            yield
        finally:
            N.ledger_add(int(label), int(space), -int(nbytes))

    @staticmethod
    def report() -> Dict[str, Dict[str, int]]:
        return {l.name: {s.name: {"current": MemoryLedger.current(l, s), "peak": MemoryLedger.peak(l, s)} for s in Space}
                for l in Label}
