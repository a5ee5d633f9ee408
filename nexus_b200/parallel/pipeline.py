"""Pipeline-parallel schedules: GPipe, 1F1B, interleaved 1F1B (virtual stages) and ZB-H1
(zero-bubble: backward split into input-gradient B and weight-gradient W, W deferred into bubbles).

The model is cut into ``pp * v`` chunks; chunk g lives on rank ``g % pp`` (local index ``g // pp``).
For every chunk the B/W actions visit micro-batches in increasing order, so gradient accumulation
order — and therefore the result — is bit-identical across schedules.  A pipeline executor drives
the actions with overlapped point-to-point transfers (NCCL p2p on side streams on GPUs).

Parity: include/nexus/dist/pipeline.hpp:6-62 and src/dist/pipeline.cpp of the reference
(schedule definitions, warm-up counts, bubble formulas, `balance_partition`).  The schedule builder, the partition
and the simulation run in the native host module (`csrc/host/pipeline_sched.cpp`); this file is their typed front.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

from .. import _native

SCHEDULES = ("gpipe", "1f1b", "interleaved_1f1b", "zb_h1")


@dataclass(frozen=True)
class PipeAction:
    kind: str  # "F" | "B" | "W"
    mb: int
    chunk: int  # global chunk index

    def __str__(self) -> str:
        return f"{self.kind}{self.mb}.{self.chunk}"


def parse_pipe_schedule(name: str) -> str:
    if name not in SCHEDULES:
        raise ValueError(f"unknown pipeline schedule '{name}'")
    return name


def make_schedule(schedule: str, pp: int, rank: int, microbatches: int, virtual_stages: int = 1) -> List[PipeAction]:
    """Action order of ``rank``.  ZB-H1 returns the 1F1B order without W actions: the executor decides
    at run time when a deferred W runs."""
    return [PipeAction(k, mb, c) for k, mb, c in _native.pipe_make_schedule(schedule, pp, rank, microbatches, virtual_stages)]


def theoretical_bubble(schedule: str, pp: int, microbatches: int, virtual_stages: int = 1, tf: float = 1.0,
                       tb: float = 1.0, tw: float = 1.0) -> float:
    """Closed-form idle fraction: (p-1)/(m+p-1) for GPipe and 1F1B, (p-1)/(v*m+p-1) interleaved, and for ZB-H1
    (p-1)(tf+tb-tw) / (m(tf+tb+tw) + (p-1)(tf+tb-tw))."""
    return _native.pipe_theoretical_bubble(schedule, pp, microbatches, virtual_stages, tf, tb, tw)


def balance_partition(costs: Sequence[float], parts: int) -> List[Tuple[int, int]]:
    """Cuts ``costs`` into ``parts`` contiguous non-empty ranges minimising the largest range cost."""
    return [tuple(r) for r in _native.pipe_balance_partition([float(c) for c in costs], parts)]


def simulate_bubble(schedule: str, pp: int, microbatches: int, virtual_stages: int = 1, tf: float = 1.0,
                    tb: float = 1.0, tw: float = 1.0) -> float:
    """Event-driven simulation of the schedule (unit-latency transfers ignored); returns idle / total."""
    return _native.pipe_simulate_bubble(schedule, pp, microbatches, virtual_stages, tf, tb, tw)
