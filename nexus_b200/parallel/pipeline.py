"""Pipeline-parallel schedules: GPipe, 1F1B, interleaved 1F1B (virtual stages) and ZB-H1
(zero-bubble: backward split into input-gradient B and weight-gradient W, W deferred into bubbles).

The model is cut into ``pp * v`` chunks; chunk g lives on rank ``g % pp`` (local index ``g // pp``).
For every chunk the B/W actions visit micro-batches in increasing order, so gradient accumulation
order — and therefore the result — is bit-identical across schedules.  A pipeline executor drives
the actions with overlapped point-to-point transfers (NCCL p2p on side streams on GPUs).

Parity: include/nexus/dist/pipeline.hpp:6-62 and src/dist/pipeline.cpp of the reference
(schedule definitions, warm-up counts, bubble formulas, `balance_partition`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

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
    parse_pipe_schedule(schedule)
    m, v = microbatches, virtual_stages
    if pp < 1 or not (0 <= rank < pp) or m < 1 or v < 1:
        raise ValueError("make_schedule: pp >= 1, 0 <= rank < pp, microbatches >= 1, virtual_stages >= 1")
    acts: List[PipeAction] = []
    if schedule == "gpipe":
        for c in range(v):
            acts += [PipeAction("F", i, c * pp + rank) for i in range(m)]
        for c in reversed(range(v)):
            acts += [PipeAction("B", i, c * pp + rank) for i in range(m)]
        return acts
    if schedule in ("1f1b", "zb_h1"):
        if v != 1:
            raise ValueError(f"{schedule} uses one chunk per rank (virtual_stages = 1)")
        warm = min(pp - rank - 1, m)
        f = b = 0
        for _ in range(warm):
            acts.append(PipeAction("F", f, rank)); f += 1
        while f < m:
            acts.append(PipeAction("F", f, rank)); f += 1
            acts.append(PipeAction("B", b, rank)); b += 1
        while b < m:
            acts.append(PipeAction("B", b, rank)); b += 1
        return acts
    # interleaved 1F1B
    if m % pp != 0:
        raise ValueError("interleaved_1f1b needs microbatches % pp == 0")
    total = m * v

    def fwd(k):
        return PipeAction("F", (k // (pp * v)) * pp + k % pp, ((k // pp) % v) * pp + rank)

    def bwd(k):
        return PipeAction("B", (k // (pp * v)) * pp + k % pp, (v - 1 - (k // pp) % v) * pp + rank)
    warm = min((pp - rank - 1) * 2 + (v - 1) * pp, total)
    f = b = 0
    for _ in range(warm):
        acts.append(fwd(f)); f += 1
    while f < total:
        acts.append(fwd(f)); f += 1
        acts.append(bwd(b)); b += 1
    while b < total:
        acts.append(bwd(b)); b += 1
    return acts


def theoretical_bubble(schedule: str, pp: int, microbatches: int, virtual_stages: int = 1, tf: float = 1.0,
                       tb: float = 1.0, tw: float = 1.0) -> float:
    p, m, v = pp, microbatches, virtual_stages
    if schedule in ("gpipe", "1f1b"):
        return (p - 1) / (m + p - 1)
    if schedule == "interleaved_1f1b":
        return (p - 1) / (v * m + p - 1)
    if schedule == "zb_h1":
        idle = (p - 1) * (tf + tb - tw)
        return idle / (m * (tf + tb + tw) + idle)
    raise ValueError(f"unknown pipeline schedule '{schedule}'")


def balance_partition(costs: Sequence[float], parts: int) -> List[Tuple[int, int]]:
    """Cuts ``costs`` into ``parts`` contiguous non-empty ranges minimising the largest range cost."""
    n = len(costs)
    if not (1 <= parts <= n):
        raise ValueError("balance_partition: 1 <= parts <= number of layers")
    pre = [0.0]
    for c in costs:
        pre.append(pre[-1] + c)
    INF = float("inf")
    best = [[INF] * (n + 1) for _ in range(parts + 1)]
    cut = [[0] * (n + 1) for _ in range(parts + 1)]
    best[0][0] = 0.0
    for k in range(1, parts + 1):
        for i in range(k, n + 1):
            for j in range(k - 1, i):
                c = max(best[k - 1][j], pre[i] - pre[j])
                if c < best[k][i]:
                    best[k][i], cut[k][i] = c, j
    out, i = [], n
    for k in range(parts, 0, -1):
        j = cut[k][i]
        out.append((j, i))
        i = j
    return list(reversed(out))


def simulate_bubble(schedule: str, pp: int, microbatches: int, virtual_stages: int = 1, tf: float = 1.0,
                    tb: float = 1.0, tw: float = 1.0) -> float:
    """Event-driven simulation of the schedule (unit-latency transfers ignored); returns idle / total."""
    v = virtual_stages
    split = schedule == "zb_h1"
    acts = [make_schedule(schedule, pp, r, microbatches, v) for r in range(pp)]
    nchunks = pp * v
    done: Dict[Tuple[str, int, int], float] = {}
    clock = [0.0] * pp
    busy = [0.0] * pp
    ptr = [0] * pp
    pending_w = [[] for _ in range(pp)]
    progressed = True
    while progressed:
        progressed = False
        for r in range(pp):
            while ptr[r] < len(acts[r]):
                a = acts[r][ptr[r]]
                if a.kind == "F":
                    dep = ("F", a.mb, a.chunk - 1) if a.chunk > 0 else None
                else:
                    dep = ("B", a.mb, a.chunk + 1) if a.chunk < nchunks - 1 else ("F", a.mb, a.chunk)
                if dep is not None and dep not in done:
                    break
                ready = done.get(dep, 0.0) if dep else 0.0
                if split:
                    # run deferred W work while waiting for the input of the next action
                    while pending_w[r] and clock[r] + tw <= ready + 1e-12:
                        pending_w[r].pop(0)
                        clock[r] += tw
                        busy[r] += tw
                    while len(pending_w[r]) > pp - r:
                        pending_w[r].pop(0)
                        clock[r] += tw
                        busy[r] += tw
                start = max(clock[r], ready)
                dur = tf if a.kind == "F" else (tb if split else tb + tw)
                clock[r] = start + dur
                busy[r] += dur
                done[(a.kind, a.mb, a.chunk)] = clock[r]
                if split and a.kind == "B":
                    pending_w[r].append(a)
                ptr[r] += 1
                progressed = True
    for r in range(pp):
        clock[r] += tw * len(pending_w[r])
        busy[r] += tw * len(pending_w[r])
    total = max(clock)
    return 1.0 - sum(busy) / (total * pp)
