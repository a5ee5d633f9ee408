"""Memory management: the host caching allocator (64-byte aligned power-of-two size classes), the
stream-aware device caching allocator (small / large pools, split + merge, per-stream free lists,
`record_stream`, out-of-memory retry), the static arena planner and its `LifetimeRecorder`, and the cache of
narrow parameter copies keyed by tensor version.
Parity: include/nexus/core/allocator.hpp, include/nexus/cuda/caching_allocator.hpp,
include/nexus/memory/planner.hpp:18-54, include/nexus/cuda/cast_cache.hpp of the reference."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import _native as N

HostCachingAllocator = N.HostCachingAllocator
DeviceCachingAllocator = N.DeviceCachingAllocator


def plan_memory(lifetimes: List[Tuple[int, int, int]], alignment: int = 256):
    """[(bytes, first_use, last_use)] -> (offsets, arena_bytes): greedy-by-size best-fit placement."""
    return N.plan_memory(lifetimes, alignment)


class LifetimeRecorder:
    """Records `define(name, bytes)` / `use(name)` against a running step counter and turns the result into
    planner input."""

    def __init__(self):
        self.step = 0
        self.items: Dict[str, List[int]] = {}

    def tick(self) -> int:
        self.step += 1
        return self.step

    def define(self, name: str, nbytes: int) -> None:
        self.items[name] = [int(nbytes), self.step, self.step]

    def use(self, name: str) -> None:
        self.items[name][2] = self.step

    def plan(self, alignment: int = 256):
        names = list(self.items)
        offsets, arena = plan_memory([tuple(self.items[n]) for n in names], alignment)
        return dict(zip(names, offsets)), arena


class CastCache:
    """Narrow (e.g. BF16) copies of FP32 parameters, refreshed only when the parameter's version changed."""

    def __init__(self, dtype: torch.dtype = torch.bfloat16):
        self.dtype = dtype
        self._cache: Dict[int, Tuple[int, torch.Tensor]] = {}
        self.hits = self.misses = 0

    def get(self, p: torch.Tensor) -> torch.Tensor:
        key, ver = id(p), p._version
        hit = self._cache.get(key)
        if hit is not None and hit[0] == ver and hit[1].shape == p.shape:
            self.hits += 1
            return hit[1]
        self.misses += 1
        if hit is not None and hit[1].shape == p.shape:
            hit[1].copy_(p.detach())
            self._cache[key] = (ver, hit[1])
            return hit[1]
        t = p.detach().to(self.dtype)
        self._cache[key] = (ver, t)
        return t

    def clear(self) -> None:
        self._cache.clear()
