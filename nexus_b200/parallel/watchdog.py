"""Heartbeat watchdog: every rank beats (step, duration) onto a board; a monitor thread flags ranks
that are **stalled** (behind the leader and silent for longer than ``stall_timeout``) or
**stragglers** (arrival lag above a fraction of the median step time over a window).  It reports
and never kills.  Boards: `LocalBoard` (in-process) and `StoreBoard` (any key-value store with
set/get, e.g. ``torch.distributed.TCPStore``; keys ``nexus/wd/<rank>``).
Parity: include/nexus/dist/watchdog.hpp:37-125 and src/dist/watchdog.cpp of the reference."""
from __future__ import annotations

import json
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


@dataclass
class WatchdogOptions:
    stall_timeout_s: float = 30.0
    poll_s: float = 0.05
    straggler_fraction: float = 0.5
    min_lag_s: float = 0.010
    window: int = 5


@dataclass
class WatchdogEvent:
    kind: str  # "stalled" | "straggler"
    rank: int
    step: int
    detail: float


class LocalBoard:
    def __init__(self):
        self._d: Dict[int, dict] = {}
        self._lock = threading.Lock()

    def post(self, rank: int, rec: dict) -> None:
        with self._lock:
            self._d[rank] = rec

    def read(self, rank: int) -> Optional[dict]:
        with self._lock:
            return self._d.get(rank)


class StoreBoard:
    def __init__(self, store, prefix: str = "nexus/wd/"):
        self.store, self.prefix = store, prefix

    def post(self, rank: int, rec: dict) -> None:
        self.store.set(f"{self.prefix}{rank}", json.dumps(rec))

    def read(self, rank: int) -> Optional[dict]:
        try:
            if hasattr(self.store, "check") and not self.store.check([f"{self.prefix}{rank}"]):
                return None
            return json.loads(self.store.get(f"{self.prefix}{rank}"))
        except Exception:
            return None


class Watchdog:
    def __init__(self, board, rank: int, world: int, options: Optional[WatchdogOptions] = None,
                 on_event: Optional[Callable[[WatchdogEvent], None]] = None, monitor: bool = True):
        self.board, self.rank, self.world = board, rank, world
        self.o = options or WatchdogOptions()
        self.on_event = on_event
        self.events: List[WatchdogEvent] = []
        self._arrivals: Dict[int, Dict[int, float]] = {}
        self._flagged = set()
        self._stop = threading.Event()
        self._thread = None
        if monitor:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def beat(self, step: int, step_ms: float = 0.0) -> None:
        self.board.post(self.rank, {"step": int(step), "ms": float(step_ms), "t": time.time()})

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def _emit(self, ev: WatchdogEvent) -> None:
        key = (ev.kind, ev.rank, ev.step)
        if key in self._flagged:
            return
        self._flagged.add(key)
        self.events.append(ev)
        if self.on_event:
            self.on_event(ev)

    def check_once(self, now: Optional[float] = None) -> None:
        """One pass over the board; the comparison of the ranks' heartbeats is native (`_native.watchdog_scan`)."""
        from .. import _native
        now = time.time() if now is None else now
        recs = [self.board.read(r) for r in range(self.world)]
        for kind, rank, step, detail in _native.watchdog_scan(recs, float(now), float(self.o.stall_timeout_s),
                                                              float(self.o.straggler_fraction), float(self.o.min_lag_s),
                                                              self._arrivals, int(self.o.window)):
            self._emit(WatchdogEvent(kind, int(rank), int(step), float(detail)))

    def _loop(self) -> None:
        while not self._stop.wait(self.o.poll_s):
            try:
                self.check_once()
            except Exception:
                pass
