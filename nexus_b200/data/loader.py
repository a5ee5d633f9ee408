"""GPU token loader: a background thread fills pinned host buffers with the next token batches and copies
them to the device on its own stream; `next()` hands the batches out in order and makes the consumer's
stream wait on the copy's event.  Parity: include/nexus/cuda/token_loader.hpp, src/cuda/token_loader.cpp."""
from __future__ import annotations

import queue
import threading
from typing import Optional

import numpy as np
import torch


class GpuTokenLoader:
    def __init__(self, source, micro_batch: int, seq_len: int, device: str = "cuda", depth: int = 2):
        self.source, self.B, self.T, self.depth = source, micro_batch, seq_len, depth
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self._q: "queue.Queue" = queue.Queue(maxsize=depth)
        self._free: "queue.Queue" = queue.Queue()
        for _ in range(depth + 1):
            host = torch.empty((micro_batch, seq_len), dtype=torch.int32)
            if self.cuda:
                host = host.pin_memory()
            dev = torch.empty((micro_batch, seq_len), dtype=torch.int32, device=self.device)
            self._free.put((host, dev))
        self._stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._stop = False
        self._error: Optional[BaseException] = None
        self.batches = 0
        self.h2d_bytes = 0
        self._thread = threading.Thread(target=self._run, name="nexus-token-loader", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        try:
            while not self._stop:
                host, dev = self._free.get()
                if self._stop:
                    return
                if hasattr(self.source, "next_into"):     # native reader: decode straight into the pinned buffer
                    self.source.next_into(host.data_ptr(), self.B, self.T)
                else:
                    rows = self.source.next_rows(self.B, self.T)
                    host.copy_(torch.from_numpy(np.asarray(rows, dtype=np.int32)))
                ev = None
                if self.cuda:
                    with torch.cuda.stream(self._stream):
                        dev.copy_(host, non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record(self._stream)
                else:
                    dev.copy_(host)
                self._q.put((host, dev, ev))
        except BaseException as e:   # surfaced by next()
            self._error = e
            self._q.put(None)

    def next(self) -> torch.Tensor:
        """The next batch on the device (valid until the following call returns)."""
        item = self._q.get()
        if item is None:
            raise RuntimeError("token loader thread failed") from self._error
        host, dev, ev = item
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
        if hasattr(self, "_held"):
            self._free.put(self._held)
        self._held = (host, dev)
        self.batches += 1
        self.h2d_bytes += host.numel() * 4
        return dev

    def close(self) -> None:
        self._stop = True
        self._free.put((None, None))
        self._thread.join(timeout=5)
