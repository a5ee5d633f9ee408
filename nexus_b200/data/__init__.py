"""Data facade: `Table`, `parse_csv`, `read_csv`, `DataLoader`, `make_loader`, `AsyncPrefetcher`,
and a device token loader that uploads batches ahead of the consumer.
Parity: include/nexus/data, lib/NexusTrain AsyncPrefetcher and include/nexus/cuda/token_loader.hpp of the reference."""
from __future__ import annotations

import queue
import threading
from dataclasses import dataclass
from typing import Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class Table:
    columns: List[str]
    values: np.ndarray  # [rows, cols] float32

    def column(self, name: str) -> np.ndarray:
        return self.values[:, self.columns.index(name)]

    def split_xy(self, target: str) -> Tuple[np.ndarray, np.ndarray]:
        i = self.columns.index(target)
        keep = [j for j in range(len(self.columns)) if j != i]
        return self.values[:, keep], self.values[:, i]


def parse_csv(text: str, header: bool = True, delimiter: str = ",") -> Table:
    lines = [l for l in text.splitlines() if l.strip()]
    if not lines:
        raise ValueError("parse_csv: empty input")
    cols = [c.strip() for c in lines[0].split(delimiter)] if header else [f"c{i}" for i in range(len(lines[0].split(delimiter)))]
    rows = []
    for n, l in enumerate(lines[1:] if header else lines):
        parts = l.split(delimiter)
        if len(parts) != len(cols):
            raise ValueError(f"parse_csv: row {n} has {len(parts)} fields, expected {len(cols)}")
        rows.append([float(p) for p in parts])
    return Table(cols, np.asarray(rows, dtype=np.float32))


def read_csv(path: str, header: bool = True, delimiter: str = ",") -> Table:
    with open(path) as f:
        return parse_csv(f.read(), header, delimiter)


class DataLoader:
    """In-memory loader over (x, y) arrays with deterministic shuffling (seed + epoch)."""

    def __init__(self, x, y, batch_size: int = 32, shuffle: bool = False, seed: int = 0, drop_last: bool = False):
        self.x, self.y = np.asarray(x), np.asarray(y)
        if len(self.x) != len(self.y):
            raise ValueError("DataLoader: x and y differ in length")
        self.batch_size, self.shuffle, self.seed, self.drop_last = batch_size, shuffle, seed, drop_last
        self.epoch = 0

    def __len__(self) -> int:
        n = len(self.x)
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def __iter__(self) -> Iterator:
        n = len(self.x)
        idx = np.arange(n)
        if self.shuffle:
            np.random.default_rng(self.seed + self.epoch).shuffle(idx)
        self.epoch += 1
        for b in range(len(self)):
            sel = idx[b * self.batch_size: (b + 1) * self.batch_size]
            yield torch.from_numpy(self.x[sel]), torch.from_numpy(self.y[sel])


def make_loader(table: Table, target: str, batch_size: int = 32, shuffle: bool = True, seed: int = 0) -> DataLoader:
    x, y = table.split_xy(target)
    return DataLoader(x, y.astype(np.int64), batch_size, shuffle, seed)


class AsyncPrefetcher:
    """Runs an iterable in a background thread, ``depth`` items ahead, preserving order."""

    def __init__(self, source: Iterable, depth: int = 2, transform=None):
        self.source, self.depth, self.transform = source, depth, transform

    def __iter__(self):
        q: "queue.Queue" = queue.Queue(maxsize=self.depth)
        end = object()

        def run():
            try:
                for item in self.source:
                    q.put(self.transform(item) if self.transform else item)
                q.put(end)
            except BaseException as e:
                q.put(e)
        threading.Thread(target=run, daemon=True).start()
        while True:
            item = q.get()
            if item is end:
                return
            if isinstance(item, BaseException):
                raise item
            yield item


class DeviceTokenLoader:
    """Background prefetch of token batches to the device through pinned staging buffers, in order."""

    def __init__(self, source, rows: int, seq_len: int, device="cuda", depth: int = 2):
        self.source, self.rows, self.T, self.device, self.depth = source, rows, seq_len, torch.device(device), depth

    def __iter__(self):
        def upload(arr):
            t = torch.from_numpy(np.ascontiguousarray(arr, dtype=np.int32))
            if self.device.type == "cuda":
                return t.pin_memory().to(self.device, non_blocking=True)
            return t

        def gen():
            while True:
                yield self.source.next_rows(self.rows, self.T)
        return iter(AsyncPrefetcher(gen(), self.depth, upload))
