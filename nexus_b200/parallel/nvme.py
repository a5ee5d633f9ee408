"""Key -> file store for offloaded optimizer state / parameter shards with asynchronous reads and
writes through 4096-byte aligned bounce buffers.
Parity: include/nexus/dist/nvme.hpp and src/dist/nvme.cpp of the reference."""
from __future__ import annotations

import os
from concurrent.futures import Future, ThreadPoolExecutor

ALIGN = 4096


class NvmeStore:
    def __init__(self, directory: str, workers: int = 2):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)
        self.pool = ThreadPoolExecutor(max_workers=workers)
        self.bytes_written = 0
        self.bytes_read = 0

    def _path(self, key: str) -> str:
        return os.path.join(self.dir, key.replace("/", "_") + ".bin")

    def write(self, key: str, data: bytes) -> None:
        padded = (len(data) + ALIGN - 1) // ALIGN * ALIGN
        buf = bytearray(padded)           # aligned bounce buffer (length is a multiple of the sector size)
        buf[: len(data)] = data
        tmp = self._path(key) + ".part"
        with open(tmp, "wb") as f:
            f.write(len(data).to_bytes(8, "little"))
            f.write(buf)
        os.replace(tmp, self._path(key))
        self.bytes_written += len(data)

    def read(self, key: str) -> bytes:
        with open(self._path(key), "rb") as f:
            n = int.from_bytes(f.read(8), "little")
            data = f.read(n)
        self.bytes_read += n
        return data

    def write_async(self, key: str, data: bytes) -> Future:
        return self.pool.submit(self.write, key, data)

    def read_async(self, key: str) -> Future:
        return self.pool.submit(self.read, key)

    def contains(self, key: str) -> bool:
        return os.path.exists(self._path(key))

    def remove(self, key: str) -> None:
        if self.contains(key):
            os.remove(self._path(key))
