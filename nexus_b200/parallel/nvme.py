"""Key -> file store for offloaded optimizer state / parameter shards.  Every file is one 4096-byte header sector
(payload length) followed by the payload padded to whole sectors; reads and writes go through page-aligned bounce
buffers (anonymous mappings) and, where the file system allows it, through ``O_DIRECT`` so that offloaded state does
not pass through (and evict) the page cache.  File systems that refuse direct I/O (tmpfs) get buffered I/O on the same
layout.  Asynchronous forms run on a small thread pool.
Parity: include/nexus/dist/nvme.hpp and src/dist/nvme.cpp of the reference."""
from __future__ import annotations

import errno
import mmap
import os
from concurrent.futures import Future, ThreadPoolExecutor

ALIGN = 4096


def _round_up(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


class NvmeStore:
    def __init__(self, directory: str, workers: int = 2, direct: bool = True):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)
        self.pool = ThreadPoolExecutor(max_workers=workers)
        self.bytes_written = 0
        self.bytes_read = 0
        self.direct = bool(direct) and hasattr(os, "O_DIRECT") and self._probe_direct()

    def _probe_direct(self) -> bool:
        """One aligned sector written with O_DIRECT: does this directory's file system take it?"""
        path = os.path.join(self.dir, ".direct_probe")
        try:
            fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC | os.O_DIRECT, 0o600)
        except OSError:
            return False
        try:
            buf = mmap.mmap(-1, ALIGN)
            try:
                return os.write(fd, buf) == ALIGN
            finally:
                buf.close()
        except OSError:
            return False
        finally:
            os.close(fd)
            try:
                os.remove(path)
            except OSError:
                pass

    def _path(self, key: str) -> str:
        return os.path.join(self.dir, key.replace("/", "_") + ".bin")

    def _open(self, path: str, flags: int) -> int:
        if self.direct:
            try:
                return os.open(path, flags | os.O_DIRECT, 0o600)
            except OSError as e:
                if e.errno != errno.EINVAL:
                    raise
        return os.open(path, flags, 0o600)

    def write(self, key: str, data: bytes) -> None:
        n = len(data)
        total = ALIGN + _round_up(n)
        buf = mmap.mmap(-1, total)                # page-aligned, zero-filled bounce buffer
        try:
            buf[0:8] = n.to_bytes(8, "little")
            buf[ALIGN: ALIGN + n] = data
            tmp = self._path(key) + ".part"
            fd = self._open(tmp, os.O_WRONLY | os.O_CREAT | os.O_TRUNC)
            try:
                view, done = memoryview(buf), 0
                while done < total:               # whole sectors at sector offsets: valid for direct I/O
                    done += os.write(fd, view[done:])
                view.release()
                os.fsync(fd)
            finally:
                os.close(fd)
            os.replace(tmp, self._path(key))
        finally:
            buf.close()
        self.bytes_written += n

    def read(self, key: str) -> bytes:
        path = self._path(key)
        total = _round_up(os.path.getsize(path))
        buf = mmap.mmap(-1, max(total, ALIGN))
        try:
            fd = self._open(path, os.O_RDONLY)
            try:
                view, done = memoryview(buf), 0
                while done < total:
                    got = os.readv(fd, [view[done:]])
                    if got <= 0:
                        break
                    done += got
                view.release()
            finally:
                os.close(fd)
            n = int.from_bytes(buf[0:8], "little")
            if ALIGN + n > done:
                raise IOError(f"{path}: truncated ({done} bytes for a payload of {n})")
            data = bytes(buf[ALIGN: ALIGN + n])
        finally:
            buf.close()
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
