"""Durable training checkpoints (NXS3): per-rank sealed archives under an atomically renamed step
directory, a manifest with sizes and SHA-256 of every file, a ``latest`` pointer, pruning, an
optional double-buffered asynchronous writer, resharding-aware loading and crash injection.

Directory protocol: ``<dir>/step-000000123/{manifest.json, rank<r>.nxs3}`` + ``<dir>/latest``.
Each rank writes ``.tmp-step-.../rank<r>.nxs3.part`` -> rename -> ``rank<r>.done``; rank 0 waits for
every ``.done`` file (through the filesystem: no collective is used, so a dead rank cannot deadlock
the writer), writes the manifest, renames the temporary directory once, updates ``latest`` and
prunes to ``keep``.  A crash at any point leaves the previous checkpoint intact.

Crash injection (tests): ``NEXUS_CKPT_CRASH=rank_file|before_manifest|before_rename`` with optional
``NEXUS_CKPT_CRASH_RANK`` / ``NEXUS_CKPT_CRASH_STEP`` terminates the process with exit code 86 at
that point.

Parity: include/nexus/ckpt/checkpoint.hpp:8-190 and src/ckpt/checkpoint.cpp of the reference.
"""
from __future__ import annotations

import json
import os
import queue
import shutil
import threading
import time
from dataclasses import dataclass, field
from typing import List, Optional

from .. import _native


@dataclass
class CheckpointOptions:
    directory: str = "checkpoints"
    every: int = 0            # save when step % every == 0 (0: only on request)
    keep: int = 3
    asynchronous: bool = False
    timeout_s: float = 300.0


@dataclass
class LoadedCheckpoint:
    step: int
    state: dict
    backend_blobs: List[bytes]
    layout: str
    world: int
    resharded: bool


class CheckpointError(RuntimeError):
    pass


def _crash_point(name: str, rank: int, step: int) -> None:
    want = os.environ.get("NEXUS_CKPT_CRASH", "")
    if want != name:
        return
    r = os.environ.get("NEXUS_CKPT_CRASH_RANK")
    s = os.environ.get("NEXUS_CKPT_CRASH_STEP")
    if r is not None and int(r) != rank:
        return
    if s is not None and int(s) != step:
        return
    os._exit(86)


def _step_dir(step: int) -> str:
    return f"step-{step:09d}"


class CheckpointManager:
    def __init__(self, options: CheckpointOptions, rank: int = 0, world: int = 1):
        self.o, self.rank, self.world = options, rank, world
        os.makedirs(options.directory, exist_ok=True)
        if rank == 0:
            for name in os.listdir(options.directory):  # stale temporaries of a crashed writer
                if name.startswith(".tmp-step-"):
                    shutil.rmtree(os.path.join(options.directory, name), ignore_errors=True)
        self._queue: "queue.Queue" = queue.Queue(maxsize=1)   # one pending + one being written
        self._worker: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        if options.asynchronous:
            self._worker = threading.Thread(target=self._run, daemon=True)
            self._worker.start()

    def due(self, step: int) -> bool:
        return self.o.every > 0 and step > 0 and step % self.o.every == 0

    # ----------------------------------------------------------------------------------- save
    def save(self, step: int, state: dict, backend_blob: bytes, layout: str = "replicated") -> None:
        job = (step, dict(state), bytes(backend_blob), layout)
        if self._worker is None:
            self._write(*job)
            return
        if self._error is not None:
            e, self._error = self._error, None
            raise CheckpointError(f"asynchronous checkpoint writer failed: {e}")
        self._queue.put(job)  # blocks while one checkpoint is pending and another is being written

    def wait(self) -> None:
        if self._worker is not None:
            self._queue.join()
        if self._error is not None:
            e, self._error = self._error, None
            raise CheckpointError(f"asynchronous checkpoint writer failed: {e}")

    def _run(self) -> None:
        while True:
            job = self._queue.get()
            try:
                self._write(*job)
            except BaseException as e:  # surfaced by the next save()/wait()
                self._error = e
            finally:
                self._queue.task_done()

    def _write(self, step: int, state: dict, backend_blob: bytes, layout: str) -> None:
        d = self.o.directory
        tmp = os.path.join(d, ".tmp-" + _step_dir(step))
        final = os.path.join(d, _step_dir(step))
        os.makedirs(tmp, exist_ok=True)
        st = dict(state)
        st.update(world=self.world, rank=self.rank, step=step)
        blob = _native.nxs3_encode([("state", json.dumps(st).encode()), ("backend", backend_blob)])
        fname = os.path.join(tmp, f"rank{self.rank}.nxs3")
        _crash_point("rank_file", self.rank, step)
        _native.write_file_atomic(fname, blob)
        with open(os.path.join(tmp, f"rank{self.rank}.done"), "w") as f:
            f.write(_native.sha256_hex(blob))
        if self.rank != 0:
            return
        deadline = time.monotonic() + self.o.timeout_s
        while True:
            if all(os.path.exists(os.path.join(tmp, f"rank{r}.done")) for r in range(self.world)):
                break
            if time.monotonic() > deadline:
                raise CheckpointError(f"checkpoint step {step}: not every rank finished within {self.o.timeout_s}s")
            time.sleep(0.005)
        files = []
        for r in range(self.world):
            p = os.path.join(tmp, f"rank{r}.nxs3")
            files.append({"name": f"rank{r}.nxs3", "bytes": os.path.getsize(p), "sha256": _native.sha256_file(p)})
        manifest = {"format": "NXS3", "version": 3, "step": step, "world": self.world, "layout": layout,
                    "files": files, "state": st}
        _crash_point("before_manifest", self.rank, step)
        with open(os.path.join(tmp, "manifest.json"), "w") as f:
            json.dump(manifest, f)
        for r in range(self.world):
            os.remove(os.path.join(tmp, f"rank{r}.done"))
        _crash_point("before_rename", self.rank, step)
        if os.path.exists(final):
            shutil.rmtree(final)
        os.rename(tmp, final)
        _native.write_file_atomic(os.path.join(d, "latest"), _step_dir(step).encode())
        self._prune()

    def _prune(self) -> None:
        steps = sorted(n for n in os.listdir(self.o.directory) if n.startswith("step-"))
        for old in steps[: max(0, len(steps) - self.o.keep)]:
            shutil.rmtree(os.path.join(self.o.directory, old), ignore_errors=True)

    # ----------------------------------------------------------------------------------- load
    def list_steps(self) -> List[int]:
        return sorted(int(n[5:]) for n in os.listdir(self.o.directory) if n.startswith("step-"))

    def load_latest(self) -> Optional[LoadedCheckpoint]:
        """Newest checkpoint whose files verify; falls back to older ones when the newest is damaged."""
        for step in reversed(self.list_steps()):
            try:
                return self.load(step)
            except (CheckpointError, OSError, RuntimeError, json.JSONDecodeError):
                continue
        return None

    def load(self, step: int) -> LoadedCheckpoint:
        base = os.path.join(self.o.directory, _step_dir(step))
        with open(os.path.join(base, "manifest.json")) as f:
            man = json.load(f)
        blobs, state0 = [], None
        for entry in man["files"]:
            p = os.path.join(base, entry["name"])
            if os.path.getsize(p) != entry["bytes"]:
                raise CheckpointError(f"{p}: size differs from the manifest")
            if _native.sha256_file(p) != entry["sha256"]:
                raise CheckpointError(f"{p}: SHA-256 differs from the manifest")
            with open(p, "rb") as f:
                items = dict(_native.nxs3_decode(f.read()))
            blobs.append(items["backend"])
            if state0 is None:
                state0 = json.loads(items["state"].decode())
        old_world = int(man["world"])
        resharded = old_world != self.world
        if not resharded:
            with open(os.path.join(base, f"rank{self.rank}.nxs3"), "rb") as f:
                state0 = json.loads(dict(_native.nxs3_decode(f.read()))["state"].decode())
        return LoadedCheckpoint(step=int(man["step"]), state=state0, backend_blobs=blobs, layout=man["layout"],
                                world=old_world, resharded=resharded)
