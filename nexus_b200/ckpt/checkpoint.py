"""Durable training checkpoints (NXS3): per-rank sealed archives under an atomically renamed step
directory, a manifest with sizes and SHA-256 of every file, a ``latest`` pointer, pruning, an
optional double-buffered asynchronous writer, resharding-aware loading and crash injection.

Directory protocol: ``<dir>/step-000000123/{manifest.json, rank<r>.nxs3}`` + ``<dir>/latest`` (the bare
step number).  Each rank writes ``.tmp-step-.../rank<r>.nxs3.part`` -> rename -> ``rank<r>.done``
(``"<sha256 hex> <bytes>"``); rank 0 waits for every ``.done`` file (through the filesystem: no collective
is used, so a dead rank cannot deadlock the writer), writes the manifest from them, renames the temporary
directory once, updates ``latest`` and prunes to ``keep``.  A crash at any point leaves the previous
checkpoint intact.

Interchange with the reference's writer: the archive layout, the ``state`` entry (`TrainerState.encode`:
u32 schema 1 followed by the fixed little-endian field list), the manifest's per-file ``sha256`` (the
archive's own 32-byte trailer, i.e. the digest of everything before it, so no second hashing pass), the
``.done`` records and the ``latest`` pointer all use the reference's bytes.  The ``backend`` entry is
whatever the training backend serialises and is only meaningful to the same backend.

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
import struct
import threading
import time
import warnings
from dataclasses import asdict, dataclass, field
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
class TrainerState:
    """The trainer-side record of a checkpoint, with the reference's binary encoding
    (include/nexus/ckpt/checkpoint.hpp:81-102, src/ckpt/checkpoint.cpp:375-423)."""
    step: int = 0
    epoch: int = 0
    global_sample_index: int = 0
    train_cursor: str = ""
    val_cursor: str = ""
    lr_factor: float = 1.0
    schedule_step: int = 0
    loss_scale: float = 1.0
    rng_seed: int = 0
    rng_offset: int = 0
    accum_counter: int = 0
    accum_steps: int = 1
    micro_batch: int = 1
    seq_len: int = 2
    global_batch_tokens: int = 0
    rollbacks: int = 0
    world: int = 1
    rank: int = 0

    def encode(self) -> bytes:
        def s(text: str) -> bytes:
            raw = text.encode()
            return struct.pack("<Q", len(raw)) + raw
        return (struct.pack("<IqqQ", 1, self.step, self.epoch, self.global_sample_index) + s(self.train_cursor)
                + s(self.val_cursor) + struct.pack("<dqdQQiiiiqiii", self.lr_factor, self.schedule_step,
                                                   self.loss_scale, self.rng_seed, self.rng_offset, self.accum_counter,
                                                   self.accum_steps, self.micro_batch, self.seq_len,
                                                   self.global_batch_tokens, self.rollbacks, self.world, self.rank))

    @staticmethod
    def decode(raw: bytes) -> "TrainerState":
        try:
            ver, step, epoch, gsi = struct.unpack_from("<IqqQ", raw, 0)
            if ver != 1:
                raise CheckpointError("TrainerState: unsupported schema version %d" % ver)
            pos = 28
            texts = []
            for _ in range(2):
                (n,) = struct.unpack_from("<Q", raw, pos)
                pos += 8
                if pos + n > len(raw):
                    raise struct.error("short")
                texts.append(raw[pos: pos + n].decode())
                pos += n
            rest = struct.unpack_from("<dqdQQiiiiqiii", raw, pos)
        except struct.error:
            raise CheckpointError("TrainerState: short data (damaged or truncated)") from None
        return TrainerState(step, epoch, gsi, texts[0], texts[1], *rest)

    @staticmethod
    def from_dict(d: dict) -> "TrainerState":
        """Accepts the trainers' plain dictionaries: unknown keys are ignored, cursors may be integers and
        ``tokens_seen`` is folded into ``global_sample_index`` (rows consumed = tokens / seq_len)."""
        st = TrainerState()
        for k in asdict(st):
            if k in d and d[k] is not None:
                cur = getattr(st, k)
                setattr(st, k, str(d[k]) if isinstance(cur, str) else type(cur)(d[k]))
        if "tokens_seen" in d and "global_sample_index" not in d:
            st.global_sample_index = int(d["tokens_seen"]) // max(st.seq_len, 1)
        return st

    def to_dict(self) -> dict:
        d = asdict(self)
        for k in ("train_cursor", "val_cursor"):
            if d[k].lstrip("-").isdigit():
                d[k] = int(d[k])
        d["tokens_seen"] = self.global_sample_index * self.seq_len
        return d

    def to_json(self) -> str:
        """The manifest's human-readable copy (the reference's key set and order)."""
        return ('{"step":%d,"epoch":%d,"global_sample_index":%d,"lr_factor":%.17g,"schedule_step":%d,"loss_scale":%.17g,'
                '"rng":{"seed":%d,"offset":%d},"accum_counter":%d,"accum_steps":%d,"micro_batch":%d,"seq_len":%d,'
                '"global_batch_tokens":%d,"rollbacks":%d,"world":%d,"train_cursor_rank0":%s}'
                % (self.step, self.epoch, self.global_sample_index, self.lr_factor, self.schedule_step,
                   self.loss_scale, self.rng_seed, self.rng_offset, self.accum_counter, self.accum_steps,
                   self.micro_batch, self.seq_len, self.global_batch_tokens, self.rollbacks, self.world,
                   json.dumps(self.train_cursor)))


def trailer_hex(archive: bytes) -> str:
    """Hex of the 32-byte SHA-256 an NXS3 archive ends with (the digest of everything before it)."""
    if len(archive) < 32:
        raise CheckpointError("archive shorter than its checksum")
    return bytes(archive[-32:]).hex()


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


def _crash_armed(name: str, rank: int, step: int) -> bool:
    if os.environ.get("NEXUS_CKPT_CRASH", "") != name:
        return False
    r = os.environ.get("NEXUS_CKPT_CRASH_RANK")
    s = os.environ.get("NEXUS_CKPT_CRASH_STEP")
    return (r is None or int(r) == rank) and (s is None or int(s) == step)


def _crash_point(name: str, rank: int, step: int) -> None:
    if _crash_armed(name, rank, step):
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
        ts = TrainerState.from_dict(st)
        # entries the reference does not know ride in a third entry; its loader looks entries up by name
        extra = {k: v for k, v in st.items() if k not in asdict(ts) and k != "tokens_seen"}
        entries = [("state", ts.encode()), ("backend", backend_blob)]
        if extra:
            entries.append(("state_extra", json.dumps(extra).encode()))
        blob = _native.nxs3_encode(entries)
        fname = os.path.join(tmp, f"rank{self.rank}.nxs3")
        if _crash_armed("rank_file", self.rank, step):
            with open(fname + ".part", "wb") as f:   # what a real crash leaves: the first half of the file
                f.write(blob[: len(blob) // 2])
        _crash_point("rank_file", self.rank, step)
        _native.write_file_atomic(fname, blob)
        _native.write_file_atomic(os.path.join(tmp, f"rank{self.rank}.done"),
                                  ("%s %d" % (trailer_hex(blob), len(blob))).encode())
        deadline = time.monotonic() + self.o.timeout_s
        if self.rank != 0:
            # synchronous meaning for every rank: when save() returns the checkpoint is committed
            while not os.path.exists(os.path.join(final, "manifest.json")):
                if time.monotonic() > deadline:
                    raise CheckpointError(f"checkpoint step {step}: rank 0 did not commit within {self.o.timeout_s}s")
                time.sleep(0.002)
            return
        files = []
        for r in range(self.world):
            done = os.path.join(tmp, f"rank{r}.done")
            while not os.path.exists(done):
                if time.monotonic() > deadline:
                    raise CheckpointError(f"checkpoint step {step}: rank {r} did not finish within {self.o.timeout_s}s")
                time.sleep(0.002)
            sha, nbytes = open(done).read().split()
            files.append({"name": f"rank{r}.nxs3", "bytes": int(nbytes), "sha256": sha})
        manifest = ('{"format":"NXS3","version":3,"step":%d,"world":%d,"layout":%s,"files":%s,"state":%s}\n'
                    % (step, self.world, json.dumps(layout), json.dumps(files, separators=(",", ":")), ts.to_json()))
        _crash_point("before_manifest", self.rank, step)
        _native.write_file_atomic(os.path.join(tmp, "manifest.json"), manifest.encode())
        for r in range(self.world):
            os.remove(os.path.join(tmp, f"rank{r}.done"))
        _crash_point("before_rename", self.rank, step)
        if os.path.exists(final):
            shutil.rmtree(final)
        os.rename(tmp, final)
        _native.write_file_atomic(os.path.join(d, "latest"), str(step).encode())
        self._prune()

    def _prune(self) -> None:
        if self.o.keep <= 0:
            return
        steps = self.list_steps()
        for old in steps[: max(0, len(steps) - self.o.keep)]:
            shutil.rmtree(os.path.join(self.o.directory, _step_dir(old)), ignore_errors=True)

    # ----------------------------------------------------------------------------------- load
    def list_steps(self) -> List[int]:
        """Committed steps: ``step-<9 digits>`` directories that hold a manifest."""
        out = []
        for n in os.listdir(self.o.directory):
            if len(n) == 14 and n.startswith("step-") and n[5:].isdigit() and \
                    os.path.exists(os.path.join(self.o.directory, n, "manifest.json")):
                out.append(int(n[5:]))
        return sorted(out)

    def load_latest(self, fallback: bool = True) -> Optional[LoadedCheckpoint]:
        """Newest committed checkpoint.  When it does not verify, the reference stops with an error; here
        ``fallback=True`` (default) warns loudly and tries the next older one, ``fallback=False`` raises."""
        steps = self.list_steps()
        for i, step in enumerate(reversed(steps)):
            try:
                return self.load(step)
            except (CheckpointError, OSError, RuntimeError, json.JSONDecodeError) as e:
                if not fallback:
                    raise CheckpointError(f"newest checkpoint (step {step}) failed verification: {e}") from e
                warnings.warn(f"checkpoint step {step} failed verification ({e}); falling back to an older one",
                              RuntimeWarning, stacklevel=2)
        return None

    def _load_rank(self, base: str, entry: dict):
        p = os.path.join(base, entry["name"])
        with open(p, "rb") as f:
            raw = f.read()
        if len(raw) != int(entry["bytes"]) or len(raw) < 32 or trailer_hex(raw) != entry["sha256"]:
            raise CheckpointError(f"{p}: differs from the manifest (size or SHA-256)")
        try:
            items = dict(_native.nxs3_decode(raw))   # verifies the content against the trailer
        except RuntimeError as e:
            raise CheckpointError(f"{p}: {e}") from e
        if "backend" not in items or "state" not in items:
            raise CheckpointError(f"{p}: archive lacks the 'state' / 'backend' entries")
        state = TrainerState.decode(items["state"]).to_dict()
        if "state_extra" in items:
            state.update(json.loads(items["state_extra"].decode()))
        return state, items["backend"]

    def load(self, step: int) -> LoadedCheckpoint:
        """Reads and verifies this rank's file only; every old rank's file when the world size changed."""
        base = os.path.join(self.o.directory, _step_dir(step))
        with open(os.path.join(base, "manifest.json")) as f:
            man = json.load(f)
        if man.get("format") != "NXS3" or int(man.get("version", 0)) != 3:
            raise CheckpointError(f"{base}: unsupported checkpoint format")
        old_world = int(man["world"])
        if len(man["files"]) != old_world:
            raise CheckpointError(f"{base}: manifest lists {len(man['files'])} files for world {old_world}")
        resharded = old_world != self.world
        if resharded:
            loaded = [self._load_rank(base, e) for e in man["files"]]
            state0, blobs = loaded[0][0], [b for _, b in loaded]
        else:
            state0, mine = self._load_rank(base, man["files"][self.rank])
            blobs = [None] * old_world
            blobs[self.rank] = mine
        return LoadedCheckpoint(step=int(man["step"]), state=state0, backend_blobs=blobs, layout=man["layout"],
                                world=old_world, resharded=resharded)
