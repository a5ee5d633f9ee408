"""Metric sinks for the trainers: console, CSV, JSONL, TensorBoard event files (written without
protobuf: TFRecord framing with masked CRC32C around hand-encoded Event/Summary messages) with a
reader for tests, and a W&B-offline style ``wandb-history.jsonl``.

Parity: include/nexus/train/loggers.hpp:6-60 and src/train/loggers.cpp of the reference.
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
import time
from typing import Dict, List, Tuple

from .. import _native


def _record_dict(rec) -> dict:
    return dataclasses.asdict(rec) if dataclasses.is_dataclass(rec) else dict(rec)


class ConsoleLogger:
    def log(self, rec) -> None:
        d = _record_dict(rec)
        print("step %6d  loss %.4f  lr %.3e  gnorm %.3f  %.0f tok/s  mfu %.3f  %.1f ms" % (
            d["step"], d["loss"], d["lr"], d["grad_norm"], d["tokens_per_s"], d["mfu"], d["step_ms"]), flush=True)

    def flush(self) -> None:
        pass


class CsvLogger:
    def __init__(self, path: str):
        self.path, self._f, self._keys = path, None, None

    def log(self, rec) -> None:
        d = _record_dict(rec)
        if self._f is None:
            self._f = open(self.path, "w")
            self._keys = list(d.keys())
            self._f.write(",".join(self._keys) + "\n")
        self._f.write(",".join(str(d[k]) for k in self._keys) + "\n")

    def flush(self) -> None:
        if self._f:
            self._f.flush()


class JsonlLogger:
    def __init__(self, path: str):
        self._f = open(path, "w")

    def log(self, rec) -> None:
        d = {k: (None if isinstance(v, float) and not math.isfinite(v) else v) for k, v in _record_dict(rec).items()}
        self._f.write(json.dumps(d) + "\n")

    def flush(self) -> None:
        self._f.flush()


class WandbOfflineLogger:
    """Writes ``<run_dir>/wandb-history.jsonl`` with ``_step`` / ``_timestamp`` fields."""

    def __init__(self, run_dir: str):
        os.makedirs(run_dir, exist_ok=True)
        self._f = open(os.path.join(run_dir, "wandb-history.jsonl"), "w")

    def log(self, rec) -> None:
        d = _record_dict(rec)
        row = {k: v for k, v in d.items() if isinstance(v, (int, float)) and (not isinstance(v, float) or math.isfinite(v))}
        row["_step"] = d.get("step", 0)
        row["_timestamp"] = time.time()
        self._f.write(json.dumps(row) + "\n")

    def flush(self) -> None:
        self._f.flush()


# ---------------------------------------------------------------------------- TensorBoard events
# CRC32C, the TFRecord framing and the hand-encoded Event / Summary messages live in the native host module
# (`csrc/host/tb_events.cpp`).
def crc32c(data: bytes) -> int:
    return _native.crc32c(bytes(data))


def masked_crc32c(data: bytes) -> int:
    return _native.masked_crc32c(bytes(data))


class TensorBoardLogger:
    def __init__(self, logdir: str):
        os.makedirs(logdir, exist_ok=True)
        self.path = os.path.join(logdir, "events.out.tfevents.%d.nexus" % int(time.time()))
        self._f = open(self.path, "wb")
        self._f.write(_native.tb_version_record(time.time(), "brain.Event:2"))

    def scalar(self, tag: str, value: float, step: int) -> None:
        self._f.write(_native.tb_scalar_record(time.time(), int(step), tag, float(value)))

    def log(self, rec) -> None:
        d = _record_dict(rec)
        for k in ("loss", "lr", "grad_norm", "tokens_per_s", "mfu", "step_ms", "val_loss"):
            v = d.get(k)
            if isinstance(v, (int, float)) and math.isfinite(v):
                self.scalar("train/" + k, v, d["step"])

    def flush(self) -> None:
        self._f.flush()


def read_tensorboard_scalars(path: str) -> List[Tuple[int, str, float]]:
    """(step, tag, value) of every scalar in an event file; both CRCs of every record are verified."""
    with open(path, "rb") as f:
        data = f.read()
    try:
        return [tuple(r) for r in _native.tb_read_scalars(data)]
    except RuntimeError as e:
        raise ValueError(str(e)) from None
