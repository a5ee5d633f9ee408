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
import struct
import time
from typing import Dict, List, Tuple


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
def _crc32c_table():
    poly = 0x82F63B78
    t = []
    for i in range(256):
        c = i
        for _ in range(8):
            c = (c >> 1) ^ poly if c & 1 else c >> 1
        t.append(c)
    return t


_TABLE = _crc32c_table()


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def masked_crc32c(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


def _event(wall_time: float, step: int, tag: str = None, value: float = None, file_version: str = None) -> bytes:
    msg = _field(1, 1, struct.pack("<d", wall_time)) + _field(2, 0, _varint(step))
    if file_version is not None:
        v = file_version.encode()
        msg += _field(3, 2, _varint(len(v)) + v)
    if tag is not None:
        t = tag.encode()
        val = _field(1, 2, _varint(len(t)) + t) + _field(2, 5, struct.pack("<f", value))
        summary = _field(1, 2, _varint(len(val)) + val)
        msg += _field(5, 2, _varint(len(summary)) + summary)
    return msg


def _tfrecord(payload: bytes) -> bytes:
    hdr = struct.pack("<Q", len(payload))
    return hdr + struct.pack("<I", masked_crc32c(hdr)) + payload + struct.pack("<I", masked_crc32c(payload))


class TensorBoardLogger:
    def __init__(self, logdir: str):
        os.makedirs(logdir, exist_ok=True)
        self.path = os.path.join(logdir, "events.out.tfevents.%d.nexus" % int(time.time()))
        self._f = open(self.path, "wb")
        self._f.write(_tfrecord(_event(time.time(), 0, file_version="brain.Event:2")))

    def scalar(self, tag: str, value: float, step: int) -> None:
        self._f.write(_tfrecord(_event(time.time(), step, tag, float(value))))

    def log(self, rec) -> None:
        d = _record_dict(rec)
        for k in ("loss", "lr", "grad_norm", "tokens_per_s", "mfu", "step_ms", "val_loss"):
            v = d.get(k)
            if isinstance(v, (int, float)) and math.isfinite(v):
                self.scalar("train/" + k, v, d["step"])

    def flush(self) -> None:
        self._f.flush()


def read_tensorboard_scalars(path: str) -> List[Tuple[int, str, float]]:
    """Parses an event file written above; verifies both CRCs of every record."""
    out = []
    data = open(path, "rb").read()
    pos = 0

    def varint(buf, i):
        n = shift = 0
        while True:
            b = buf[i]
            i += 1
            n |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                return n, i

    def fields(buf):
        i = 0
        while i < len(buf):
            key, i = varint(buf, i)
            num, wire = key >> 3, key & 7
            if wire == 0:
                v, i = varint(buf, i)
            elif wire == 1:
                v, i = buf[i:i + 8], i + 8
            elif wire == 5:
                v, i = buf[i:i + 4], i + 4
            else:
                ln, i = varint(buf, i)
                v, i = buf[i:i + ln], i + ln
            yield num, wire, v

    while pos < len(data):
        (ln,) = struct.unpack_from("<Q", data, pos)
        if struct.unpack_from("<I", data, pos + 8)[0] != masked_crc32c(data[pos:pos + 8]):
            raise ValueError("tfrecord length CRC mismatch")
        payload = data[pos + 12: pos + 12 + ln]
        if struct.unpack_from("<I", data, pos + 12 + ln)[0] != masked_crc32c(payload):
            raise ValueError("tfrecord payload CRC mismatch")
        pos += 16 + ln
        step, summ = 0, None
        for num, wire, v in fields(payload):
            if num == 2:
                step = v
            elif num == 5:
                summ = v
        if summ is not None:
            for _, _, val in fields(summ):
                tag, fv = None, None
                for n2, _, v2 in fields(val):
                    if n2 == 1:
                        tag = v2.decode()
                    elif n2 == 2:
                        fv = struct.unpack("<f", v2)[0]
                out.append((step, tag, fv))
    return out
