"""safetensors reader (memory-mapped, strict validation) and writer.

File = u64 little-endian header length, JSON header {name: {dtype, shape, data_offsets:[b, e]}, ...,
"__metadata__": {str: str}}, then the byte buffer.  The reader rejects: a header longer than the file or
100 MB, invalid JSON, duplicate names, unknown dtypes, negative or overflowing shapes, offsets that do not
match shape x dtype size, overlapping or out-of-range ranges, and holes in the buffer.
Parity: include/nexus/interop/safetensors.hpp, src/interop/safetensors.cpp of the reference."""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from typing import Dict, Optional

import numpy as np
import torch

_DT = {"F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
       "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
       "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1),
       "F8_E5M2": (torch.float8_e5m2, 1)}
_NAME = {v[0]: k for k, v in _DT.items()}
MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


def _no_dup(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise SafetensorsError(f"duplicate key {k!r} in the header")
        out[k] = v
    return out


class SafetensorsFile:
    """Zero-copy view of a file: tensors alias the memory map (read-only)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = self._f.seek(0, 2)
        if size < 8:
            raise SafetensorsError("file shorter than the 8-byte header length")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"header length {hlen} exceeds the file or the {MAX_HEADER}-byte limit")
        try:
            header = json.loads(self._mm[8: 8 + hlen].decode("utf-8"), object_pairs_hook=_no_dup)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"invalid header JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError("the header is not a JSON object")
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        if not all(isinstance(k, str) and isinstance(v, str) for k, v in self.metadata.items()):
            raise SafetensorsError("__metadata__ must map strings to strings")
        self._base = 8 + hlen
        data_len = size - self._base
        self.entries: Dict[str, dict] = {}
        spans = []
        for name, e in header.items():
            if not isinstance(e, dict) or set(e) - {"dtype", "shape", "data_offsets"} or len(e) != 3:
                raise SafetensorsError(f"{name}: entry must have exactly dtype, shape, data_offsets")
            if e["dtype"] not in _DT:
                raise SafetensorsError(f"{name}: unknown dtype {e['dtype']!r}")
            shape, off = e["shape"], e["data_offsets"]
            if not isinstance(shape, list) or any((not isinstance(d, int)) or isinstance(d, bool) or d < 0 for d in shape):
                raise SafetensorsError(f"{name}: bad shape {shape!r}")
            if (not isinstance(off, list)) or len(off) != 2 or any((not isinstance(o, int)) or isinstance(o, bool) for o in off):
                raise SafetensorsError(f"{name}: bad data_offsets {off!r}")
            n = 1
            for d in shape:
                n *= d
                if n > (1 << 62):
                    raise SafetensorsError(f"{name}: element count overflows")
            b, en = off
            if b < 0 or en < b or en > data_len:
                raise SafetensorsError(f"{name}: data_offsets {off} outside the buffer of {data_len} bytes")
            if en - b != n * _DT[e["dtype"]][1]:
                raise SafetensorsError(f"{name}: {en - b} bytes for shape {shape} of {e['dtype']}")
            spans.append((b, en, name))
            self.entries[name] = e
        spans.sort()
        pos = 0
        for b, en, name in spans:
            if b < pos:
                raise SafetensorsError(f"{name}: overlaps the previous tensor")
            if b > pos:
                raise SafetensorsError(f"{name}: hole of {b - pos} bytes before it")
            pos = en
        if pos != data_len:
            raise SafetensorsError(f"{data_len - pos} trailing bytes after the last tensor")

    def keys(self):
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        dt, size = _DT[e["dtype"]]
        b, en = e["data_offsets"]
        raw = np.frombuffer(self._mm, dtype=np.uint8, count=en - b, offset=self._base + b)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)
            t = torch.from_numpy(raw)          # aliases the map (read-only memory: clone before writing)
        return t.view(dt).view(e["shape"]) if en > b else torch.empty(e["shape"], dtype=dt)

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass                                # tensors still alias the map
        self._f.close()


def load_file(path: str, device: str = "cpu") -> Dict[str, torch.Tensor]:
    f = SafetensorsFile(path)
    return {k: f.tensor(k).clone().to(device) for k in f.keys()}


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    header, pos, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):            # sorted: the file is reproducible
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAME:
            raise SafetensorsError(f"{name}: dtype {t.dtype} has no safetensors name")
        raw = t.view(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAME[t.dtype], "shape": list(t.shape), "data_offsets": [pos, pos + len(raw)]}
        pos += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((-len(hj)) % 8)            # keep the data 8-byte aligned
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)
