"""ONNX export of the traced LM graph (forward to logits) with a hand-written protobuf encoder.

Opset 17 (LayerNormalization) or 18; dynamic axes ``B`` / ``T`` on the token input and the logits;
weights inline or as external data (one side file, offset / length per tensor).  Ops without a compact
standard form (fused attention over packed heads, rotary embedding, RMS norm) are emitted in the
``ai.nexus`` custom domain with their attributes, so that the file stays loss-less for this framework's
own importer and is still inspectable with standard tools.
Parity: include/nexus/interop/onnx.hpp, src/interop/onnx.cpp of the reference."""
from __future__ import annotations

import os
import struct
from typing import Dict, List, Optional, Tuple

import torch

from ..compile.ir import Graph, Value
from ..compile.trace import trace_lm

FLOAT, INT64, INT32 = 1, 7, 6


# ------------------------------------------------------------------------------------------ protobuf
def _varint(n: int) -> bytes:
    out = bytearray()
    n &= (1 << 64) - 1
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _key(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def f_int(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(v)


def f_bytes(field: int, b: bytes) -> bytes:
    return _key(field, 2) + _varint(len(b)) + b


def f_str(field: int, s: str) -> bytes:
    return f_bytes(field, s.encode())


def f_float(field: int, v: float) -> bytes:
    return _key(field, 5) + struct.pack("<f", v)


def attr(name: str, v) -> bytes:
    body = f_str(1, name)
    if isinstance(v, bool) or isinstance(v, int):
        body += f_int(3, int(v)) + f_int(20, 2)
    elif isinstance(v, float):
        body += f_float(2, v) + f_int(20, 1)
    elif isinstance(v, str):
        body += f_bytes(4, v.encode()) + f_int(20, 3)
    elif isinstance(v, (list, tuple)):
        body += b"".join(f_int(8, int(i)) for i in v) + f_int(20, 7)
    else:
        raise TypeError(f"attribute {name}: {type(v)}")
    return body


def node(op: str, ins: List[str], outs: List[str], name: str = "", domain: str = "", **attrs) -> bytes:
    b = b"".join(f_str(1, i) for i in ins) + b"".join(f_str(2, o) for o in outs)
    b += f_str(3, name or outs[0]) + f_str(4, op)
    b += b"".join(f_bytes(5, attr(k, v)) for k, v in attrs.items())
    if domain:
        b += f_str(7, domain)
    return b


def tensor(name: str, t: torch.Tensor, external: Optional[Tuple[str, int]] = None) -> Tuple[bytes, bytes]:
    """Returns (TensorProto bytes, raw payload to append to the side file or b'')."""
    dt = {torch.float32: FLOAT, torch.int64: INT64, torch.int32: INT32}[t.dtype]
    raw = t.detach().cpu().contiguous().numpy().tobytes()
    b = b"".join(f_int(1, d) for d in t.shape) + f_int(2, dt) + f_str(8, name)
    if external is None:
        return b + f_bytes(9, raw), b""
    loc, off = external
    for k, v in (("location", loc), ("offset", str(off)), ("length", str(len(raw)))):
        b += f_bytes(13, f_str(1, k) + f_str(2, v))
    return b + f_int(14, 1), raw


def value_info(name: str, elem: int, dims: List) -> bytes:
    shape = b"".join(f_bytes(1, f_int(1, d) if isinstance(d, int) else f_str(2, str(d))) for d in dims)
    return f_str(1, name) + f_bytes(2, f_bytes(1, f_int(1, elem) + f_bytes(2, shape)))


# ------------------------------------------------------------------------------------------ export
def export_onnx(model, path: str, opset: int = 17, external_data_threshold: Optional[int] = None) -> Dict[str, int]:
    """Writes ``path`` (and ``path + '.data'`` when weights are external).  Returns node / initializer counts."""
    if opset not in (17, 18):
        raise ValueError("opset must be 17 or 18")
    cfg = model.config
    g: Graph = trace_lm(cfg)
    params = dict(model.named_parameters())
    nodes: List[bytes] = []
    inits: List[bytes] = []
    side = bytearray()
    side_name = os.path.basename(path) + ".data"
    nm = lambda v: v.name if v.name else f"v{v.id}"   # noqa: E731
    transposed: Dict[str, str] = {}

    def init(name: str, t: torch.Tensor) -> None:
        ext = None
        nbytes = t.numel() * t.element_size()
        if external_data_threshold is not None and nbytes >= external_data_threshold:
            pad = (-len(side)) % 64
            side.extend(b"\0" * pad)
            ext = (side_name, len(side))
        proto, raw = tensor(name, t, ext)
        side.extend(raw)
        inits.append(proto)

    logits: Optional[Value] = None
    for n in g.nodes:
        o = [nm(v) for v in n.outputs]
        i = [nm(v) for v in n.inputs]
        if n.op == "Param":
            init(n.attrs["name"], params[n.attrs["name"]].detach().float())
        elif n.op == "Input":
            pass
        elif n.op == "Embedding":
            nodes.append(node("Gather", [i[1], "tokens"], [o[0] + "_tok"]))
            if len(i) > 2:
                nodes.append(node("Gather", [i[2], "positions"], [o[0] + "_pos"]))
                nodes.append(node("Add", [o[0] + "_tok", o[0] + "_pos"], o))
            else:
                nodes.append(node("Identity", [o[0] + "_tok"], o))
        elif n.op == "Linear":
            if i[1] not in transposed:
                transposed[i[1]] = i[1] + "_T"
                nodes.append(node("Transpose", [i[1]], [i[1] + "_T"], perm=[1, 0]))
            nodes.append(node("MatMul", [i[0], transposed[i[1]]], o))
            logits = n.outputs[0]
        elif n.op in ("Bias", "Add"):
            nodes.append(node("Add", i, o))
        elif n.op == "Mul":
            nodes.append(node("Mul", i, o))
        elif n.op == "LayerNorm":
            nodes.append(node("LayerNormalization", i, o, axis=-1, epsilon=float(n.attrs["eps"])))
        elif n.op == "Gelu":
            c = o[0]
            for cname, val in ((c + "_c0", 0.044715), (c + "_c1", 0.7978845608028654), (c + "_h", 0.5), (c + "_one", 1.0)):
                init(cname, torch.tensor(val, dtype=torch.float32))
            nodes += [node("Mul", [i[0], i[0]], [c + "_x2"]), node("Mul", [c + "_x2", i[0]], [c + "_x3"]),
                      node("Mul", [c + "_x3", c + "_c0"], [c + "_a"]), node("Add", [i[0], c + "_a"], [c + "_b"]),
                      node("Mul", [c + "_b", c + "_c1"], [c + "_u"]), node("Tanh", [c + "_u"], [c + "_t"]),
                      node("Add", [c + "_t", c + "_one"], [c + "_p"]), node("Mul", [i[0], c + "_p"], [c + "_q"]),
                      node("Mul", [c + "_q", c + "_h"], o)]
        elif n.op == "Silu":
            nodes += [node("Sigmoid", i, [o[0] + "_s"]), node("Mul", [i[0], o[0] + "_s"], o)]
        elif n.op == "CrossEntropyShifted":
            continue
        else:   # SplitQKV, Attention, Rope, RmsNorm, GatedSplit: custom domain, attributes preserved
            attrs = {k: v for k, v in n.attrs.items() if isinstance(v, (int, float, str, bool))}
            nodes.append(node(n.op, i, o, domain="ai.nexus", **attrs))
    inputs = [value_info("tokens", INT64, ["B", "T"])]
    if cfg.pos == "learned":
        inputs.append(value_info("positions", INT64, ["B", "T"]))
    outputs = [value_info(nm(logits), FLOAT, ["B", "T", logits.shape[-1].coef])]
    graph = b"".join(f_bytes(1, x) for x in nodes) + f_str(2, cfg.name or "lm") + b"".join(f_bytes(5, x) for x in inits) + \
        b"".join(f_bytes(11, x) for x in inputs) + b"".join(f_bytes(12, x) for x in outputs)
    model_b = f_int(1, 8) + f_str(2, "nexus_b200") + f_bytes(7, graph) + f_bytes(8, f_str(1, "") + f_int(2, opset)) + \
        f_bytes(8, f_str(1, "ai.nexus") + f_int(2, 1))
    with open(path, "wb") as f:
        f.write(model_b)
    if side:
        with open(path + ".data", "wb") as f:
            f.write(bytes(side))
    return {"nodes": len(nodes), "initializers": len(inits), "external_bytes": len(side)}


# ------------------------------------------------------------------------------------------ reader (validation)
def parse(buf: bytes) -> List[Tuple[int, int, object]]:
    """Generic protobuf scan: [(field, wire type, value)] (length-delimited values stay bytes)."""
    out, p = [], 0
    while p < len(buf):
        key, sh = 0, 0
        while True:
            b = buf[p]
            p += 1
            key |= (b & 0x7F) << sh
            sh += 7
            if not b & 0x80:
                break
        field, wire = key >> 3, key & 7
        if wire == 0:
            v, sh = 0, 0
            while True:
                b = buf[p]
                p += 1
                v |= (b & 0x7F) << sh
                sh += 7
                if not b & 0x80:
                    break
        elif wire == 2:
            n, sh = 0, 0
            while True:
                b = buf[p]
                p += 1
                n |= (b & 0x7F) << sh
                sh += 7
                if not b & 0x80:
                    break
            v = buf[p: p + n]
            p += n
        elif wire == 5:
            v = struct.unpack_from("<f", buf, p)[0]
            p += 4
        elif wire == 1:
            v = struct.unpack_from("<d", buf, p)[0]
            p += 8
        else:
            raise ValueError(f"unsupported wire type {wire}")
        out.append((field, wire, v))
    return out
