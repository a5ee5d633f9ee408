"""StableHLO export / CPU reference interpreter, GSPMD sharding annotations and the PJRT plugin loader.

* ``StableHloModule``: a small SSA builder that prints MLIR text (`stablehlo.add`, `multiply`, `subtract`,
  `divide`, `maximum`, `exponential`, `tanh`, `logistic`, `negate`, `dot_general`, `reduce` (sum/max),
  `broadcast_in_dim`, `reshape`, `transpose`, `constant`) and can be evaluated on the CPU.
* ``sharding_annotation``: DeviceMesh + DTensor placements -> ``mhlo.sharding`` strings
  (`{replicated}`, `{devices=[a,b,...]0,1,...}`, with `last_tile_dim_replicate` for partial replication).
* ``PjrtDriver``: loads a PJRT C-API plugin named by ``PJRT_PLUGIN_LIBRARY_PATH`` and checks the
  ``GetPjrtApi`` entry point; without a plugin it reports unavailable.
Parity: include/nexus/backend/pjrt.hpp, src/backend/pjrt.cpp of the reference."""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .driver import Driver, Kind


@dataclass
class _Val:
    name: str
    shape: Tuple[int, ...]


@dataclass
class _Op:
    kind: str
    out: _Val
    ins: List[_Val]
    attrs: dict = field(default_factory=dict)


class StableHloModule:
    def __init__(self, name: str = "main"):
        self.name = name
        self.args: List[_Val] = []
        self.ops: List[_Op] = []
        self.results: List[_Val] = []
        self.arg_sharding: Dict[str, str] = {}
        self._n = 0

    @staticmethod
    def _ty(shape) -> str:
        return "tensor<" + "".join(f"{d}x" for d in shape) + "f32>"

    def _new(self, shape) -> _Val:
        self._n += 1
        return _Val(f"%{self._n}", tuple(int(d) for d in shape))

    def arg(self, shape, sharding: Optional[str] = None) -> _Val:
        v = _Val(f"%arg{len(self.args)}", tuple(int(d) for d in shape))
        self.args.append(v)
        if sharding:
            self.arg_sharding[v.name] = sharding
        return v

    def _emit(self, kind, shape, ins, **attrs) -> _Val:
        out = self._new(shape)
        self.ops.append(_Op(kind, out, list(ins), attrs))
        return out

    def constant(self, value: float, shape=()) -> _Val:
        return self._emit("constant", shape, [], value=float(value))

    def binary(self, kind: str, a: _Val, b: _Val) -> _Val:
        if a.shape != b.shape:
            raise ValueError(f"{kind}: shapes differ {a.shape} vs {b.shape}")
        return self._emit(kind, a.shape, [a, b])

    def add(self, a, b):
        return self.binary("add", a, b)

    def multiply(self, a, b):
        return self.binary("multiply", a, b)

    def subtract(self, a, b):
        return self.binary("subtract", a, b)

    def divide(self, a, b):
        return self.binary("divide", a, b)

    def maximum(self, a, b):
        return self.binary("maximum", a, b)

    def unary(self, kind: str, a: _Val) -> _Val:
        return self._emit(kind, a.shape, [a])

    def dot_general(self, a: _Val, b: _Val, contract: Tuple[int, int], batch: Tuple[Sequence[int], Sequence[int]] = ((), ())):
        ba, bb = list(batch[0]), list(batch[1])
        ca, cb = contract
        shape = [a.shape[i] for i in ba] + [d for i, d in enumerate(a.shape) if i not in ba and i != ca] + \
                [d for i, d in enumerate(b.shape) if i not in bb and i != cb]
        return self._emit("dot_general", shape, [a, b], contract=(ca, cb), batch=(ba, bb))

    def reduce(self, a: _Val, dims: Sequence[int], kind: str = "sum") -> _Val:
        shape = [d for i, d in enumerate(a.shape) if i not in dims]
        return self._emit("reduce", shape, [a], dims=list(dims), how=kind)

    def broadcast_in_dim(self, a: _Val, shape, dims: Sequence[int]) -> _Val:
        return self._emit("broadcast_in_dim", shape, [a], dims=list(dims))

    def reshape(self, a: _Val, shape) -> _Val:
        return self._emit("reshape", shape, [a])

    def transpose(self, a: _Val, perm: Sequence[int]) -> _Val:
        return self._emit("transpose", [a.shape[i] for i in perm], [a], perm=list(perm))

    def ret(self, *vals: _Val) -> None:
        self.results = list(vals)

    # -------------------------------------------------------------------------------- text
    def text(self) -> str:
        def arg_s(a):
            s = f"{a.name}: {self._ty(a.shape)}"
            if a.name in self.arg_sharding:
                s += f' {{mhlo.sharding = "{self.arg_sharding[a.name]}"}}'
            return s
        lines = [f"module @{self.name} {{",
                 f"  func.func public @main({', '.join(arg_s(a) for a in self.args)}) -> "
                 f"({', '.join(self._ty(r.shape) for r in self.results)}) {{"]
        for op in self.ops:
            o, ty = op.out, self._ty(op.out.shape)
            ins = ", ".join(v.name for v in op.ins)
            in_tys = ", ".join(self._ty(v.shape) for v in op.ins)
            if op.kind == "constant":
                lines.append(f"    {o.name} = stablehlo.constant dense<{op.attrs['value']:e}> : {ty}")
            elif op.kind == "dot_general":
                (ca, cb), (ba, bb) = op.attrs["contract"], op.attrs["batch"]
                lines.append(f"    {o.name} = stablehlo.dot_general {ins}, batching_dims = {ba} x {bb}, "
                             f"contracting_dims = [{ca}] x [{cb}] : ({in_tys}) -> {ty}")
            elif op.kind == "reduce":
                body = "stablehlo.add" if op.attrs["how"] == "sum" else "stablehlo.maximum"
                lines.append(f"    {o.name} = stablehlo.reduce({ins}) applies {body} across dimensions = "
                             f"{op.attrs['dims']} : ({in_tys}) -> {ty}")
            elif op.kind == "broadcast_in_dim":
                lines.append(f"    {o.name} = stablehlo.broadcast_in_dim {ins}, dims = {op.attrs['dims']} : "
                             f"({in_tys}) -> {ty}")
            elif op.kind == "transpose":
                lines.append(f"    {o.name} = stablehlo.transpose {ins}, dims = {op.attrs['perm']} : ({in_tys}) -> {ty}")
            elif op.kind == "reshape":
                lines.append(f"    {o.name} = stablehlo.reshape {ins} : ({in_tys}) -> {ty}")
            else:
                lines.append(f"    {o.name} = stablehlo.{op.kind} {ins} : {ty}")
        lines.append(f"    return {', '.join(r.name for r in self.results)} : "
                     f"{', '.join(self._ty(r.shape) for r in self.results)}")
        lines += ["  }", "}"]
        return "\n".join(lines)

    # -------------------------------------------------------------------------------- interpreter
    def run(self, *inputs: np.ndarray) -> List[np.ndarray]:
        if len(inputs) != len(self.args):
            raise ValueError("argument count mismatch")
        env: Dict[str, np.ndarray] = {}
        for a, x in zip(self.args, inputs):
            x = np.asarray(x, dtype=np.float32)
            if x.shape != a.shape:
                raise ValueError(f"argument {a.name}: shape {x.shape} != {a.shape}")
            env[a.name] = x
        un = {"exponential": np.exp, "tanh": np.tanh, "negate": np.negative, "log": np.log, "sqrt": np.sqrt,
              "rsqrt": lambda v: 1 / np.sqrt(v), "logistic": lambda v: 1 / (1 + np.exp(-v))}
        bi = {"add": np.add, "multiply": np.multiply, "subtract": np.subtract, "divide": np.divide,
              "maximum": np.maximum}
        for op in self.ops:
            x = [env[v.name] for v in op.ins]
            if op.kind == "constant":
                r = np.full(op.out.shape, op.attrs["value"], dtype=np.float32)
            elif op.kind in bi:
                r = bi[op.kind](x[0], x[1])
            elif op.kind in un:
                r = un[op.kind](x[0])
            elif op.kind == "dot_general":
                (ca, cb), (ba, bb) = op.attrs["contract"], op.attrs["batch"]
                la = "abcdefgh"[: x[0].ndim]
                lb = list("ijklmnop"[: x[1].ndim])
                lb[cb] = la[ca]
                for i, j in zip(ba, bb):
                    lb[j] = la[i]
                outl = [la[i] for i in ba] + [c for i, c in enumerate(la) if i not in ba and i != ca] + \
                       [c for j, c in enumerate(lb) if j not in bb and j != cb]
                r = np.einsum(f"{la},{''.join(lb)}->{''.join(outl)}", x[0].astype(np.float64), x[1].astype(np.float64))
            elif op.kind == "reduce":
                f = np.sum if op.attrs["how"] == "sum" else np.max
                r = f(x[0].astype(np.float64), axis=tuple(op.attrs["dims"]))
            elif op.kind == "broadcast_in_dim":
                shape = [1] * len(op.out.shape)
                for src, dst in enumerate(op.attrs["dims"]):
                    shape[dst] = x[0].shape[src]
                r = np.broadcast_to(x[0].reshape(shape), op.out.shape)
            elif op.kind == "reshape":
                r = x[0].reshape(op.out.shape)
            elif op.kind == "transpose":
                r = x[0].transpose(op.attrs["perm"])
            else:
                raise NotImplementedError(f"stablehlo.{op.kind}")
            env[op.out.name] = np.asarray(r, dtype=np.float32)
        return [env[r.name] for r in self.results]


def sharding_annotation(mesh_shape: Sequence[int], placements: Sequence, rank: int) -> str:
    """GSPMD sharding of a rank-``rank`` tensor on a row-major mesh.  ``placements[i]`` describes mesh
    dimension i: ``("shard", d)``, ``"replicate"`` or ``"partial"`` (also objects with ``.kind`` / ``.dim``)."""
    def norm(p):
        if isinstance(p, str):
            return p.lower(), None
        if isinstance(p, tuple):
            return p[0].lower(), p[1]
        return getattr(p, "kind", type(p).__name__).lower(), getattr(p, "dim", None)
    tile = [1] * rank
    order_mesh_dims = []
    replicated_mesh_dims = []
    for i, p in enumerate(placements):
        kind, d = norm(p)
        if kind == "shard":
            if tile[d] != 1:
                raise ValueError("two mesh dimensions shard the same tensor dimension")
            tile[d] = mesh_shape[i]
            order_mesh_dims.append((d, i))
        else:
            replicated_mesh_dims.append(i)
    if not order_mesh_dims:
        return "{replicated}"
    # device order: iterate tensor dims in order, then the replicated mesh dims last
    mesh = np.arange(int(np.prod(mesh_shape))).reshape(mesh_shape)
    perm = [i for _, i in sorted(order_mesh_dims)] + replicated_mesh_dims
    devs = mesh.transpose(perm).reshape(-1)
    rep = int(np.prod([mesh_shape[i] for i in replicated_mesh_dims])) if replicated_mesh_dims else 1
    dims = tile + ([rep] if rep > 1 else [])
    tail = " last_tile_dim_replicate" if rep > 1 else ""
    return "{devices=[" + ",".join(str(d) for d in dims) + "]" + ",".join(str(int(d)) for d in devs) + tail + "}"


class PjrtDriver(Driver):
    def __init__(self):
        super().__init__()
        self._lib = None
        self._why = ""
        path = os.environ.get("PJRT_PLUGIN_LIBRARY_PATH", "")
        if not path:
            self._why = "no PJRT plugin configured (PJRT_PLUGIN_LIBRARY_PATH is empty)"
            return
        try:
            self._lib = ctypes.CDLL(path)
            if not hasattr(self._lib, "GetPjrtApi"):
                self._why, self._lib = f"{path} exports no GetPjrtApi", None
        except OSError as e:
            self._why = f"cannot load {path}: {e}"

    def kind(self):
        return Kind.Pjrt

    def name(self):
        return "pjrt"

    def unavailable_reason(self):
        return self._why or "the plugin loaded, but executing through PJRT is not wired in this build"
