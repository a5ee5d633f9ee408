"""SSA intermediate representation of a language-model training step.

Values carry symbolic shapes: every dimension is ``coef * prod(symbols)`` with the symbols ``B`` and ``T``
bound at run time.  The op set covers the decoder LM (embedding, norms, linear, attention, gated MLP,
shifted cross-entropy), the fused forms produced by the rewrite patterns (``LinearBiasGelu``, ``AddNorm``,
``AttentionQKV``, ``SwiGlu``, ``FusedLinearCE``), communication ops and ``Fused`` element-wise clusters.
Graphs print as text and as Graphviz dot and have a content fingerprint.
Parity: include/nexus/compile/ir.hpp:16-140, src/compile/ir.cpp of the reference."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class Dim:
    coef: int = 1
    syms: Tuple[str, ...] = ()

    @staticmethod
    def of(x) -> "Dim":
        if isinstance(x, Dim):
            return x
        if isinstance(x, int):
            return Dim(x, ())
        return Dim(1, (str(x),))

    def __mul__(self, o) -> "Dim":
        o = Dim.of(o)
        return Dim(self.coef * o.coef, tuple(sorted(self.syms + o.syms)))

    __rmul__ = __mul__

    def bind(self, env: Dict[str, int]) -> int:
        v = self.coef
        for s in self.syms:
            v *= env[s]
        return v

    def __str__(self) -> str:
        if not self.syms:
            return str(self.coef)
        body = "*".join(self.syms)
        return body if self.coef == 1 else f"{self.coef}*{body}"


@dataclass
class Value:
    id: int
    shape: Tuple[Dim, ...]
    dtype: str = "f32"
    name: str = ""
    producer: Optional["Node"] = None

    def __hash__(self):
        return self.id

    def __eq__(self, o):
        return self is o

    def sig(self) -> str:
        return f"%{self.id}:{self.dtype}[{','.join(str(d) for d in self.shape)}]"

    def numel(self, env) -> int:
        n = 1
        for d in self.shape:
            n *= d.bind(env)
        return n


ELEMENTWISE = {"Add", "Mul", "Sub", "Gelu", "Silu", "Scale", "Cast", "Relu", "Tanh", "Sigmoid"}
COMM = {"AllReduce", "AllGather", "ReduceScatter", "AllToAll", "Send", "Recv"}
OPS = ELEMENTWISE | COMM | {"Param", "Input", "Const", "Embedding", "Linear", "Bias", "MatMul", "LayerNorm", "RmsNorm",
                            "Softmax", "SplitQKV", "Attention", "AttentionQKV", "Rope", "SwiGlu", "GeGlu", "GatedSplit",
                            "LinearBiasGelu", "AddNorm", "CrossEntropyShifted", "FusedLinearCE", "Fused", "Reshape",
                            "Transpose", "Vjp", "Accumulate", "Recompute", "Output"}


@dataclass
class Node:
    op: str
    inputs: List[Value]
    outputs: List[Value]
    attrs: Dict[str, object] = field(default_factory=dict)

    def __hash__(self):
        return id(self)

    def __eq__(self, o):
        return self is o


class Graph:
    def __init__(self, name: str = "g"):
        self.name = name
        self.nodes: List[Node] = []
        self.inputs: List[Value] = []
        self.params: Dict[str, Value] = {}
        self.outputs: List[Value] = []
        self._next = 0

    def value(self, shape: Sequence, dtype: str = "f32", name: str = "") -> Value:
        v = Value(self._next, tuple(Dim.of(d) for d in shape), dtype, name)
        self._next += 1
        return v

    def add(self, op: str, inputs: Sequence[Value], out_shapes: Sequence[Sequence], dtype: str = "f32", **attrs) -> List[Value]:
        if op not in OPS:
            raise ValueError(f"unknown op {op!r}")
        outs = [self.value(s, dtype) for s in out_shapes]
        n = Node(op, list(inputs), outs, dict(attrs))
        for o in outs:
            o.producer = n
        self.nodes.append(n)
        return outs

    def param(self, name: str, shape: Sequence[int]) -> Value:
        (v,) = self.add("Param", [], [shape], name=name)
        v.name = name
        self.params[name] = v
        return v

    def input(self, name: str, shape: Sequence, dtype: str = "i32") -> Value:
        (v,) = self.add("Input", [], [shape], dtype=dtype, name=name)
        v.name = name
        self.inputs.append(v)
        return v

    def users(self) -> Dict[Value, List[Node]]:
        u: Dict[Value, List[Node]] = {}
        for n in self.nodes:
            for v in n.inputs:
                u.setdefault(v, []).append(n)
        return u

    def count(self, op: str) -> int:
        return sum(1 for n in self.nodes if n.op == op)

    # ------------------------------------------------------------------ dumps
    @staticmethod
    def _attr_s(a: Dict[str, object]) -> str:
        items = []
        for k in sorted(a):
            v = a[k]
            if isinstance(v, Graph):
                v = f"<graph {v.fingerprint()[:8]}>"
            elif isinstance(v, list) and v and isinstance(v[0], Node):
                v = "[" + ";".join(n.op for n in v) + "]"
            items.append(f"{k}={v}")
        return "{" + ", ".join(items) + "}" if items else ""

    def text(self) -> str:
        lines = [f"graph @{self.name} {{"]
        for n in self.nodes:
            outs = ", ".join(o.sig() for o in n.outputs)
            ins = ", ".join(f"%{v.id}" for v in n.inputs)
            lines.append(f"  {outs} = {n.op}({ins}) {self._attr_s(n.attrs)}".rstrip())
        lines.append("  return " + ", ".join(f"%{v.id}" for v in self.outputs))
        lines.append("}")
        return "\n".join(lines)

    def dot(self) -> str:
        lines = [f'digraph "{self.name}" {{', "  rankdir=TB;"]
        for i, n in enumerate(self.nodes):
            label = n.op + ("\\n" + str(n.attrs.get("name")) if "name" in n.attrs else "")
            shape = "box" if n.op not in ("Param", "Input") else "ellipse"
            lines.append(f'  n{i} [label="{label}", shape={shape}];')
        idx = {id(n): i for i, n in enumerate(self.nodes)}
        for i, n in enumerate(self.nodes):
            for v in n.inputs:
                if v.producer is not None:
                    lines.append(f"  n{idx[id(v.producer)]} -> n{i};")
        lines.append("}")
        return "\n".join(lines)

    def fingerprint(self) -> str:
        """SHA-256 of the canonical text with value ids renumbered in definition order."""
        remap: Dict[int, int] = {}
        parts = []
        for n in self.nodes:
            for o in n.outputs:
                remap[o.id] = len(remap)
            outs = ",".join(f"{remap[o.id]}:{o.dtype}[{','.join(str(d) for d in o.shape)}]" for o in n.outputs)
            ins = ",".join(str(remap.get(v.id, -1)) for v in n.inputs)
            parts.append(f"{outs}={n.op}({ins}){self._attr_s(n.attrs)}")
        parts.append("ret " + ",".join(str(remap.get(v.id, -1)) for v in self.outputs))
        return hashlib.sha256("\n".join(parts).encode()).hexdigest()
