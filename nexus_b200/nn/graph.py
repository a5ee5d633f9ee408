"""`nn.Graph`: a named multi-input DAG of catalog layers.

``add(name, layer)`` chains after the previous node; ``add(name, layer, inputs, concatenate)``
merges several named inputs by summation (merge kind 1) or by concatenation on the last axis
(merge kind 32); ``"input"`` names the graph input.  Backward runs in reverse order, a concat
splits its gradient and fan-out sums (autograd does both here).  Unknown names and cycles raise
``ValueError``.  Archives carry ``graph_name``, ``graph_inputs`` (comma-joined) and
``graph_merge`` on every child.

Parity: include/nexus/nn/graph.inl:13-15,144-360 of the reference.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as tnn

from .modules import I32, KIND, STR, Module, make_one

MERGE_SINGLE, MERGE_ADD, MERGE_CONCAT = 0, 1, 32


class Graph(Module):
    kind = KIND["Graph"]
    INPUT = "input"

    def __init__(self):
        super().__init__()
        self.nodes = tnn.ModuleDict()
        self.order: List[str] = []
        self.inputs: Dict[str, List[str]] = {}
        self.merge: Dict[str, int] = {}
        self.output: Optional[str] = None

    def add(self, name: str, layer: Module, inputs: Optional[Sequence[str]] = None, concatenate: bool = False) -> "Graph":
        if name == self.INPUT or name in self.nodes:
            raise ValueError(f"graph node name '{name}' is reserved or already used")
        if inputs is None:
            inputs = [self.order[-1] if self.order else self.INPUT]
        inputs = list(inputs)
        if not inputs:
            raise ValueError("a graph node needs at least one input")
        for i in inputs:
            if i != self.INPUT and i not in self.nodes:
                raise ValueError(f"unknown graph input '{i}' (nodes must be added after their inputs: no cycles)")
        self.nodes[name] = layer
        self.order.append(name)
        self.inputs[name] = inputs
        self.merge[name] = MERGE_SINGLE if len(inputs) == 1 else (MERGE_CONCAT if concatenate else MERGE_ADD)
        self.output = name
        return self

    def concat(self, name: str, layer: Module, inputs: Sequence[str]) -> "Graph":
        return self.add(name, layer, inputs, concatenate=True)

    def set_output(self, name: str) -> "Graph":
        if name not in self.nodes:
            raise ValueError(f"unknown graph node '{name}'")
        self.output = name
        return self

    def forward(self, x):
        vals = {self.INPUT: x}
        for name in self.order:
            ins = [vals[i] for i in self.inputs[name]]
            m = self.merge[name]
            if m == MERGE_SINGLE:
                h = ins[0]
            elif m == MERGE_ADD:
                h = ins[0]
                for t in ins[1:]:
                    h = h + t
            else:
                h = torch.cat(ins, dim=-1)
            vals[name] = self.nodes[name](h)
        return vals[self.output]

    # ------------------------------------------------------------------------------ archive
    def nxs_spec(self) -> dict:
        children = []
        for name in self.order:
            spec = self.nodes[name].nxs_spec()
            spec["attrs"] = list(spec["attrs"]) + [("graph_name", STR, name),
                                                   ("graph_inputs", STR, ",".join(self.inputs[name])),
                                                   ("graph_merge", I32, self.merge[name])]
            children.append(spec)
        return {"type": self.kind, "name": "Graph", "attrs": [("graph_output", STR, self.output or "")],
                "children": children}

    @staticmethod
    def from_spec(spec: dict) -> "Graph":
        g = Graph()
        for child in spec["children"]:
            meta = {k: v for k, _, v in child["attrs"] if k.startswith("graph_")}
            plain = dict(child)
            plain["attrs"] = [a for a in child["attrs"] if not a[0].startswith("graph_")]
            inputs = meta["graph_inputs"].split(",") if meta.get("graph_inputs") else None
            g.add(meta["graph_name"], make_one(plain), inputs, meta.get("graph_merge", 0) == MERGE_CONCAT)
        out = next((v for k, _, v in spec["attrs"] if k == "graph_output"), "")
        if out:
            g.set_output(out)
        return g

    restore = from_spec

    def save_nxs(self, path: str) -> None:
        from ..nxs.archive import save_model
        save_model(self, path)

    @staticmethod
    def load_nxs(path: str) -> "Graph":
        from ..nxs.archive import load_model
        return load_model(path)
