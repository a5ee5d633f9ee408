"""Executor for (joint) graphs and the ``CompiledLm`` front end.

Values live in a table; forward nodes run through torch (and this framework's fused ops), ``Fused``
clusters through their JIT-compiled kernels, ``Vjp`` nodes through the local autograd graph of the forward
node they differentiate, communication nodes through a process group.  ``CompiledLm`` traces a model's
config, runs the pass pipeline, binds the model's own parameters and offers ``loss`` /
``loss_and_grads``, an autotuner that times two pipeline variants, CUDA-graph capture on the GPU, and
StableHLO / HLO text export.
Parity: include/nexus/compile/compile.hpp:31-120, src/compile/executor.cpp, src/compile/compile.cpp of the
reference (arena executor on CPU threads)."""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..fused import ops as F_
from ..lm.config import LmConfig
from ..lm.rope import RopeCache, apply_rope
from . import passes as P
from .codegen import FusedKernel
from .ir import Graph, Node, Value
from .trace import trace_lm


class Executor:
    def __init__(self, graph: Graph, params: Dict[str, torch.Tensor], cfg: Optional[LmConfig] = None, group=None,
                 jit: bool = True):
        self.g, self.params, self.cfg, self.group, self.jit = graph, params, cfg, group, jit
        self._kernels: Dict[int, FusedKernel] = {}
        self._rope: Optional[RopeCache] = None

    # ------------------------------------------------------------------ single node semantics
    def _rope_cache(self, dev) -> RopeCache:
        if self._rope is None:
            self._rope = RopeCache(self.cfg)
        if self._rope.cos.device != dev:
            self._rope.to(dev)
        return self._rope

    def _attention(self, q, k, v, attrs):
        o = F_.attention(q, k, v, causal=bool(attrs.get("causal", True)), window=int(attrs.get("window", 0)))
        return o.reshape(o.shape[0], o.shape[1], -1)

    def _split(self, qkv, H, Hk):
        B, T, _ = qkv.shape
        D = qkv.shape[-1] // (H + 2 * Hk)
        if H == Hk:
            q5 = qkv.view(B, T, 3, H, D)
            return q5[:, :, 0], q5[:, :, 1], q5[:, :, 2]
        return (qkv[..., : H * D].view(B, T, H, D), qkv[..., H * D: (H + Hk) * D].view(B, T, Hk, D),
                qkv[..., (H + Hk) * D:].view(B, T, Hk, D))

    def _run(self, n: Node, x: List[torch.Tensor]):
        op, a = n.op, n.attrs
        if op == "Embedding":
            y = x[1][x[0].long()]
            return [y + x[2][: x[0].shape[1]][None] if len(x) > 2 else y]
        if op == "Linear":
            return [F.linear(x[0], x[1], x[2] if len(x) > 2 else None)]
        if op == "LinearBiasGelu":
            return [F.gelu(F.linear(x[0], x[1], x[2]), approximate="tanh")]
        if op == "Bias":
            return [x[0] + x[1]]
        if op == "Add":
            return [x[0] + x[1]]
        if op == "Sub":
            return [x[0] - x[1]]
        if op == "Mul":
            return [x[0] * x[1]]
        if op == "Scale":
            return [x[0] * float(a["factor"])]
        if op == "Gelu":
            return [F.gelu(x[0], approximate="tanh")]
        if op == "Silu":
            return [F.silu(x[0])]
        if op in ("Relu", "Tanh", "Sigmoid"):
            return [getattr(torch, op.lower())(x[0])]
        if op == "Const":
            return [torch.full((), float(a["value"]), device=self._dev)]   # a fill kernel: safe under graph capture
        if op == "LayerNorm":
            return [F.layer_norm(x[0], x[0].shape[-1:], x[1], x[2], float(a["eps"]))]
        if op == "RmsNorm":
            return [F_.rms_norm(x[0], x[1], float(a["eps"]))]
        if op == "AddNorm":
            s = x[0] + x[1]
            if a["kind"] == "LayerNorm":
                return [s, F.layer_norm(s, s.shape[-1:], x[2], x[3], float(a["eps"]))]
            return [s, F_.rms_norm(s, x[2], float(a["eps"]))]
        if op == "SplitQKV":
            return list(self._split(x[0], int(a["heads"]), int(a["kv_heads"])))
        if op == "Rope":
            rc = self._rope_cache(x[0].device)
            return [apply_rope(x[0], rc.cos, rc.sin, None)]
        if op == "Attention":
            return [self._attention(x[0], x[1], x[2], a)]
        if op == "AttentionQKV":
            q, k, v = self._split(x[0], int(a["heads"]), int(a["kv_heads"]))
            return [self._attention(q, k, v, a)]
        if op == "GatedSplit":
            h = x[0].shape[-1] // 2
            return [x[0][..., :h], x[0][..., h:]]
        if op in ("SwiGlu", "GeGlu"):
            h = x[0].shape[-1] // 2
            g = F.silu(x[0][..., :h]) if op == "SwiGlu" else F.gelu(x[0][..., :h], approximate="tanh")
            return [g * x[0][..., h:]]
        if op == "CrossEntropyShifted":
            return [F_.cross_entropy_shifted(x[0], x[1], vocab=int(a["vocab"]))]
        if op == "FusedLinearCE":
            return [F_.cross_entropy_shifted(F.linear(x[0], x[1]), x[2], vocab=int(a["vocab"]))]
        if op == "Fused":
            return self._fused(n, x)
        if op == "Accumulate":
            return [x[0] + x[1]]
        if op in ("AllReduce", "AllGather", "ReduceScatter"):
            if self.group is None or self.group.size() == 1:
                return [x[0]]
            t = x[0].contiguous().clone()
            if op == "AllReduce":
                self.group.all_reduce_tensor(t)
                return [t]
            raise NotImplementedError(op)
        if op == "Reshape":
            return [x[0].reshape(a["shape"])]
        raise NotImplementedError(f"executor: op {op}")

    def _fused(self, n: Node, x: List[torch.Tensor]):
        body = n.attrs["body"]
        if n.attrs.get("kind") == "horizontal":
            out_steps = list(range(len(body)))
        else:
            out_steps = [len(body) - 1]
        if self.jit and not any(t.requires_grad for t in x) and all(t.dtype == torch.float32 for t in x):
            k = self._kernels.get(id(n))
            if k is None:
                k = self._kernels[id(n)] = FusedKernel(body, len(x), out_steps)
            return k(*x)
        tmp: List[torch.Tensor] = []
        for op, attrs, srcs in body:      # reference semantics (also the differentiable path)
            ins = [x[i] if kind == "in" else tmp[i] for kind, i in srcs]
            tmp.append(self._run(Node(op, [], [], attrs), ins)[0])
        return [tmp[s] for s in out_steps]

    # ------------------------------------------------------------------ whole graph
    def run(self, tokens: torch.Tensor, want_grads: bool = False):
        env: Dict[int, torch.Tensor] = {}
        self._dev = tokens.device
        taped: Dict[int, tuple] = {}
        joint = any(n.op == "Vjp" for n in self.g.nodes)
        for n in self.g.nodes:
            if n.op == "Param":
                env[n.outputs[0].id] = self.params[n.attrs["name"]]
                continue
            if n.op == "Input":
                env[n.outputs[0].id] = tokens
                continue
            if n.op == "Vjp":
                if not want_grads:
                    continue
                f: Node = n.attrs["fwd"]
                ins, outs = taped[id(f)]
                have = n.attrs["have"]
                acc = n.attrs.get("accumulate", {})       # output index -> input position of a running sum (beta = 1)
                n_g = len(n.inputs) - len(acc)
                gouts = [env[v.id] for v in n.inputs[len(f.inputs) + len(f.outputs):n_g]]
                wrt = [ins[i] for i in n.attrs["wrt"]]
                gs = torch.autograd.grad([outs[i] for i in have], wrt, gouts, allow_unused=True)
                for k, (o, gval, w) in enumerate(zip(n.outputs, gs, wrt)):
                    gval = gval if gval is not None else torch.zeros_like(w)
                    env[o.id] = env[n.inputs[acc[k]].id] + gval if k in acc else gval
                continue
            if n.op == "Accumulate" and not want_grads:
                continue
            x = [env[v.id] for v in n.inputs]
            if joint and want_grads and n.op not in ("Const", "Accumulate"):
                x = [t.detach().requires_grad_(True) if t.is_floating_point() else t for t in x]
                with torch.enable_grad():
                    y = self._run(n, x)
                taped[id(n)] = (x, y)
                y = list(y)
            else:
                with torch.no_grad():
                    y = self._run(n, x)
            for o, t in zip(n.outputs, y):
                env[o.id] = t
        outs = [env[v.id] for v in self.g.outputs if v.id in env]
        return outs


@dataclass
class CompileOptions:
    patterns: int = P.P_ALL
    fuse: bool = True
    jit: bool = True
    joint: bool = True
    epilogues: bool = True       # fold gradient accumulation / DGELU / bias gradients into the backward nodes
    cuda_graph: bool = False


class CompiledLm:
    def __init__(self, model, options: Optional[CompileOptions] = None, group=None):
        self.model, self.opt = model, options or CompileOptions()
        cfg = model.config
        g = trace_lm(cfg)
        self.traced_fingerprint = g.fingerprint()
        self.stats = {"patterns": P.rewrite_patterns(g, self.opt.patterns)}
        self.stats["cse"] = P.cse(g)
        self.stats["dce"] = P.dce(g)
        if self.opt.fuse:
            self.stats["fusion"] = P.fuse_elementwise(g)
        self.forward_nodes = len(g.nodes)
        self.pgrads: Dict[str, Value] = {}
        if self.opt.joint:
            g, self.pgrads = P.build_joint(g)
            if self.opt.epilogues:
                self.stats["epilogues"] = P.fuse_epilogues(g)
        self.graph = g
        params = dict(model.named_parameters())
        self.exec = Executor(g, {k: params[k] for k in g.params}, cfg, group, jit=self.opt.jit)
        self._cg = None

    def loss(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.exec.run(tokens, want_grads=False)[0]

    def loss_and_grads(self, tokens: torch.Tensor):
        outs = self.exec.run(tokens, want_grads=True)
        return outs[0], dict(zip(self.pgrads.keys(), outs[1:]))

    def memory_plan(self, batch: int, seq: int):
        return P.plan_memory(self.graph, {"B": batch, "T": seq})

    def recompute_plan(self, batch: int, seq: int):
        return P.min_cut_recompute(self.graph, {"B": batch, "T": seq})

    def capture(self, tokens: torch.Tensor):
        """CUDA graph of loss_and_grads for this token shape (GPU only); returns a replay callable."""
        static_tokens = tokens.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.loss_and_grads(static_tokens)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            loss, grads = self.loss_and_grads(static_tokens)

        def replay(new_tokens):
            static_tokens.copy_(new_tokens)
            graph.replay()
            return loss, grads
        return replay

    # ------------------------------------------------------------------ export
    def export_stablehlo(self, batch: int, seq: int) -> str:
        """StableHLO text of the forward graph's dense sub-ops (linear / add / gelu chains are lowered op by
        op; attention, norms and the loss appear as `stablehlo.custom_call` with their attributes)."""
        env = {"B": batch, "T": seq}
        ty = lambda v: "tensor<" + "".join(f"{d.bind(env)}x" for d in v.shape) + ("i32>" if v.dtype == "i32" else "f32>")  # noqa: E731
        args = [v for n in self.graph.nodes if n.op in ("Param", "Input") for v in n.outputs]
        lines = [f"module @{self.graph.name} {{", "  func.func public @main(" +
                 ", ".join(f"%{v.id}: {ty(v)}" for v in args) + f") -> ({ty(self.graph.outputs[0])}) {{"]
        simple = {"Add": "add", "Mul": "multiply", "Sub": "subtract", "Tanh": "tanh", "Sigmoid": "logistic",
                  "Accumulate": "add"}
        for n in self.graph.nodes[: self.forward_nodes]:
            if n.op in ("Param", "Input"):
                continue
            ins = ", ".join(f"%{v.id}" for v in n.inputs)
            o = n.outputs[0]
            if n.op in simple and all(v.shape == o.shape for v in n.inputs):
                lines.append(f"    %{o.id} = stablehlo.{simple[n.op]} {ins} : {ty(o)}")
            elif n.op == "Linear":
                r = len(n.inputs[0].shape) - 1
                x_, w_ = n.inputs[0], n.inputs[1]
                mm = f"%{o.id}" if len(n.inputs) == 2 else f"%{o.id}_mm"
                lines.append(f"    {mm} = stablehlo.dot_general %{x_.id}, %{w_.id}, contracting_dims = [{r}] x [1] : "
                             f"({ty(x_)}, {ty(w_)}) -> {ty(o)}")
                if len(n.inputs) == 3:
                    lines.append(f"    %{o.id}_b = stablehlo.broadcast_in_dim %{n.inputs[2].id}, dims = [{r}] : "
                                 f"({ty(n.inputs[2])}) -> {ty(o)}")
                    lines.append(f"    %{o.id} = stablehlo.add {mm}, %{o.id}_b : {ty(o)}")
            else:
                outs = ", ".join(f"%{v.id}" for v in n.outputs)
                attrs = ", ".join(f'{k} = "{v}"' for k, v in sorted(n.attrs.items()) if isinstance(v, (int, float, str, bool)))
                lines.append(f"    {outs} = stablehlo.custom_call @nexus.{n.op}({ins}) {{{attrs}}} : "
                             f"({', '.join(ty(v) for v in n.inputs)}) -> ({', '.join(ty(v) for v in n.outputs)})")
        lines += [f"    return %{self.graph.outputs[0].id} : {ty(self.graph.outputs[0])}", "  }", "}"]
        return "\n".join(lines)

    def export_hlo_text(self, batch: int, seq: int) -> str:
        env = {"B": batch, "T": seq}
        lines = [f"HloModule {self.graph.name}", "", "ENTRY main {"]
        for n in self.graph.nodes[: self.forward_nodes]:
            for o in n.outputs:
                shp = "f32[" + ",".join(str(d.bind(env)) for d in o.shape) + "]"
                ins = ", ".join(f"v{v.id}" for v in n.inputs)
                lines.append(f"  v{o.id} = {shp} {n.op.lower()}({ins})")
        lines += [f"  ROOT out = f32[] copy(v{self.graph.outputs[0].id})", "}"]
        return "\n".join(lines)


def compile_lm(model, options: Optional[CompileOptions] = None, group=None) -> CompiledLm:
    return CompiledLm(model, options, group)


def autotune(model, tokens: torch.Tensor, variants=None, iters: int = 3):
    """Times ``loss_and_grads`` for two (or more) pipeline variants and returns (best CompiledLm, timings)."""
    variants = variants or [CompileOptions(), CompileOptions(patterns=0, fuse=False)]
    results = []
    for opt in variants:
        c = CompiledLm(model, opt)
        c.loss_and_grads(tokens)
        t0 = time.perf_counter()
        for _ in range(iters):
            c.loss_and_grads(tokens)
        if tokens.is_cuda:
            torch.cuda.synchronize()
        results.append(((time.perf_counter() - t0) / iters, c))
    best = min(results, key=lambda r: r[0])
    return best[1], [r[0] for r in results]
