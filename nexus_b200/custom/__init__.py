"""User extension points: `CustomActivation` (scalar or batch functions with an explicit or numeric
derivative), `CustomLoss` (explicit gradient, finite differences, or a scalar `MicroTape` program),
`CustomMetric`, `CustomOptimizer` (per-element update rule with named state slots), `CustomCallback` /
`CallbackList`, `CustomModule` (forward / backward callables with parameter slots), the tensor `Tape`
(Input, Add, Mul, Matmul, Relu, Module) and the scalar reverse-mode `MicroTape` (Const, Add, Sub, Mul, Div,
Neg, Square, Exp, Log, Abs, Max).
Parity: include/nexus/custom/{activation,loss,metric,optimizer,callback,module,tape,microtape}.hpp of the
reference."""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import torch

__all__ = ["MicroTape", "Tape", "CustomActivation", "CustomLoss", "CustomMetric", "CustomOptimizer", "CustomCallback",
           "CallbackList", "CustomModule"]


# --------------------------------------------------------------------------------------------- MicroTape
class MicroTape:
    """Scalar reverse-mode AD: record arithmetic on `Var`s, then `gradient(out)`."""

    class Var:
        __slots__ = ("tape", "idx")

        def __init__(self, tape: "MicroTape", idx: int):
            self.tape, self.idx = tape, idx

        @property
        def value(self) -> float:
            return self.tape.vals[self.idx]

        def _b(self, other, op):
            o = other if isinstance(other, MicroTape.Var) else self.tape.const(float(other))
            return self.tape._push(op, self.idx, o.idx)

        def __add__(self, o): return self._b(o, "add")
        def __radd__(self, o): return self.tape.const(float(o))._b(self, "add")
        def __sub__(self, o): return self._b(o, "sub")
        def __rsub__(self, o): return self.tape.const(float(o))._b(self, "sub")
        def __mul__(self, o): return self._b(o, "mul")
        def __rmul__(self, o): return self.tape.const(float(o))._b(self, "mul")
        def __truediv__(self, o): return self._b(o, "div")
        def __rtruediv__(self, o): return self.tape.const(float(o))._b(self, "div")
        def __neg__(self): return self.tape._push("neg", self.idx)

    def __init__(self):
        self.ops: List[tuple] = []
        self.vals: List[float] = []

    def _push(self, op: str, a: int = -1, b: int = -1, value: Optional[float] = None) -> "MicroTape.Var":
        v = self.vals
        if value is None:
            x, y = (v[a] if a >= 0 else 0.0), (v[b] if b >= 0 else 0.0)
            value = {"add": lambda: x + y, "sub": lambda: x - y, "mul": lambda: x * y, "div": lambda: x / y,
                     "neg": lambda: -x, "square": lambda: x * x, "exp": lambda: math.exp(x), "log": lambda: math.log(x),
                     "abs": lambda: abs(x), "max": lambda: max(x, y)}[op]()
        self.ops.append((op, a, b))
        self.vals.append(float(value))
        return MicroTape.Var(self, len(self.vals) - 1)

    def const(self, x: float) -> "MicroTape.Var":
        return self._push("const", value=x)

    variable = const

    def square(self, a): return self._push("square", a.idx)
    def exp(self, a): return self._push("exp", a.idx)
    def log(self, a): return self._push("log", a.idx)
    def abs(self, a): return self._push("abs", a.idx)
    def max(self, a, b): return self._push("max", a.idx, (b if isinstance(b, MicroTape.Var) else self.const(b)).idx)

    def gradient(self, out: "MicroTape.Var") -> List[float]:
        g = [0.0] * len(self.vals)
        g[out.idx] = 1.0
        v = self.vals
        for i in range(out.idx, -1, -1):
            op, a, b = self.ops[i]
            gi = g[i]
            if gi == 0.0 or op == "const":
                continue
            if op == "add":
                g[a] += gi; g[b] += gi
            elif op == "sub":
                g[a] += gi; g[b] -= gi
            elif op == "mul":
                g[a] += gi * v[b]; g[b] += gi * v[a]
            elif op == "div":
                g[a] += gi / v[b]; g[b] -= gi * v[a] / (v[b] * v[b])
            elif op == "neg":
                g[a] -= gi
            elif op == "square":
                g[a] += gi * 2 * v[a]
            elif op == "exp":
                g[a] += gi * v[i]
            elif op == "log":
                g[a] += gi / v[a]
            elif op == "abs":
                g[a] += gi * (1.0 if v[a] > 0 else (-1.0 if v[a] < 0 else 0.0))
            elif op == "max":
                if v[a] >= v[b]:
                    g[a] += gi
                else:
                    g[b] += gi
        return g


# --------------------------------------------------------------------------------------------- Tape
class Tape:
    """Tensor tape with explicit backward: Input, Add, Mul, Matmul, Relu, Module (forward/backward pair)."""

    def __init__(self):
        self.nodes: List[dict] = []

    def _push(self, op, inputs, value, **extra) -> int:
        self.nodes.append({"op": op, "in": list(inputs), "val": value, **extra})
        return len(self.nodes) - 1

    def input(self, t: torch.Tensor) -> int:
        return self._push("input", [], t.detach().float())

    def add(self, a: int, b: int) -> int:
        return self._push("add", [a, b], self.nodes[a]["val"] + self.nodes[b]["val"])

    def mul(self, a: int, b: int) -> int:
        return self._push("mul", [a, b], self.nodes[a]["val"] * self.nodes[b]["val"])

    def matmul(self, a: int, b: int) -> int:
        return self._push("matmul", [a, b], self.nodes[a]["val"] @ self.nodes[b]["val"])

    def relu(self, a: int) -> int:
        return self._push("relu", [a], self.nodes[a]["val"].clamp_min(0))

    def module(self, mod, a: int) -> int:
        """``mod`` has ``forward(x)`` and ``backward(grad_out) -> grad_in`` (it keeps its own state)."""
        return self._push("module", [a], mod.forward(self.nodes[a]["val"]), mod=mod)

    def value(self, i: int) -> torch.Tensor:
        return self.nodes[i]["val"]

    def backward(self, out: int, grad: Optional[torch.Tensor] = None) -> Dict[int, torch.Tensor]:
        g: Dict[int, torch.Tensor] = {out: grad if grad is not None else torch.ones_like(self.nodes[out]["val"])}

        def acc(i, t):
            shape = self.nodes[i]["val"].shape
            while t.dim() > len(shape):
                t = t.sum(0)
            for d, s in enumerate(shape):
                if s == 1 and t.shape[d] != 1:
                    t = t.sum(d, keepdim=True)
            g[i] = g[i] + t if i in g else t
        for i in range(out, -1, -1):
            if i not in g:
                continue
            n, gi = self.nodes[i], g[i]
            v = [self.nodes[j]["val"] for j in n["in"]]
            if n["op"] == "add":
                acc(n["in"][0], gi); acc(n["in"][1], gi)
            elif n["op"] == "mul":
                acc(n["in"][0], gi * v[1]); acc(n["in"][1], gi * v[0])
            elif n["op"] == "matmul":
                acc(n["in"][0], gi @ v[1].transpose(-1, -2)); acc(n["in"][1], v[0].transpose(-1, -2) @ gi)
            elif n["op"] == "relu":
                acc(n["in"][0], gi * (v[0] > 0))
            elif n["op"] == "module":
                acc(n["in"][0], n["mod"].backward(gi))
        return g


# --------------------------------------------------------------------------------------------- activation
class CustomActivation(torch.nn.Module):
    """Element-wise activation from a scalar function (vectorised through a lookup-free torch map when the
    callable accepts tensors, else applied per element) or a batch function; derivative explicit or numeric."""

    def __init__(self, name: str, fn: Callable, derivative: Optional[Callable] = None, batch: bool = True,
                 epsilon: float = 1e-3):
        super().__init__()
        self.name, self.fn, self.dfn, self.batch, self.eps = name, fn, derivative, batch, epsilon

    def _map(self, f, x: torch.Tensor) -> torch.Tensor:
        if self.batch:
            return f(x)
        flat = x.reshape(-1)
        return torch.tensor([float(f(float(v))) for v in flat], dtype=x.dtype).view(x.shape)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        outer = self

        class Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, inp):
                ctx.save_for_backward(inp)
                return outer._map(outer.fn, inp.detach())

            @staticmethod
            def backward(ctx, gy):
                (inp,) = ctx.saved_tensors
                if outer.dfn is not None:
                    d = outer._map(outer.dfn, inp.detach())
                else:
                    e = outer.eps
                    d = (outer._map(outer.fn, inp.detach() + e) - outer._map(outer.fn, inp.detach() - e)) / (2 * e)
                return gy * d
        return Fn.apply(x)


# --------------------------------------------------------------------------------------------- loss
class CustomLoss:
    """`forward_backward(pred, target) -> (loss, dloss/dpred)` in one of three modes."""

    def __init__(self, name: str, mode: str, fn: Callable, epsilon: float = 1e-3):
        self.name, self.mode, self.fn, self.eps = name, mode, fn, epsilon

    @staticmethod
    def from_explicit(name: str, fn: Callable) -> "CustomLoss":
        """fn(pred, target) -> (loss, grad)."""
        return CustomLoss(name, "explicit", fn)

    @staticmethod
    def from_numeric(name: str, fn: Callable, epsilon: float = 1e-3) -> "CustomLoss":
        """fn(pred, target) -> loss; the gradient is a central difference per element."""
        return CustomLoss(name, "numeric", fn, epsilon)

    @staticmethod
    def from_tape(name: str, fn: Callable) -> "CustomLoss":
        """fn(tape, pred_vars, target_values) -> loss Var (scalar program on a MicroTape)."""
        return CustomLoss(name, "tape", fn)

    def forward_backward(self, pred: torch.Tensor, target: torch.Tensor):
        if self.mode == "explicit":
            loss, grad = self.fn(pred, target)
            return float(loss), torch.as_tensor(grad, dtype=pred.dtype).view(pred.shape)
        if self.mode == "numeric":
            base = float(self.fn(pred, target))
            flat = pred.detach().clone().reshape(-1)
            grad = torch.zeros_like(flat)
            for i in range(flat.numel()):
                old = float(flat[i])
                flat[i] = old + self.eps
                up = float(self.fn(flat.view(pred.shape), target))
                flat[i] = old - self.eps
                dn = float(self.fn(flat.view(pred.shape), target))
                flat[i] = old
                grad[i] = (up - dn) / (2 * self.eps)
            return base, grad.view(pred.shape)
        tape = MicroTape()
        pv = [tape.variable(float(v)) for v in pred.detach().reshape(-1)]
        out = self.fn(tape, pv, [float(v) for v in target.reshape(-1)])
        g = tape.gradient(out)
        return out.value, torch.tensor([g[v.idx] for v in pv], dtype=pred.dtype).view(pred.shape)

    def __call__(self, pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """Autograd-compatible scalar."""
        outer = self

        class Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, p):
                loss, grad = outer.forward_backward(p.detach(), target)
                ctx.save_for_backward(grad)
                return torch.tensor(loss, dtype=p.dtype)

            @staticmethod
            def backward(ctx, gy):
                return gy * ctx.saved_tensors[0]
        return Fn.apply(pred)


class CustomMetric:
    """Streaming metric from `update(state, pred, target) -> state` and `result(state) -> float`."""

    def __init__(self, name: str, init, update: Callable, result: Callable):
        self.name, self._init, self._update, self._result = name, init, update, result
        self.reset()

    def reset(self) -> None:
        self.state = self._init() if callable(self._init) else self._init

    def update(self, pred, target) -> None:
        self.state = self._update(self.state, pred, target)

    def result(self) -> float:
        return float(self._result(self.state))


class CustomOptimizer(torch.optim.Optimizer):
    """Optimizer from a rule ``rule(p, g, state, step, hyper) -> new p`` with named zero-initialised slots."""

    def __init__(self, params, rule: Callable, slots: Sequence[str] = (), **hyper):
        super().__init__(list(params), dict(hyper))
        self.rule, self.slots = rule, tuple(slots)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            hyper = {k: v for k, v in group.items() if k != "params"}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    for s in self.slots:
                        st[s] = torch.zeros_like(p)
                st["step"] += 1
                p.copy_(self.rule(p, p.grad, st, st["step"], hyper))
        return loss


class CustomCallback:
    """Hooks: on_train_begin / on_epoch_begin / on_batch_end / on_epoch_end / on_train_end (keyword callables)."""
    HOOKS = ("on_train_begin", "on_epoch_begin", "on_batch_end", "on_epoch_end", "on_train_end")

    def __init__(self, **hooks: Callable):
        bad = set(hooks) - set(self.HOOKS)
        if bad:
            raise ValueError(f"unknown hooks: {sorted(bad)}")
        self.hooks = hooks

    def fire(self, hook: str, *args, **kw):
        f = self.hooks.get(hook)
        return f(*args, **kw) if f is not None else None


class CallbackList:
    def __init__(self, callbacks: Sequence[CustomCallback] = ()):
        self.items = list(callbacks)

    def add(self, cb: CustomCallback) -> None:
        self.items.append(cb)

    def fire(self, hook: str, *args, **kw) -> bool:
        """Returns True when any callback asks to stop (returns False explicitly)."""
        stop = False
        for cb in self.items:
            if cb.fire(hook, *args, **kw) is False:
                stop = True
        return stop


class CustomModule(torch.nn.Module):
    """Module from ``forward(x, params) -> y`` and ``backward(x, params, grad_y) -> (grad_x, {name: grad})``
    with named parameter slots; usable inside autograd models and on the `Tape`."""

    def __init__(self, name: str, slots: Dict[str, Sequence[int]], forward: Callable, backward: Callable, seed: int = 0):
        super().__init__()
        self.name, self._f, self._b = name, forward, backward
        g = torch.Generator().manual_seed(seed)
        self.slots = torch.nn.ParameterDict({k: torch.nn.Parameter(torch.randn(*shape, generator=g) * 0.1)
                                             for k, shape in slots.items()})
        self._last = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        outer = self
        names = list(self.slots.keys())

        class Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, inp, *ps):
                ctx.save_for_backward(inp, *ps)
                return outer._f(inp.detach(), {n: p.detach() for n, p in zip(names, ps)})

            @staticmethod
            def backward(ctx, gy):
                inp, *ps = ctx.saved_tensors
                gx, gp = outer._b(inp, dict(zip(names, ps)), gy)
                return (gx,) + tuple(gp.get(n) for n in names)
        self._last = x.detach()
        return Fn.apply(x, *[self.slots[n] for n in names])

    def backward(self, grad_out: torch.Tensor) -> torch.Tensor:
        """Explicit backward for the `Tape`: accumulates parameter gradients, returns the input gradient."""
        gx, gp = self._b(self._last, {n: p.detach() for n, p in self.slots.items()}, grad_out)
        for n, gval in gp.items():
            p = self.slots[n]
            p.grad = gval.clone() if p.grad is None else p.grad + gval
        return gx
