"""The `nexus` autograd surface on top of ``torch.autograd``: `Variable`, `Node`, `Edge`,
`AccumulateGrad`, grad-mode guards, anomaly mode, gradient / post-accumulate hooks, `retain_grad`,
saved-tensor hooks (`set_saved_tensors_hooks`, `SavedTensorsHooksGuard`), `custom_function`,
`checkpoint`, `gradcheck`, `backward` and the differentiable op set.

Parity: include/nexus/autograd/autograd.hpp:50-404, src/autograd/engine.cpp:83-737,
src/autograd/ops.cpp:407-1538 of the reference.
"""
from __future__ import annotations

import contextlib
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .checkpoint import SavedBytesCounter, checkpoint  # noqa: F401


class Edge:
    """(function, input_nr): where a gradient flows next."""

    def __init__(self, function, input_nr: int):
        self.function, self.input_nr = function, input_nr

    def is_valid(self) -> bool:
        return self.function is not None


class Node:
    """View of one backward function of the graph (wraps ``torch.autograd.graph.Node``)."""

    def __init__(self, fn):
        self._fn = fn

    def name(self) -> str:
        return self._fn.name() if self._fn is not None else "None"

    def next_edges(self) -> List[Edge]:
        return [Edge(Node(f) if f is not None else None, i) for f, i in self._fn.next_functions]

    def register_hook(self, hook):
        return self._fn.register_hook(hook)

    def is_accumulate_grad(self) -> bool:
        return self.name() == "torch::autograd::AccumulateGrad"

    @property
    def metadata(self):
        return self._fn.metadata


class AccumulateGrad(Node):
    """Leaf sink: adds the incoming gradient into ``variable.grad``."""

    @property
    def variable(self):
        return self._fn.variable


class Variable:
    """A tensor plus autograd metadata.  Copying a Variable deep-copies its storage (the reference's
    Tensor copy constructor is a deep copy); ``shallow()`` shares it."""

    def __init__(self, data, requires_grad: bool = False, dtype=None, device=None):
        if isinstance(data, Variable):
            t = data.tensor.detach().clone()
        elif isinstance(data, torch.Tensor):
            t = data
        else:
            t = torch.tensor(data, dtype=dtype or torch.float32)
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        if device is not None:
            t = t.to(device)
        if requires_grad and not t.requires_grad:
            t = t.detach().requires_grad_(True)
        self.tensor = t

    # --- metadata
    @property
    def requires_grad(self) -> bool: return self.tensor.requires_grad
    @property
    def grad(self): return None if self.tensor.grad is None else Variable(self.tensor.grad)
    @property
    def is_leaf(self) -> bool: return self.tensor.is_leaf
    @property
    def shape(self): return tuple(self.tensor.shape)
    @property
    def dtype(self): return self.tensor.dtype
    @property
    def version(self) -> int: return self.tensor._version

    def grad_fn(self) -> Optional[Node]:
        return None if self.tensor.grad_fn is None else Node(self.tensor.grad_fn)

    def grad_accumulator(self) -> Optional[AccumulateGrad]:
        if not (self.tensor.is_leaf and self.tensor.requires_grad):
            return None
        return AccumulateGrad(self.tensor.view_as(self.tensor).grad_fn.next_functions[0][0])

    def shallow(self) -> "Variable":
        v = Variable.__new__(Variable)
        v.tensor = self.tensor
        return v

    def clone(self) -> "Variable": return Variable(self.tensor.clone())
    def detach(self) -> "Variable": return Variable(self.tensor.detach())
    def zero_grad(self) -> None: self.tensor.grad = None
    def retain_grad(self) -> None: self.tensor.retain_grad()
    def register_hook(self, hook): return self.tensor.register_hook(lambda g: _unwrap(hook(Variable(g))))

    def register_post_accumulate_grad_hook(self, hook):
        return self.tensor.register_post_accumulate_grad_hook(lambda t: hook(Variable(t)))

    def backward(self, grad=None, retain_graph: bool = False) -> None:
        backward([self], [grad] if grad is not None else None, retain_graph)

    def item(self): return self.tensor.item()
    def tolist(self): return self.tensor.tolist()
    def numpy(self): return self.tensor.detach().cpu().numpy()
    def to(self, *a, **k) -> "Variable": return Variable(self.tensor.to(*a, **k))

    # --- operators
    def __add__(self, o): return add(self, o)
    def __radd__(self, o): return add(o, self)
    def __sub__(self, o): return sub(self, o)
    def __rsub__(self, o): return sub(o, self)
    def __mul__(self, o): return mul(self, o)
    def __rmul__(self, o): return mul(o, self)
    def __truediv__(self, o): return div(self, o)
    def __neg__(self): return neg(self)
    def __matmul__(self, o): return matmul(self, o)
    def __pow__(self, e): return pow(self, e)
    def __repr__(self): return f"Variable({self.tensor!r})"


def _unwrap(x):
    return x.tensor if isinstance(x, Variable) else x


def _t(x):
    return x.tensor if isinstance(x, Variable) else x


def _wrap(t) -> Variable:
    v = Variable.__new__(Variable)
    v.tensor = t
    return v


# ------------------------------------------------------------------------------------------- modes
NoGradGuard = torch.no_grad
EnableGradGuard = torch.enable_grad
is_grad_enabled = torch.is_grad_enabled
set_grad_enabled = torch.set_grad_enabled


class AnomalyError(RuntimeError):
    pass


@contextlib.contextmanager
def detect_anomaly(enabled: bool = True):
    """Anomaly mode: a NaN/Inf produced by a backward node raises with the forward context."""
    with torch.autograd.set_detect_anomaly(enabled, check_nan=enabled):
        try:
            yield
        except RuntimeError as e:
            if "nan" in str(e).lower() or "inf" in str(e).lower():
                raise AnomalyError(str(e)) from e
            raise


set_anomaly_enabled = torch.autograd.set_detect_anomaly

# ----------------------------------------------------------------------------- saved-tensor hooks
_hook_stack: List = []


def set_saved_tensors_hooks(pack: Optional[Callable], unpack: Optional[Callable]) -> None:
    """Installs (or with ``None, None`` removes) process-wide pack/unpack hooks."""
    while _hook_stack:
        _hook_stack.pop().__exit__(None, None, None)
    if pack is not None:
        ctx = torch.autograd.graph.saved_tensors_hooks(pack, unpack)
        ctx.__enter__()
        _hook_stack.append(ctx)


SavedTensorsHooksGuard = torch.autograd.graph.saved_tensors_hooks


class SavedTensor:
    """A tensor saved for backward with a version check on use."""

    def __init__(self, t):
        self._t = _t(t)
        self._version = self._t._version

    def unpack(self):
        if self._t._version != self._version:
            raise RuntimeError("a tensor saved for backward was modified in place "
                               f"(version {self._version} -> {self._t._version})")
        return self._t


# --------------------------------------------------------------------------------------- functions
def backward(roots: Sequence, grads: Optional[Sequence] = None, retain_graph: bool = False) -> None:
    ts = [_t(r) for r in roots]
    gs = None if grads is None else [None if g is None else _t(g) for g in grads]
    torch.autograd.backward(ts, gs, retain_graph=retain_graph)


def grad(outputs, inputs, grad_outputs=None, retain_graph=False, create_graph=False):
    res = torch.autograd.grad([_t(o) for o in outputs], [_t(i) for i in inputs],
                              None if grad_outputs is None else [_t(g) for g in grad_outputs],
                              retain_graph=retain_graph, create_graph=create_graph, allow_unused=True)
    return [None if r is None else _wrap(r) for r in res]


def gradcheck(fn: Callable, inputs: Sequence[Variable], eps: float = 1e-6, atol: float = 1e-5,
              rtol: float = 1e-3) -> bool:
    ts = tuple(_t(i).detach().double().requires_grad_(True) for i in inputs)
    return torch.autograd.gradcheck(lambda *a: _t(fn(*[_wrap(x) for x in a])), ts, eps=eps, atol=atol, rtol=rtol)


def custom_function(forward: Callable, backward: Callable, name: str = "CustomFunction") -> Callable:
    """Builds a differentiable op from ``forward(ctx, *tensors)`` and ``backward(ctx, grad)`` callables;
    ``ctx.save_for_backward`` / ``ctx.saved_tensors`` as usual."""
    fn = type(name, (torch.autograd.Function,), {"forward": staticmethod(forward), "backward": staticmethod(backward)})

    def apply(*args):
        return _wrap(fn.apply(*[_t(a) for a in args]))
    return apply


def _op1(f):
    return lambda a, *rest, **kw: _wrap(f(_t(a), *rest, **kw))


def _op2(f):
    return lambda a, b, *rest, **kw: _wrap(f(_t(a), _t(b), *rest, **kw))


add, sub, mul, div, matmul = _op2(torch.add), _op2(torch.sub), _op2(torch.mul), _op2(torch.div), _op2(torch.matmul)
neg, relu, silu, sigmoid, tanh, exp, log = (_op1(f) for f in (torch.neg, torch.relu, F.silu, torch.sigmoid,
                                                                  torch.tanh, torch.exp, torch.log))
gelu = _op1(F.gelu)  # erf form on this path (the flat GPU model uses the tanh form)
add_scalar = lambda a, s: _wrap(_t(a) + s)
mul_scalar = lambda a, s: _wrap(_t(a) * s)
add_bias = lambda a, b: _wrap(_t(a) + _t(b))
pow = lambda a, e: _wrap(torch.pow(_t(a), e))
sum = lambda a, dim=None, keepdim=False: _wrap(_t(a).sum() if dim is None else _t(a).sum(dim, keepdim))
mean = lambda a, dim=None, keepdim=False: _wrap(_t(a).mean() if dim is None else _t(a).mean(dim, keepdim))
reshape = lambda a, shape: _wrap(_t(a).reshape(shape))
transpose = lambda a, d0=-2, d1=-1: _wrap(_t(a).transpose(d0, d1))
softmax = lambda a, dim=-1: _wrap(torch.softmax(_t(a), dim))
log_softmax = lambda a, dim=-1: _wrap(torch.log_softmax(_t(a), dim))
cross_entropy = lambda logits, target, **kw: _wrap(F.cross_entropy(_t(logits), _t(target).long(), **kw))
embedding = lambda idx, table: _wrap(F.embedding(_t(idx).long(), _t(table)))
narrow = lambda a, dim, start, length: _wrap(_t(a).narrow(dim, start, length))
cat = lambda xs, dim=0: _wrap(torch.cat([_t(x) for x in xs], dim))
to_dtype = lambda a, dtype: _wrap(_t(a).to(dtype))
to_device = lambda a, device: _wrap(_t(a).to(device))


def dropout(a, p: float, seed: int = 0, offset: int = 0, training: bool = True):
    from ..fused.ops import dropout_philox
    return _wrap(dropout_philox(_t(a), p, seed, offset, training))


def module_function(module) -> Callable:
    """Wraps a classic module with explicit ``forward(x)`` / ``backward(grad_out) -> grad_in`` (parameter
    gradients accumulate inside the module) as ONE autograd node, so that it can sit inside a tape-based
    model.  Parity: include/nexus/autograd/module_function.hpp:57-69 of the reference."""
    def fwd(ctx, x):
        return module.forward(x)

    def bwd(ctx, grad_out):
        return module.backward(grad_out)
    return custom_function(fwd, bwd, name=type(module).__name__)
