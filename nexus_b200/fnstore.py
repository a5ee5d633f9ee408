"""Python-defined activations and modules inside NXS archives.

A user body (a plain function, or a factory returning a ``torch.nn.Module``) is registered under a name; when
a model using it is saved, its code object travels in the archive's python payload, so ``nexus.load(path)``
works in a process that never imported the defining script.

Payload = the reference's ``NXPY`` record stream: ``"NXPY" | u16 version 1 | u32 count`` then per record
``u8 kind (1 activation, 2 module) | u32 len + name | code | code`` (forward, backward) and, for modules,
``u32 n_shapes | (u32 rank | u64 dims...)``; a code field is ``u32 len | marshal bytes | u32 n_cells |
(u8 tag | 8 bytes)`` with tag 1 = float64, 2 = int64, 3 = bool.  Closure cells may only hold float, int or
bool, and nothing but ``marshal`` is used to read the payload (no pickle: loading runs no code until a body
is called).  A loaded body sees ``math``, ``torch`` and the builtins.  The backward slot is written empty:
gradients come from autograd here.  Only load archives you trust: the bodies are executable code.

Parity: python/src/nexus/fnstore.py of the reference.
"""
from __future__ import annotations

import marshal
import math
import struct
import types
from typing import Callable, Dict

import torch

_ACTIVATION_SOURCES: Dict[str, tuple] = {}     # name -> (forward, backward or None)
_MODULE_SOURCES: Dict[str, tuple] = {}         # name -> (forward or factory, backward or None, parameter shapes)
_MODULE_FACTORIES: Dict[str, Callable] = {}    # name -> callable returning the torch module that runs the body


class _ScalarFn(torch.autograd.Function):
    """Elementwise application of a body written for one number; its derivative comes from the backward body, or
    from a central difference when none was given."""

    @staticmethod
    def forward(ctx, x, fwd, bwd):
        flat = x.detach().reshape(-1).tolist()
        y = torch.tensor([float(fwd(v)) for v in flat], dtype=x.dtype, device=x.device).view(x.shape)
        ctx.save_for_backward(x)
        ctx.fwd, ctx.bwd = fwd, bwd
        return y

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        flat = x.detach().reshape(-1).tolist()
        if ctx.bwd is not None:
            d = [float(ctx.bwd(v)) for v in flat]
        else:
            d = []
            for v in flat:
                h = 1e-3 * max(1.0, abs(v))
                d.append((float(ctx.fwd(v + h)) - float(ctx.fwd(v - h))) / (2 * h))
        return g * torch.tensor(d, dtype=g.dtype, device=g.device).view(g.shape), None, None


def tensor_level(forward: Callable, backward=None) -> Callable:
    """Runtime form of an activation body.  A body that only uses arithmetic runs on the whole tensor (autograd
    differentiates it); one that needs real numbers (``math.tanh(x)``) or brings its own derivative is applied
    element by element."""
    def run(x: torch.Tensor) -> torch.Tensor:
        if backward is None:
            import warnings
            try:
                with warnings.catch_warnings():
                    warnings.simplefilter("ignore")
                    y = forward(x)
                if isinstance(y, torch.Tensor) and y.shape == x.shape:
                    return y
            except (TypeError, ValueError, RuntimeError):
                pass
        return _ScalarFn.apply(x, forward, backward)
    return run


def remember(name: str, forward: Callable, backward=None) -> None:
    """Registers an activation's bodies (checked: plain functions closing over numbers only) for archiving."""
    _check(forward)
    if backward is not None:
        _check(backward)
    _ACTIVATION_SOURCES[name] = (forward, backward)


def register_python_activation(name: str, fn: Callable, backward=None) -> None:
    from .nn.modules import register_activation
    _ACTIVATION_SOURCES[name] = (fn, backward)
    register_activation(name, tensor_level(fn, backward))


def register_python_module(name: str, factory: Callable) -> None:
    """``factory()`` returns the torch module that implements the body."""
    _MODULE_SOURCES[name] = (factory, None, [])
    _MODULE_FACTORIES[name] = factory


def remember_module(name: str, forward: Callable, backward=None, shapes=None, builder=None) -> None:
    """Registers a module given as ``forward(values, params)`` / ``backward(grad, params)`` bodies over the shell's
    tensors plus its parameter shapes; ``builder(name, forward, backward, shapes)`` returns the runtime factory."""
    _check(forward)
    if backward is not None:
        _check(backward)
    shapes = [list(map(int, s)) for s in (shapes or [])]
    _MODULE_SOURCES[name] = (forward, backward, shapes)
    if builder is None:
        builder = _shell_module_builder()
    _MODULE_FACTORIES[name] = builder(name, forward, backward, shapes)


def _shell_module_builder():
    from nexus import _shell      # the shell owns the tensor type those bodies are written against
    return _shell._py_module_factory


def set_shell_builders(activation_wrapper=None, module_builder=None) -> None:
    """Kept for the shell's start-up: nothing to install, the runtime forms live in this module."""


def module_factory(name: str):
    from .nn.modules import PythonModule
    if name not in _MODULE_FACTORIES:
        raise RuntimeError(f"python module body '{name}' is not registered in this process")
    made = _MODULE_FACTORIES[name]()
    return made if isinstance(made, PythonModule) else PythonModule(name, made)


_ACTIVATION, _MODULE = 1, 2


def _check(fn: Callable) -> None:
    """Only plain functions whose closure cells hold float / int / bool can be archived."""
    if not hasattr(fn, "__code__"):
        raise TypeError("this callable has no code object and cannot be written into an archive")
    if fn.__defaults__ or fn.__kwdefaults__:
        raise TypeError("python bodies with default arguments cannot be written into an archive")
    for cell in fn.__closure__ or ():
        v = cell.cell_contents
        if isinstance(v, bool) or isinstance(v, float):
            continue
        if isinstance(v, int) and -(1 << 63) <= v < (1 << 63):
            continue
        raise TypeError("a python body may only close over float, int or bool values")


def _write_code(buf: bytearray, fn) -> None:
    blob = b"" if fn is None else marshal.dumps(fn.__code__)
    buf += struct.pack("<I", len(blob)) + blob
    cells = () if fn is None or not fn.__closure__ else fn.__closure__
    buf += struct.pack("<I", len(cells))
    for cell in cells:
        v = cell.cell_contents
        if isinstance(v, bool):
            buf += struct.pack("<Bq", 3, int(v))
        elif isinstance(v, int):
            buf += struct.pack("<Bq", 2, v)
        else:
            buf += struct.pack("<Bd", 1, float(v))


def _cell(value):
    return (lambda: value).__closure__[0]


def _read_code(view, off: int):
    (n,) = struct.unpack_from("<I", view, off)
    off += 4
    blob = bytes(view[off: off + n])
    if len(blob) != n:
        raise ValueError("nxs python payload is truncated")
    off += n
    (ncell,) = struct.unpack_from("<I", view, off)
    off += 4
    cells = []
    for _ in range(ncell):
        (tag,) = struct.unpack_from("<B", view, off)
        if tag == 1:
            cells.append(struct.unpack_from("<d", view, off + 1)[0])
        elif tag in (2, 3):
            raw = struct.unpack_from("<q", view, off + 1)[0]
            cells.append(bool(raw) if tag == 3 else int(raw))
        else:
            raise ValueError("nxs python payload: unknown closure cell tag %d" % tag)
        off += 9
    fn = None
    if blob:
        code = marshal.loads(blob)
        closure = tuple(_cell(v) for v in cells) if cells else None
        fn = types.FunctionType(code, {"__builtins__": __builtins__, "math": math, "torch": torch}, closure=closure)
    return fn, off


def payload_for(model) -> bytes:
    """``NXPY`` records of every Python-defined activation / module that ``model`` uses (empty when none)."""
    from .nn.modules import KIND, Module
    acts, mods = {}, {}
    for m in model.modules():
        if isinstance(m, Module):
            if m.kind == KIND["NamedActivation"] and m.layer_name in _ACTIVATION_SOURCES:
                acts[m.layer_name] = _ACTIVATION_SOURCES[m.layer_name]
            if m.kind == KIND["PythonModule"] and m.layer_name in _MODULE_SOURCES:
                mods[m.layer_name] = _MODULE_SOURCES[m.layer_name]
    if not acts and not mods:
        return b""
    buf = bytearray(b"NXPY") + struct.pack("<HI", 1, len(acts) + len(mods))
    for name, (fwd, bwd) in acts.items():
        _check(fwd)
        if bwd is not None:
            _check(bwd)
        raw = name.encode("utf-8")
        buf += struct.pack("<BI", _ACTIVATION, len(raw)) + raw
        _write_code(buf, fwd)
        _write_code(buf, bwd)
    for name, (fwd, bwd, shapes) in mods.items():
        _check(fwd)
        if bwd is not None:
            _check(bwd)
        raw = name.encode("utf-8")
        buf += struct.pack("<BI", _MODULE, len(raw)) + raw
        _write_code(buf, fwd)
        _write_code(buf, bwd)
        buf += struct.pack("<I", len(shapes))
        for shp in shapes:
            buf += struct.pack("<I", len(shp))
            for dim in shp:
                buf += struct.pack("<Q", int(dim))
    return bytes(buf)


def restore_payload(blob: bytes) -> None:
    """Registers the bodies of an ``NXPY`` payload that this process does not know yet."""
    if not blob:
        return
    view = memoryview(blob)
    if bytes(view[:4]) != b"NXPY":
        raise ValueError("nxs python payload: not an NXPY record stream")
    try:
        version, count = struct.unpack_from("<HI", view, 4)
        if version != 1:
            raise ValueError("nxs python payload version %d is unsupported" % version)
        off = 10
        for _ in range(count):
            kind, nlen = struct.unpack_from("<BI", view, off)
            off += 5
            name = bytes(view[off: off + nlen]).decode("utf-8")
            off += nlen
            forward, off = _read_code(view, off)
            backward, off = _read_code(view, off)
            if kind == _MODULE:
                (nshape,) = struct.unpack_from("<I", view, off)
                off += 4
                shapes = []
                for _s in range(nshape):
                    (rank,) = struct.unpack_from("<I", view, off)
                    off += 4
                    shapes.append([int(v) for v in struct.unpack_from("<%dQ" % rank, view, off)])
                    off += 8 * rank
                if forward is not None and name not in _MODULE_FACTORIES:
                    if forward.__code__.co_argcount == 0 and backward is None and not shapes:
                        register_python_module(name, forward)      # a factory returning the torch module
                    else:
                        remember_module(name, forward, backward, shapes)
            elif kind == _ACTIVATION:
                if forward is not None and name not in _ACTIVATION_SOURCES:
                    register_python_activation(name, forward, backward)
            else:
                raise ValueError("nxs python payload: unknown record kind %d" % kind)
    except struct.error:
        raise ValueError("nxs python payload is truncated") from None
