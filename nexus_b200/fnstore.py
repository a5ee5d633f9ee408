"""Python-defined activations and modules inside NXS archives.

A user body (a plain function or a ``torch.nn.Module`` subclass defined in Python) is registered
under a name; when a model using it is saved, the code object (``marshal``) and defaults travel in
the archive's python payload, so ``nexus.load(path)`` works in a process that never imported the
defining script.  Only load archives you trust: the payload is executable code.

Parity: python/src/nexus/fnstore.py of the reference.
"""
from __future__ import annotations

import marshal
import pickle
import types
from typing import Callable, Dict

import torch

_ACTIVATION_SOURCES: Dict[str, Callable] = {}
_MODULE_FACTORIES: Dict[str, Callable] = {}


def register_python_activation(name: str, fn: Callable) -> None:
    from .nn.modules import register_activation
    _ACTIVATION_SOURCES[name] = fn
    register_activation(name, fn)


def register_python_module(name: str, factory: Callable) -> None:
    _MODULE_FACTORIES[name] = factory


def module_factory(name: str):
    from .nn.modules import PythonModule
    if name not in _MODULE_FACTORIES:
        raise RuntimeError(f"python module body '{name}' is not registered in this process")
    return PythonModule(name, _MODULE_FACTORIES[name]())


def _dump_fn(fn: Callable) -> dict:
    return {"code": marshal.dumps(fn.__code__), "name": fn.__name__, "defaults": fn.__defaults__}


def _load_fn(rec: dict) -> Callable:
    code = marshal.loads(rec["code"])
    return types.FunctionType(code, {"torch": torch, "__builtins__": __builtins__}, rec["name"], rec["defaults"])


def payload_for(model) -> bytes:
    """Bodies of every Python-defined activation / module that ``model`` uses (empty when none)."""
    from .nn.modules import KIND, Module
    acts, mods = {}, {}
    for m in model.modules():
        if isinstance(m, Module):
            if m.kind == KIND["NamedActivation"] and m.layer_name in _ACTIVATION_SOURCES:
                acts[m.layer_name] = _dump_fn(_ACTIVATION_SOURCES[m.layer_name])
            if m.kind == KIND["PythonModule"] and m.layer_name in _MODULE_FACTORIES:
                mods[m.layer_name] = _dump_fn(_MODULE_FACTORIES[m.layer_name])
    if not acts and not mods:
        return b""
    return pickle.dumps({"activations": acts, "modules": mods})


def restore_payload(blob: bytes) -> None:
    if not blob:
        return
    d = pickle.loads(blob)
    for name, rec in d.get("activations", {}).items():
        if name not in _ACTIVATION_SOURCES:
            register_python_activation(name, _load_fn(rec))
    for name, rec in d.get("modules", {}).items():
        if name not in _MODULE_FACTORIES:
            register_python_module(name, _load_fn(rec))
