"""`nexus`: the same-named Python shell.  Every sub-module of :mod:`nexus_b200` is importable under the
name the reference's shell uses (``nexus.nn``, ``nexus.train``, ``nexus.lm``, ``nexus.rl``, ...)."""
import importlib
import sys

import nexus_b200 as _impl

__version__ = _impl.__version__

_SUBMODULES = ("nn", "loss", "optim", "data", "metrics", "train", "rl", "custom", "linalg", "interop", "lm", "config",
               "dist", "serve", "prof", "autograd", "fused", "moe", "ckpt", "nxs", "compile", "backend", "core",
               "infer", "models", "ops", "parallel", "utils", "amp", "memory", "cpu")


def __getattr__(name):
    if name in _SUBMODULES:
        target = {"dist": "parallel"}.get(name, name)
        mod = importlib.import_module(f"nexus_b200.{target}")
        sys.modules[f"nexus.{name}"] = mod
        globals()[name] = mod
        return mod
    if hasattr(_impl, name):
        return getattr(_impl, name)
    raise AttributeError(f"module 'nexus' has no attribute {name!r}")
