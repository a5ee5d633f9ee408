"""`nexus`: the same-named Python shell.

`nexus.Tensor`, `nexus.load`, `nexus.save` and the sub-modules `nn`, `train`, `data`, `optim`, `loss`, `metrics`, `rl`,
`custom`, `linalg` speak the reference shell's interface (flat Python lists and shell tensors, explicit
`forward` / `backward`, `parameters()` records); scripts written against the reference's `import nexus` run as they are.
Every other sub-module of :mod:`nexus_b200` is importable under the reference's name too (``nexus.lm``, ``nexus.dist``,
``nexus.serve``, ...), with the native torch-tensor interface.
"""
import importlib
import sys

import nexus_b200 as _impl
from nexus._shell import Tensor, load, save  # noqa: F401
from nexus import custom, data, linalg, loss, metrics, nn, optim, rl, train  # noqa: F401
from nexus_b200.fnstore import remember, remember_module  # noqa: F401

__version__ = _impl.__version__

_SUBMODULES = ("interop", "lm", "config", "dist", "serve", "prof", "autograd", "fused", "moe", "ckpt", "nxs", "compile",
               "backend", "core", "infer", "models", "ops", "parallel", "utils", "amp", "memory", "cpu")

__all__ = ["Tensor", "__version__", "custom", "data", "linalg", "load", "loss", "metrics", "nn", "optim", "rl", "save",
           "train"]


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
