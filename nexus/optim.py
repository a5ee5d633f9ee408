"""`nexus.optim`: the shell's call signatures (flat lists, shell tensors); every other name of
:mod:`nexus_b200.optim` stays reachable from here with its native (torch) interface."""
import importlib as _importlib

from nexus._shell import (SGD, AdamW, CosineAnnealing)  # noqa: F401

_native = _importlib.import_module("nexus_b200.optim")


def __getattr__(name):
    return getattr(_native, name)
