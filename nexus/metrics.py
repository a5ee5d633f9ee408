"""`nexus.metrics`: the shell's call signatures (flat lists, shell tensors); every other name of
:mod:`nexus_b200.metrics` stays reachable from here with its native (torch) interface."""
import importlib as _importlib

from nexus._shell import (Accuracy)  # noqa: F401

_native = _importlib.import_module("nexus_b200.metrics")


def __getattr__(name):
    return getattr(_native, name)
