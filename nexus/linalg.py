"""`nexus.linalg`: the shell's call signatures (flat lists, shell tensors); every other name of
:mod:`nexus_b200.linalg` stays reachable from here with its native (torch) interface."""
import importlib as _importlib

from nexus._shell import (gemm, kernel_name)  # noqa: F401

_native = _importlib.import_module("nexus_b200.linalg")


def __getattr__(name):
    return getattr(_native, name)
