"""`nexus.loss`: the shell's call signatures (flat lists, shell tensors); every other name of
:mod:`nexus_b200.loss` stays reachable from here with its native (torch) interface."""
import importlib as _importlib

from nexus._shell import (CrossEntropy, MSE, MAE, Huber, BCE)  # noqa: F401

_native = _importlib.import_module("nexus_b200.loss")


def __getattr__(name):
    return getattr(_native, name)
