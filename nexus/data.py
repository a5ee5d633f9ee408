"""`nexus.data`: the shell's call signatures (flat lists, shell tensors); every other name of
:mod:`nexus_b200.data` stays reachable from here with its native (torch) interface."""
import importlib as _importlib

from nexus._shell import (DataLoader, CsvTable, read_csv, save_image, load_image)  # noqa: F401

_native = _importlib.import_module("nexus_b200.data")


def __getattr__(name):
    return getattr(_native, name)
