"""nexus_b200: a Blackwell-native (sm_100a) deep-learning framework with the public surface of Nexus.

PyTorch is the framework layer; the hot operators are hand-written CUDA kernels
(tcgen05 / TMEM / TMA) loaded from ``lib/libnexus_b200_cuda.so``; the runtime pieces around them
(archives, checkpoints, launcher, environments) are native C++ in the ``_native`` module.
"""
__version__ = "0.1.0"


def _load_alternative_native() -> None:
    """``NEXUS_B200_NATIVE=<path>``: load that build of the host module (a sanitizer build, say) as
    ``nexus_b200._native`` instead of the one beside this file."""
    import importlib.util
    import os
    import sys
    path = os.environ.get("NEXUS_B200_NATIVE")
    if not path:
        return
    spec = importlib.util.spec_from_file_location("nexus_b200._native", path)
    if spec is None or spec.loader is None:
        raise ImportError(f"NEXUS_B200_NATIVE: cannot load {path}")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["nexus_b200._native"] = mod
    spec.loader.exec_module(mod)


_load_alternative_native()
