"""nexus_b200: a Blackwell-native (sm_100a) deep-learning framework with the public surface of Nexus.

PyTorch is the framework layer; the hot operators are hand-written CUDA kernels
(tcgen05 / TMEM / TMA) loaded from ``lib/libnexus_b200_cuda.so``; the runtime pieces around them
(archives, checkpoints, launcher, environments) are native C++ in the ``_native`` module.
"""
__version__ = "0.1.0"
