"""`nexus.nn`: the shell's call signatures (flat lists, shell tensors); every other name of
:mod:`nexus_b200.nn` stays reachable from here with its native (torch) interface."""
import importlib as _importlib

from nexus._shell import (Sequential, Graph, Linear, Conv1d, Conv2d, Conv3d, DepthwiseConv2d, MultiHeadAttention, LSTM, GRU, RNN, TransformerEncoder, TransformerDecoder, CausalTransformerBlock, Embedding, BatchNorm1d, BatchNorm2d, LayerNorm, GroupNorm, InstanceNorm, ReLU, Dropout, MaxPool2d, AvgPool2d, GlobalAvgPool2d, Flatten, Reshape, PositionalEncoding, Residual, swish, gelu, silu, mish, activation, PythonModule, conv2d_device, Layer)  # noqa: F401

_native = _importlib.import_module("nexus_b200.nn")


def __getattr__(name):
    return getattr(_native, name)
