"""`nn.functional`: stateless forms of the catalog operators.  Everything that has a fused kernel goes through
`fused.ops` (CUDA kernels on a GPU, the FP32 reference statements on the CPU); the rest comes from torch.
Parity: include/nexus/nn/functional.hpp (relu, silu, softmax) and the operator set of include/nexus/nn/modules.hpp of
the reference."""
from __future__ import annotations

from typing import Optional

import torch
from torch.nn.functional import (avg_pool2d, conv1d, conv2d, conv3d, elu, leaky_relu, max_pool2d, mish,  # noqa: F401
                                 relu, sigmoid, silu, softplus, tanh)

from ..fused import ops as _F
from ..fused.ops import (attention, attention_varlen, cross_entropy, cross_entropy_shifted, dropout_philox,  # noqa: F401
                         embedding_pos, fused_layernorm as layer_norm, fused_linear as linear,
                         fused_residual_layernorm as residual_layer_norm, fused_softmax as softmax, gated_activation,
                         rms_norm)

__all__ = ["relu", "silu", "gelu", "sigmoid", "tanh", "elu", "leaky_relu", "mish", "softplus", "softmax", "linear",
           "layer_norm", "residual_layer_norm", "rms_norm", "swiglu", "geglu", "gated_activation", "attention",
           "attention_varlen", "scaled_dot_product_attention", "embedding", "embedding_pos", "cross_entropy",
           "cross_entropy_shifted", "dropout", "dropout_philox", "conv1d", "conv2d", "conv3d", "avg_pool2d",
           "max_pool2d"]


def gelu(x: torch.Tensor, approximate: str = "tanh") -> torch.Tensor:
    """GELU; the tanh form is the one the fused GEMM epilogues apply."""
    if approximate == "tanh":
        return _F.gelu_tanh(x)
    return torch.nn.functional.gelu(x, approximate=approximate)


def swiglu(h: torch.Tensor) -> torch.Tensor:
    """``silu(h[..., :F]) * h[..., F:]`` for a gate | up projection ``h`` of width 2F."""
    return gated_activation(h, "swiglu")


def geglu(h: torch.Tensor) -> torch.Tensor:
    """``gelu(h[..., :F]) * h[..., F:]``."""
    return gated_activation(h, "geglu")


def scaled_dot_product_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False,
                                 scale: Optional[float] = None, window: int = 0, dropout_p: float = 0.0,
                                 dropout_seed: int = 0, dropout_offset: int = 0) -> torch.Tensor:
    """Attention over ``[batch, heads, tokens, head_dim]`` tensors (the layout of
    ``torch.nn.functional.scaled_dot_product_attention``); fewer key / value heads than query heads mean grouped-query
    attention.  The kernels take ``[batch, tokens, heads, head_dim]``: the transposes here are views."""
    o = attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal, window, scale, 0.0, None,
                  dropout_p, dropout_seed, dropout_offset)
    return o.transpose(1, 2)


def embedding(tokens: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Token embedding lookup (no position table)."""
    return embedding_pos(tokens, weight, None)


def dropout(x: torch.Tensor, p: float, seed: int = 0, offset: int = 0, training: bool = True) -> torch.Tensor:
    """Dropout drawn from the library's Philox stream (seed, offset): the same mask on CPU and GPU, and the mask the
    backward pass regenerates instead of storing."""
    return dropout_philox(x, p, seed, offset, training)
