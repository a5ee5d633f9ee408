"""The `nn` layer catalog: torch modules with the reference's fluent shell — explicit
``forward`` / ``backward(grad)`` (a backward pass without touching autograd from user code),
``parameters()``, ``zero_grad()`` and an ``nxs_spec()`` describing the layer for the NXS2 archive
(fixed type ids 1-36 and attribute keys).

Parity: include/nexus/nn/modules.hpp:35-781, include/nexus/nn/activations.hpp and the archive
factory src/model/nxs.cpp:415-521 of the reference.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn as tnn
import torch.nn.functional as F

import threading

I32, F32, BOOL, STR = 1, 2, 3, 4
_CALL_DEPTH = threading.local()

KIND = dict(Linear=1, Conv2d=2, MultiHeadAttention=3, Lstm=4, Gru=5, TransformerEncoder=6, Embedding=7,
            BatchNorm1d=8, LayerNorm=9, Relu=10, Swish=11, Dropout=12, MaxPool2d=13, AvgPool2d=14,
            GlobalAvgPool2d=15, Flatten=16, BatchNorm2d=17, Conv1d=18, Conv3d=19, DepthwiseConv2d=20, GroupNorm=21,
            InstanceNorm=22, Residual=23, Reshape=24, Rnn=25, PositionalEncoding=26, TransformerDecoder=27,
            Sequential=28, NamedActivation=29, PythonModule=30, Graph=31, Concat=32, CausalBlock=33,
            DecoderBlock=34, LanguageModel=35, MoEFFN=36)


class Module(tnn.Module):
    """Base of the catalog.  ``backward`` differentiates the last ``forward`` call."""

    kind: int = 0
    layer_name: str = ""

    def __init__(self):
        super().__init__()
        self._last_in = None
        self._last_out = None

    def __call__(self, *args, **kwargs):
        # The outermost catalog module of a call records its inputs/outputs so that `backward(grad)`
        # can run later; data inputs (float tensors that do not require grad) become graph leaves so
        # the gradient w.r.t. the input can be returned.  Nested modules behave like plain torch modules.
        if getattr(_CALL_DEPTH, "n", 0) > 0 or not torch.is_grad_enabled():
            return super().__call__(*args, **kwargs)
        _CALL_DEPTH.n = 1
        try:
            ins = [a.detach().requires_grad_(True)
                   if isinstance(a, torch.Tensor) and a.is_floating_point() and not a.requires_grad else a
                   for a in args]
            out = super().__call__(*ins, **kwargs)
        finally:
            _CALL_DEPTH.n = 0
        self._last_in, self._last_out = ins, out
        return out

    def backward(self, grad_output: torch.Tensor):
        """Accumulates parameter gradients and returns the gradient w.r.t. the (first) input."""
        if self._last_out is None:
            raise RuntimeError("backward called before forward")
        torch.autograd.backward([self._last_out], [grad_output])
        g = [i.grad for i in self._last_in if isinstance(i, torch.Tensor) and i.requires_grad]
        self._last_out = None
        return g[0] if g else None

    def nxs_attrs(self) -> list:
        return []

    def nxs_children(self) -> list:
        return []

    def nxs_spec(self) -> dict:
        return {"type": self.kind, "name": self.layer_name or type(self).__name__, "attrs": self.nxs_attrs(),
                "children": [c.nxs_spec() for c in self.nxs_children()]}

    def parameter_count(self) -> int:
        return sum(p.numel() for p in self.parameters())


def _attr(spec: dict, key: str, default=None):
    for k, _, v in spec["attrs"]:
        if k == key:
            return v
    if default is None:
        raise KeyError(f"nxs layer '{spec['name']}' lacks attribute '{key}'")
    return default


# ------------------------------------------------------------------------------------------ layers
class Linear(Module):
    kind = KIND["Linear"]

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.inner = tnn.Linear(in_features, out_features, bias)
        self.cfg = (in_features, out_features, bias)

    def forward(self, x):
        from ..fused.ops import fused_linear
        return fused_linear(x, self.inner.weight, self.inner.bias)

    def nxs_attrs(self):
        return [("in", I32, self.cfg[0]), ("out", I32, self.cfg[1]), ("bias", BOOL, self.cfg[2])]


class _ConvNd(Module):
    ND = 2

    def __init__(self, in_ch, out_ch, kernel, stride=1, padding=0, bias=True):
        super().__init__()
        cls = {1: tnn.Conv1d, 2: tnn.Conv2d, 3: tnn.Conv3d}[self.ND]
        self.inner = cls(in_ch, out_ch, kernel, stride, padding, bias=bias)
        self.cfg = (in_ch, out_ch, kernel, stride, padding, bias)

    def forward(self, x):
        return self.inner(x)

    def nxs_attrs(self):
        c = self.cfg
        return [("in", I32, c[0]), ("out", I32, c[1]), ("kernel", I32, c[2]), ("stride", I32, c[3]),
                ("padding", I32, c[4]), ("bias", BOOL, c[5])]


class Conv1d(_ConvNd):
    ND, kind = 1, KIND["Conv1d"]


class Conv2d(_ConvNd):
    ND, kind = 2, KIND["Conv2d"]


class Conv3d(_ConvNd):
    ND, kind = 3, KIND["Conv3d"]


class DepthwiseConv2d(Module):
    kind = KIND["DepthwiseConv2d"]

    def __init__(self, channels, kernel, stride=1, padding=0):
        super().__init__()
        self.inner = tnn.Conv2d(channels, channels, kernel, stride, padding, groups=channels)
        self.cfg = (channels, kernel, stride, padding)

    def forward(self, x):
        return self.inner(x)

    def nxs_attrs(self):
        c = self.cfg
        return [("channels", I32, c[0]), ("kernel", I32, c[1]), ("stride", I32, c[2]), ("padding", I32, c[3])]


class MultiHeadAttention(Module):
    """Self-attention over [B, T, E]; ``causal`` masks the future."""
    kind = KIND["MultiHeadAttention"]

    def __init__(self, embed: int, heads: int, causal: bool = False):
        super().__init__()
        if embed % heads:
            raise ValueError("embed must be divisible by heads")
        self.embed, self.heads, self.causal = embed, heads, causal
        self.qkv = tnn.Linear(embed, 3 * embed)
        self.out = tnn.Linear(embed, embed)

    def forward(self, x):
        from ..fused.ops import attention, fused_linear
        B, T, E = x.shape
        H, D = self.heads, E // self.heads
        qkv = fused_linear(x, self.qkv.weight, self.qkv.bias).view(B, T, 3, H, D)
        o = attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=self.causal)
        return fused_linear(o.reshape(B, T, E), self.out.weight, self.out.bias)

    def nxs_attrs(self):
        return [("embed", I32, self.embed), ("heads", I32, self.heads)]


class _Recurrent(Module):
    CLS = tnn.LSTM

    def __init__(self, input_size: int, hidden: int):
        super().__init__()
        self.inner = self.CLS(input_size, hidden, batch_first=True)
        self.cfg = (input_size, hidden)

    def forward(self, x):
        return self.inner(x)[0]

    def nxs_attrs(self):
        return [("input", I32, self.cfg[0]), ("hidden", I32, self.cfg[1])]


class LSTM(_Recurrent):
    CLS, kind = tnn.LSTM, KIND["Lstm"]


class GRU(_Recurrent):
    CLS, kind = tnn.GRU, KIND["Gru"]


class RNN(_Recurrent):
    CLS, kind = tnn.RNN, KIND["Rnn"]


class TransformerEncoder(Module):
    """One post-norm, NON-causal encoder layer: attention + GELU feed-forward."""
    kind = KIND["TransformerEncoder"]
    causal = False

    def __init__(self, embed: int, heads: int, feedforward: int):
        super().__init__()
        self.attn = MultiHeadAttention(embed, heads, causal=self.causal)
        self.ln1, self.ln2 = tnn.LayerNorm(embed), tnn.LayerNorm(embed)
        self.fc1, self.fc2 = tnn.Linear(embed, feedforward), tnn.Linear(feedforward, embed)
        self.cfg = (embed, heads, feedforward)

    def forward(self, x):
        n = self.ln1(x + self.attn(x))
        return self.ln2(n + self.fc2(F.gelu(self.fc1(n))))

    def nxs_attrs(self):
        return [("embed", I32, self.cfg[0]), ("heads", I32, self.cfg[1]), ("feedforward", I32, self.cfg[2])]


class TransformerDecoder(TransformerEncoder):
    """Decoder-only layer: the same block with a causal mask."""
    kind = KIND["TransformerDecoder"]
    causal = True


class CausalTransformerBlock(Module):
    """POST-norm causal block: ``r1 = x + drop(MHA_causal(x)); n = LN1(r1); r2 = n + drop(fc2(GELU(fc1(n))));
    out = LN2(r2)``; parameter order attn, ln1, fc1, fc2, ln2."""
    kind = KIND["CausalBlock"]

    def __init__(self, embed: int, heads: int, feedforward: int, dropout: float = 0.0):
        super().__init__()
        self.attn = MultiHeadAttention(embed, heads, causal=True)
        self.ln1 = tnn.LayerNorm(embed)
        self.fc1 = tnn.Linear(embed, feedforward)
        self.fc2 = tnn.Linear(feedforward, embed)
        self.ln2 = tnn.LayerNorm(embed)
        self.drop = tnn.Dropout(dropout)
        self.cfg = (embed, heads, feedforward)

    def forward(self, x):
        n = self.ln1(x + self.drop(self.attn(x)))
        return self.ln2(n + self.drop(self.fc2(F.gelu(self.fc1(n)))))

    def nxs_attrs(self):
        return [("embed", I32, self.cfg[0]), ("heads", I32, self.cfg[1]), ("feedforward", I32, self.cfg[2])]


class Embedding(Module):
    kind = KIND["Embedding"]

    def __init__(self, num: int, dim: int, padding: int = -1):
        super().__init__()
        self.inner = tnn.Embedding(num, dim, padding_idx=padding if padding >= 0 else None)
        self.cfg = (num, dim, padding)

    def forward(self, idx):
        return self.inner(idx.long())

    def nxs_attrs(self):
        return [("num", I32, self.cfg[0]), ("dim", I32, self.cfg[1]), ("padding", I32, self.cfg[2])]


class BatchNorm1d(Module):
    kind = KIND["BatchNorm1d"]

    def __init__(self, features: int):
        super().__init__()
        self.inner = tnn.BatchNorm1d(features)
        self.features = features

    def forward(self, x):
        return self.inner(x)

    def nxs_attrs(self):
        return [("features", I32, self.features)]


class BatchNorm2d(BatchNorm1d):
    kind = KIND["BatchNorm2d"]

    def __init__(self, features: int):
        Module.__init__(self)
        self.inner = tnn.BatchNorm2d(features)
        self.features = features


class LayerNorm(Module):
    kind = KIND["LayerNorm"]

    def __init__(self, size: int, eps: float = 1e-5):
        super().__init__()
        self.inner = tnn.LayerNorm(size, eps)
        self.cfg = (size, eps)

    def forward(self, x):
        from ..fused.ops import fused_layernorm
        return fused_layernorm(x, self.inner.weight, self.inner.bias, self.cfg[1])

    def nxs_attrs(self):
        return [("size", I32, self.cfg[0]), ("eps", F32, self.cfg[1])]


class GroupNorm(Module):
    kind = KIND["GroupNorm"]

    def __init__(self, groups: int, channels: int):
        super().__init__()
        self.inner = tnn.GroupNorm(groups, channels)
        self.cfg = (groups, channels)

    def forward(self, x):
        return self.inner(x)

    def nxs_attrs(self):
        return [("groups", I32, self.cfg[0]), ("channels", I32, self.cfg[1])]


class InstanceNorm(Module):
    kind = KIND["InstanceNorm"]

    def __init__(self, channels: int):
        super().__init__()
        self.inner = tnn.InstanceNorm2d(channels, affine=True)
        self.channels = channels

    def forward(self, x):
        return self.inner(x)

    def nxs_attrs(self):
        return [("channels", I32, self.channels)]


class ReLU(Module):
    kind = KIND["Relu"]

    def forward(self, x):
        return torch.relu(x)


_ACTIVATIONS: Dict[str, Callable] = {
    "relu": torch.relu, "gelu": F.gelu, "silu": F.silu, "swish": F.silu, "mish": F.mish, "tanh": torch.tanh,
    "sigmoid": torch.sigmoid, "identity": lambda x: x, "leaky_relu": F.leaky_relu, "elu": F.elu,
    "softplus": F.softplus,
}


class Activation(Module):
    """Named activation; archived as NamedActivation (29) except swish (11)."""
    kind = KIND["NamedActivation"]

    def __init__(self, name: str, fn: Optional[Callable] = None):
        super().__init__()
        if fn is None and name not in _ACTIVATIONS:
            raise ValueError(f"unknown activation '{name}'")
        self.layer_name = name
        self.fn = fn or _ACTIVATIONS[name]
        if name == "swish":
            self.kind = KIND["Swish"]

    def forward(self, x):
        return self.fn(x)


def make_activation(name: str) -> Activation:
    return Activation(name)


def register_activation(name: str, fn: Callable) -> None:
    _ACTIVATIONS[name] = fn


GELU = lambda: Activation("gelu")
SiLU = lambda: Activation("silu")
Mish = lambda: Activation("mish")
swish = lambda: Activation("swish")


class Dropout(Module):
    """Counter-based dropout: ``set_dropout_rng(seed, offset)`` makes the mask reproducible."""
    kind = KIND["Dropout"]

    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p
        self.seed, self.offset = 0, 0

    def set_dropout_rng(self, seed: int, offset: int = 0) -> None:
        self.seed, self.offset = seed, offset

    def forward(self, x):
        from ..fused.ops import dropout_philox
        y = dropout_philox(x, self.p, self.seed, self.offset, self.training)
        if self.training:
            self.offset += (x.numel() + 3) // 4
        return y

    def nxs_attrs(self):
        return [("p", F32, self.p)]


class _Pool(Module):
    def __init__(self, kernel: int, stride: int = 0, padding: int = 0):
        super().__init__()
        self.cfg = (kernel, stride or kernel, padding)

    def nxs_attrs(self):
        return [("kernel", I32, self.cfg[0]), ("stride", I32, self.cfg[1]), ("padding", I32, self.cfg[2])]


class MaxPool2d(_Pool):
    kind = KIND["MaxPool2d"]

    def forward(self, x):
        return F.max_pool2d(x, *self.cfg)


class AvgPool2d(_Pool):
    kind = KIND["AvgPool2d"]

    def forward(self, x):
        return F.avg_pool2d(x, *self.cfg)


class GlobalAvgPool2d(Module):
    kind = KIND["GlobalAvgPool2d"]

    def forward(self, x):
        return x.mean(dim=(-2, -1))


class Flatten(Module):
    kind = KIND["Flatten"]

    def forward(self, x):
        return x.flatten(1)


class Reshape(Module):
    kind = KIND["Reshape"]

    def __init__(self, shape: Sequence[int]):
        super().__init__()
        self.shape = [int(s) for s in shape]

    def forward(self, x):
        return x.reshape(x.shape[0], *self.shape)

    def nxs_attrs(self):
        return [(f"d{i}", I32, s) for i, s in enumerate(self.shape)]


class Residual(Module):
    kind = KIND["Residual"]

    def __init__(self, inner: Module):
        super().__init__()
        self.inner = inner

    def forward(self, x):
        return x + self.inner(x)

    def nxs_children(self):
        return [self.inner]


class PositionalEncoding(Module):
    kind = KIND["PositionalEncoding"]

    def __init__(self, embed: int, max_len: int = 512, learnable: bool = False):
        super().__init__()
        self.cfg = (embed, max_len, learnable)
        pe = torch.zeros(max_len, embed)
        pos = torch.arange(max_len)[:, None].float()
        div = torch.exp(torch.arange(0, embed, 2).float() * (-math.log(10000.0) / embed))
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)[:, : embed // 2]
        if learnable:
            self.pe = tnn.Parameter(pe)
        else:
            self.register_buffer("pe", pe)

    def forward(self, x):
        return x + self.pe[: x.shape[1]][None].to(x.dtype)

    def nxs_attrs(self):
        return [("embed", I32, self.cfg[0]), ("max_len", I32, self.cfg[1]), ("learnable", BOOL, self.cfg[2])]


class PythonModule(Module):
    """A user-defined module archived by name (its body travels in the archive's python payload)."""
    kind = KIND["PythonModule"]

    def __init__(self, name: str, inner: tnn.Module):
        super().__init__()
        self.layer_name = name
        self.inner = inner

    def forward(self, x):
        return self.inner(x)


class Sequential(Module):
    kind = KIND["Sequential"]

    def __init__(self, *layers: Module):
        super().__init__()
        self.layers = tnn.ModuleList(layers)

    def add(self, layer: Module) -> "Sequential":
        self.layers.append(layer)
        return self

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x

    def __len__(self):
        return len(self.layers)

    def __getitem__(self, i):
        return self.layers[i]

    def nxs_children(self):
        return list(self.layers)

    def save_nxs(self, path: str) -> None:
        from ..nxs.archive import save_model
        save_model(self, path)

    @staticmethod
    def load_nxs(path: str) -> "Sequential":
        from ..nxs.archive import load_model
        return load_model(path)


# ------------------------------------------------------------------------------- archive factory
def make_one(spec: dict) -> Module:
    """Rebuilds a layer from its archive description (weights are loaded separately, in order)."""
    k = spec["type"]
    a = lambda key, d=None: _attr(spec, key, d)
    if k == KIND["Linear"]: return Linear(a("in"), a("out"), a("bias"))
    if k in (KIND["Conv1d"], KIND["Conv2d"], KIND["Conv3d"]):
        cls = {KIND["Conv1d"]: Conv1d, KIND["Conv2d"]: Conv2d, KIND["Conv3d"]: Conv3d}[k]
        return cls(a("in"), a("out"), a("kernel"), a("stride"), a("padding"), a("bias"))
    if k == KIND["MultiHeadAttention"]: return MultiHeadAttention(a("embed"), a("heads"))
    if k == KIND["Lstm"]: return LSTM(a("input"), a("hidden"))
    if k == KIND["Gru"]: return GRU(a("input"), a("hidden"))
    if k == KIND["Rnn"]: return RNN(a("input"), a("hidden"))
    if k == KIND["TransformerEncoder"]: return TransformerEncoder(a("embed"), a("heads"), a("feedforward"))
    if k == KIND["TransformerDecoder"]: return TransformerDecoder(a("embed"), a("heads"), a("feedforward"))
    if k == KIND["CausalBlock"]: return CausalTransformerBlock(a("embed"), a("heads"), a("feedforward"))
    if k == KIND["Embedding"]: return Embedding(a("num"), a("dim"), a("padding"))
    if k == KIND["BatchNorm1d"]: return BatchNorm1d(a("features"))
    if k == KIND["BatchNorm2d"]: return BatchNorm2d(a("features"))
    if k == KIND["LayerNorm"]: return LayerNorm(a("size"), a("eps"))
    if k == KIND["GroupNorm"]: return GroupNorm(a("groups"), a("channels"))
    if k == KIND["InstanceNorm"]: return InstanceNorm(a("channels"))
    if k == KIND["Relu"]: return ReLU()
    if k == KIND["Swish"]: return swish()
    if k == KIND["NamedActivation"]:
        if spec["name"] not in _ACTIVATIONS:
            raise RuntimeError(f"activation body '{spec['name']}' is not registered in this process")
        return Activation(spec["name"])
    if k == KIND["PythonModule"]:
        from ..fnstore import module_factory
        return module_factory(spec["name"])
    if k == KIND["Dropout"]: return Dropout(a("p"))
    if k == KIND["MaxPool2d"]: return MaxPool2d(a("kernel"), a("stride"), a("padding"))
    if k == KIND["AvgPool2d"]: return AvgPool2d(a("kernel"), a("stride"), a("padding"))
    if k == KIND["GlobalAvgPool2d"]: return GlobalAvgPool2d()
    if k == KIND["Flatten"]: return Flatten()
    if k == KIND["DepthwiseConv2d"]: return DepthwiseConv2d(a("channels"), a("kernel"), a("stride"), a("padding"))
    if k == KIND["Residual"]:
        if len(spec["children"]) != 1:
            raise RuntimeError("residual nxs node needs one child")
        return Residual(make_one(spec["children"][0]))
    if k == KIND["Reshape"]: return Reshape([v for _, kind, v in spec["attrs"] if kind == I32])
    if k == KIND["PositionalEncoding"]: return PositionalEncoding(a("embed"), a("max_len"), a("learnable"))
    if k == KIND["Sequential"]: return Sequential(*[make_one(c) for c in spec["children"]])
    if k == KIND["Graph"]:
        from .graph import Graph
        return Graph.from_spec(spec)
    if k == KIND["Concat"]: raise RuntimeError("Concat is a graph merge, not a standalone layer")
    if k in (KIND["DecoderBlock"], KIND["LanguageModel"]):
        raise RuntimeError("DecoderBlock/LanguageModel archives load through lm.LanguageModel.load_nxs")
    raise RuntimeError("nxs layer type is unknown")
