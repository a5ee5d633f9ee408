"""The object model of the `nexus` Python shell: flat-list tensors, layers that own `{values, grad}` parameter
records, explicit `forward` / `backward`, builders, loaders and agents with the call signatures of the reference's
pybind module, implemented over :mod:`nexus_b200` (torch tensors inside).

Parity: python/src/nexus/__init__.py and the `nexus._core` surface that python/tests/test_kabuk.py, test_faz1-7.py and
test_graph_lm.py of the reference exercise.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import numpy as np
import torch

import nexus_b200 as _impl
import nexus_b200.custom  # noqa: F401
import nexus_b200.loss  # noqa: F401
import nexus_b200.metrics  # noqa: F401
import nexus_b200.optim  # noqa: F401
import nexus_b200.rl  # noqa: F401
import nexus_b200.train.callbacks  # noqa: F401
import nexus_b200.train.language  # noqa: F401
import nexus_b200.train.trainer  # noqa: F401
from nexus_b200 import fnstore as _fnstore
from nexus_b200 import nn as _nn


# ====================================================================================================== Tensor
class Tensor:
    """Dense FP32 tensor addressed the way the shell's users do: a shape list, flat lists in and out, scalar
    indexing, views that share storage, and the buffer protocol."""

    def __init__(self, shape: Sequence[int] = (), _t: Optional[torch.Tensor] = None):
        self._t = _t if _t is not None else torch.zeros([int(s) for s in shape], dtype=torch.float32)

    @staticmethod
    def wrap(t: torch.Tensor) -> "Tensor":
        return Tensor(_t=t)

    @property
    def shape(self) -> List[int]:
        return list(self._t.shape)

    def numel(self) -> int:
        return self._t.numel()

    def to_list(self) -> List[float]:
        return self._t.detach().reshape(-1).tolist()

    def copy_from(self, values) -> "Tensor":
        flat = torch.as_tensor(np.asarray(values, dtype=np.float32)).reshape(-1)
        if flat.numel() != self._t.numel():
            raise ValueError(f"copy_from: {flat.numel()} values for a tensor of {self._t.numel()} elements")
        with torch.no_grad():
            self._t.reshape(-1).copy_(flat) if self._t.is_contiguous() else self._t.copy_(flat.view(self._t.shape))
        return self

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(_t=self._t.view([int(s) for s in shape]))

    def fill(self, value: float) -> "Tensor":
        with torch.no_grad():
            self._t.fill_(value)
        return self

    def clone(self) -> "Tensor":
        return Tensor(_t=self._t.detach().clone())

    def torch(self) -> torch.Tensor:
        return self._t

    def _index(self, idx):
        if isinstance(idx, tuple):
            return tuple(int(i) for i in idx)
        if self._t.dim() > 1:            # a flat index into a multi-dimensional tensor
            return tuple(int(v) for v in np.unravel_index(int(idx), tuple(self._t.shape)))
        return (int(idx),)

    def __getitem__(self, idx) -> float:
        return float(self._t[self._index(idx)])

    def __setitem__(self, idx, value) -> None:
        with torch.no_grad():
            self._t[self._index(idx)] = float(value)

    def __len__(self) -> int:
        return self._t.shape[0] if self._t.dim() else 1

    def __buffer__(self, flags):
        return memoryview(self._t.detach().numpy())

    def __repr__(self) -> str:
        return f"nexus.Tensor(shape={self.shape})"


def _as_torch(x) -> torch.Tensor:
    if isinstance(x, Tensor):
        return x._t
    if isinstance(x, torch.Tensor):
        return x
    return torch.as_tensor(np.asarray(x, dtype=np.float32))


# ================================================================================================ layer wrapper
class Layer:
    """A shell layer: wraps one :mod:`nexus_b200.nn` module, runs it with an explicit backward."""

    def __init__(self, module: torch.nn.Module):
        self._m = module
        self._last_in = None
        self._last_out = None
        for p in module.parameters():
            if p.grad is None:
                p.grad = torch.zeros_like(p)

    # -- parameters ---------------------------------------------------------------------------------------
    def parameters(self) -> List[dict]:
        out = []
        for name, p in self._m.named_parameters():
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            out.append({"name": name, "values": Tensor.wrap(p.data), "grad": Tensor.wrap(p.grad)})
        return out

    def zero_grad(self) -> None:
        for p in self._m.parameters():
            if p.grad is not None:
                p.grad.zero_()

    # -- execution ----------------------------------------------------------------------------------------
    def forward(self, x) -> Tensor:
        t = _as_torch(x).detach().clone().requires_grad_(True)
        inp = t.long() if _wants_integer_input(self._m) else t
        out = self._m(inp)
        self._last_in, self._last_out = t, out
        return Tensor.wrap(out.detach())

    def backward(self, grad) -> Tensor:
        """Gradient of the last forward: accumulates into the parameters' `grad`, returns the input gradient."""
        if self._last_out is None:
            raise RuntimeError("backward called before forward")
        g = _as_torch(grad).reshape(self._last_out.shape)
        self._last_out.backward(g)
        gin = self._last_in.grad
        self._last_out = None
        return Tensor.wrap(gin if gin is not None else torch.zeros_like(self._last_in))

    def train(self, mode: bool = True):
        self._m.train(mode)
        return self

    def eval(self):
        return self.train(False)

    def save_nxs(self, path: str) -> None:
        from nexus_b200.nxs.archive import save_model
        save_model(self._m, path)

    def module(self) -> torch.nn.Module:
        return self._m

    def __call__(self, x) -> Tensor:
        return self.forward(x)


def _wants_integer_input(m: torch.nn.Module) -> bool:
    first = m
    while isinstance(first, _nn.Sequential) and len(first.layers):
        first = first.layers[0]
    return isinstance(first, _nn.Embedding)


def _unwrap(layer) -> torch.nn.Module:
    return layer._m if isinstance(layer, Layer) else layer


class Sequential(Layer):
    def __init__(self, *layers):
        super().__init__(_nn.Sequential(*[_unwrap(l) for l in layers]))

    def add(self, layer) -> "Sequential":
        self._m.add(_unwrap(layer))
        for p in self._m.parameters():
            if p.grad is None:
                p.grad = torch.zeros_like(p)
        return self

    def __len__(self) -> int:
        return len(self._m)


class Graph(Layer):
    def __init__(self):
        super().__init__(_nn.Graph())

    def add(self, name: str, layer, inputs: Optional[Sequence[str]] = None) -> "Graph":
        self._m.add(name, _unwrap(layer), inputs)
        return self

    def concat(self, name: str, layer, inputs: Sequence[str]) -> "Graph":
        self._m.concat(name, _unwrap(layer), list(inputs))
        return self

    def set_output(self, name: str) -> "Graph":
        self._m.set_output(name)
        return self


def _factory(cls):
    def make(*args, **kw):
        return Layer(cls(*args, **kw))
    make.__name__ = cls.__name__
    make.__doc__ = cls.__doc__
    return make


Linear = _factory(_nn.Linear)
Conv1d, Conv2d, Conv3d = _factory(_nn.Conv1d), _factory(_nn.Conv2d), _factory(_nn.Conv3d)
DepthwiseConv2d = _factory(_nn.DepthwiseConv2d)
MultiHeadAttention = _factory(_nn.MultiHeadAttention)
LSTM, GRU, RNN = _factory(_nn.LSTM), _factory(_nn.GRU), _factory(_nn.RNN)
TransformerEncoder, TransformerDecoder = _factory(_nn.TransformerEncoder), _factory(_nn.TransformerDecoder)
CausalTransformerBlock = _factory(_nn.CausalTransformerBlock)
Embedding = _factory(_nn.Embedding)
BatchNorm1d, BatchNorm2d = _factory(_nn.BatchNorm1d), _factory(_nn.BatchNorm2d)
LayerNorm, GroupNorm, InstanceNorm = _factory(_nn.LayerNorm), _factory(_nn.GroupNorm), _factory(_nn.InstanceNorm)
ReLU = _factory(_nn.ReLU)
Dropout = _factory(_nn.Dropout)
MaxPool2d, AvgPool2d, GlobalAvgPool2d = _factory(_nn.MaxPool2d), _factory(_nn.AvgPool2d), _factory(_nn.GlobalAvgPool2d)
Flatten, Reshape = _factory(_nn.Flatten), _factory(_nn.Reshape)
PositionalEncoding = _factory(_nn.PositionalEncoding)


def Residual(inner):
    return Layer(_nn.Residual(_unwrap(inner)))


def swish():
    return Layer(_nn.swish())


def gelu():
    return Layer(_nn.GELU())


def silu():
    return Layer(_nn.SiLU())


def mish():
    return Layer(_nn.Mish())


# ------------------------------------------------------------------------------- python-defined activations
def activation(name: str, forward: Callable, backward: Optional[Callable] = None):
    """Named activation from Python bodies ``forward(x) -> y`` (and optionally ``backward(x) -> dy/dx``) over one
    number.  The bodies are archived with any model that uses the activation (closures over numbers only)."""
    if name != "Swish":
        try:
            _fnstore.remember(name, forward, backward)
        except TypeError as e:
            raise TypeError("kapali degiskenli fonksiyon dosyaya yazilmaz (a python body may only close over "
                            "float, int or bool values): %s" % e) from None
    _nn.register_activation(name, _fnstore.tensor_level(forward, backward))
    return Layer(_nn.Activation(name))


# ----------------------------------------------------------------------------------- python-defined modules
class _PyModuleFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mod, *params):
        ctx.mod = mod
        ctx.save_for_backward(x)
        out = mod._fwd(Tensor.wrap(x.detach().clone()), [Tensor.wrap(p.data) for p in mod._ps])
        return _as_torch(out).detach().clone().view(-1).view(_as_torch(out).shape)

    @staticmethod
    def backward(ctx, g):
        mod = ctx.mod
        if mod._bwd is None:
            raise RuntimeError(f"python module '{mod.layer_name}' has no backward body")
        recs = []
        scratch = []
        for p in mod._ps:
            gbuf = torch.zeros_like(p)
            scratch.append(gbuf)
            recs.append({"values": Tensor.wrap(p.data), "grad": Tensor.wrap(gbuf)})
        gin = mod._bwd(Tensor.wrap(g.detach().clone()), recs)
        return (_as_torch(gin).detach().clone(), None) + tuple(scratch)


class _PyModule(_nn.PythonModule):
    """`nn.PythonModule` whose body is a pair of Python functions over shell tensors:
    ``forward(values, params) -> out`` and ``backward(grad, params) -> grad_in`` (the latter writes the parameter
    gradients into ``params[i]["grad"]``); ``shapes`` lists the parameter shapes."""

    def __init__(self, name: str, forward: Callable, backward: Optional[Callable], shapes):
        holder = torch.nn.Module()
        super().__init__(name, holder)
        self._fwd, self._bwd = forward, backward
        self._ps = torch.nn.ParameterList([torch.nn.Parameter(torch.zeros([int(s) for s in shp])) for shp in shapes])
        holder.params = self._ps

    def forward(self, x):
        return _PyModuleFn.apply(x, self, *self._ps)


def _py_module_factory(name, forward, backward, shapes):
    return lambda: _PyModule(name, forward, backward, shapes)


def PythonModule(name: str, forward: Callable, backward: Optional[Callable] = None, shapes=None):
    shapes = [list(s) for s in (shapes or [])]
    _fnstore.remember_module(name, forward, backward, shapes, builder=_py_module_factory)
    return Layer(_PyModule(name, forward, backward, shapes))


def conv2d_device(nchw, weight, bias, batch, in_ch, height, width, out_ch, kernel_h, kernel_w, stride, padding):
    """Explicit device convolution on flat lists (CUDA when available, else CPU).  Returns
    ``{"nchw": [...], "height": h, "width": w}``."""
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    x = torch.tensor(nchw, dtype=torch.float32, device=dev).view(batch, in_ch, height, width)
    w = torch.tensor(weight, dtype=torch.float32, device=dev).view(out_ch, in_ch, kernel_h, kernel_w)
    b = torch.tensor(bias, dtype=torch.float32, device=dev) if bias is not None and len(bias) else None
    y = torch.nn.functional.conv2d(x, w, b, stride=stride, padding=padding)
    return {"nchw": y.reshape(-1).cpu().tolist(), "height": y.shape[2], "width": y.shape[3], "channels": y.shape[1]}


# ========================================================================================================= io
def load(path: str):
    """Rebuilds whatever the archive holds: a network (as a shell layer) or a language model."""
    from nexus_b200.nxs.archive import load_model
    m = load_model(path)
    if isinstance(m, _nn.Sequential):
        out = Sequential()
        out._m = m
    elif isinstance(m, _nn.Graph):
        out = Graph()
        out._m = m
    elif isinstance(m, _nn.Module):
        out = Layer(m)
    else:
        return m
    for p in m.parameters():
        if p.grad is None:
            p.grad = torch.zeros_like(p)
    return out


def save(model, path: str) -> None:
    if isinstance(model, Layer):
        model.save_nxs(path)
    elif hasattr(model, "save_nxs"):
        model.save_nxs(path)
    else:
        from nexus_b200.nxs.archive import save_model
        save_model(model, path)


# ======================================================================================================= data
class DataLoader:
    """``DataLoader(features, labels, features_per_sample, batch_size, shuffle, seed)`` over flat lists.
    `next()` returns ``{"features", "labels", "batch_size"}`` or ``None`` at the end of the pass; iterating yields
    ``(x [n, F], y [n])`` tensors for the trainers."""

    def __init__(self, features, labels, features_per_sample: int, batch_size: int, shuffle: bool = False, seed: int = 0):
        self._f = int(features_per_sample)
        self._x = np.asarray(features, dtype=np.float32).reshape(-1, self._f)
        self._y = np.asarray(labels, dtype=np.int64)
        if len(self._x) != len(self._y):
            raise ValueError("DataLoader: features and labels disagree on the number of samples")
        self._bs, self._shuffle, self._seed = int(batch_size), bool(shuffle), int(seed)
        self._epoch = 0
        self.reset()

    def features_per_sample(self) -> int:
        return self._f

    def size(self) -> int:
        return len(self._y)

    def reset(self) -> None:
        self._order = np.arange(len(self._y))
        if self._shuffle:
            np.random.default_rng(self._seed + self._epoch).shuffle(self._order)
        self._epoch += 1
        self._pos = 0

    def next(self) -> Optional[dict]:
        if self._pos >= len(self._order):
            return None
        sel = self._order[self._pos: self._pos + self._bs]
        self._pos += self._bs
        return {"features": self._x[sel].reshape(-1).tolist(), "labels": self._y[sel].tolist(), "batch_size": len(sel)}

    def __iter__(self):
        self.reset()
        while self._pos < len(self._order):
            sel = self._order[self._pos: self._pos + self._bs]
            self._pos += self._bs
            yield torch.from_numpy(self._x[sel]), torch.from_numpy(self._y[sel])

    def __len__(self) -> int:
        return (len(self._y) + self._bs - 1) // self._bs


class CsvTable:
    def __init__(self, features: np.ndarray, labels: np.ndarray):
        self.features = features.reshape(-1).tolist()
        self.labels = labels.astype(np.int64).tolist()
        self.features_per_sample = features.shape[1]
        self.rows = features.shape[0]


def read_csv(path: str) -> CsvTable:
    """Numeric CSV without a header: the last column is the integer label, the others are features."""
    rows = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                rows.append([float(v) for v in line.split(",")])
    arr = np.asarray(rows, dtype=np.float32)
    return CsvTable(arr[:, :-1], arr[:, -1])


def save_image(path: str, chw, height: int, width: int, channels: int) -> None:
    """Writes a CHW float image in [0, 1] as an 8-bit file (format from the extension)."""
    from PIL import Image
    a = np.asarray(chw, dtype=np.float32).reshape(channels, height, width)
    img = (np.clip(a, 0.0, 1.0) * 255.0 + 0.5).astype(np.uint8).transpose(1, 2, 0)
    Image.fromarray(img[:, :, 0] if channels == 1 else img, "L" if channels == 1 else ("RGB" if channels == 3 else "RGBA")).save(path)


def load_image(path: str, channels: int = 0, height: int = 0, width: int = 0) -> dict:
    """``{"chw", "height", "width", "channels"}``; optional channel conversion (1 grey, 3 RGB, 4 RGBA) and resize."""
    from PIL import Image
    img = Image.open(path)
    if channels:
        img = img.convert({1: "L", 3: "RGB", 4: "RGBA"}[channels])
    elif img.mode not in ("L", "RGB", "RGBA"):
        img = img.convert("RGB")
    if height and width:
        img = img.resize((width, height), Image.BILINEAR)
    a = np.asarray(img, dtype=np.float32) / 255.0
    if a.ndim == 2:
        a = a[:, :, None]
    return {"chw": a.transpose(2, 0, 1).reshape(-1).tolist(), "height": a.shape[0], "width": a.shape[1],
            "channels": a.shape[2]}


# ====================================================================================================== optim
class _ShellOptimizer:
    def __init__(self, inner):
        self._o = inner

    def learning_rate(self) -> float:
        return float(self._o.lr)

    def set_learning_rate(self, lr: float) -> None:
        self._o.lr = float(lr)

    def zero_grad(self) -> None:
        self._o.zero_grad()

    def step(self) -> None:
        self._o.step()


def _params_of(model):
    return list(_unwrap(model).parameters())


def SGD(model, lr: float = 1e-2, momentum: float = 0.0, weight_decay: float = 0.0):
    return _ShellOptimizer(_impl.optim.SGD(_params_of(model), lr, momentum, weight_decay))


def AdamW(model, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01):
    return _ShellOptimizer(_impl.optim.AdamW(_params_of(model), lr, beta1, beta2, eps, weight_decay))


class CosineAnnealing:
    """``CosineAnnealing(base_lr, total_epochs, min_lr=0)``: `value(epoch)` and the multiplicative `factor(epoch)`."""

    def __init__(self, base_lr: float, total: int, min_lr: float = 0.0):
        self.base_lr, self.total, self.min_lr = float(base_lr), max(int(total), 1), float(min_lr)

    def value(self, epoch: int) -> float:
        t = min(max(epoch, 0), self.total) / self.total
        return self.min_lr + 0.5 * (self.base_lr - self.min_lr) * (1.0 + math.cos(math.pi * t))

    def factor(self, epoch: int) -> float:
        return self.value(epoch) / self.base_lr if self.base_lr else 1.0


# ======================================================================================================= loss
class CrossEntropy:
    def __init__(self, label_smoothing: float = 0.0):
        self._l = _impl.loss.CrossEntropy(label_smoothing)

    def forward_backward(self, logits, labels, classes: int) -> dict:
        lg = torch.as_tensor(np.asarray(logits, dtype=np.float32)).view(-1, int(classes))
        loss, grad = self._l.forward_backward(lg, torch.as_tensor(np.asarray(labels, dtype=np.int64)))
        return {"loss": float(loss), "grad": grad.reshape(-1).tolist()}


class _ShellElementwise:
    _cls = None

    def __init__(self, *a):
        self._l = self._cls(*a)

    def forward_backward(self, pred, target):
        loss, grad = self._l.forward_backward(torch.as_tensor(np.asarray(pred, dtype=np.float32)),
                                              torch.as_tensor(np.asarray(target, dtype=np.float32)))
        return float(loss), grad.reshape(-1).tolist()


class MSE(_ShellElementwise):
    _cls = _impl.loss.MSE


class MAE(_ShellElementwise):
    _cls = _impl.loss.MAE


class Huber(_ShellElementwise):
    _cls = _impl.loss.Huber


class BCE(_ShellElementwise):
    _cls = _impl.loss.BCE


# ==================================================================================================== metrics
class Accuracy:
    name = "accuracy"

    def __init__(self):
        self._m = _impl.metrics.Accuracy()

    def update(self, logits, labels, classes: int = 0) -> None:
        if isinstance(logits, torch.Tensor):
            self._m.update(logits, torch.as_tensor(labels))
            return
        lg = torch.as_tensor(np.asarray(logits, dtype=np.float32))
        self._m.update(lg.view(-1, int(classes)) if classes else lg, torch.as_tensor(np.asarray(labels, dtype=np.int64)))

    def value(self) -> float:
        return float(self._m.value())

    def reset(self) -> None:
        self._m.reset()


# ===================================================================================================== linalg
def gemm(m: int, n: int, k: int, a, b) -> List[float]:
    """Row-major C[m, n] = A[m, k] @ B[k, n] on flat lists (the tcgen05 GEMM on a GPU for BF16-friendly sizes)."""
    A = torch.as_tensor(np.asarray(a, dtype=np.float32)).view(m, k)
    B = torch.as_tensor(np.asarray(b, dtype=np.float32)).view(k, n)
    return (A @ B).reshape(-1).tolist()


def kernel_name() -> str:
    if torch.cuda.is_available():
        return "tcgen05 persistent GEMM (sm_100a, TMA + TMEM, CTA pairs)"
    return "native CPU GEMM (blocked FP32, thread pool)"


# ====================================================================================================== train
class Callback:
    """Subclass and override `on_epoch_end(state)` (``state``: dict with epoch, train_loss, val_loss, metrics) and
    `stop()` (return True to end training after the current epoch)."""

    def on_epoch_end(self, state: dict) -> None:
        pass

    def stop(self) -> bool:
        return False


class ProgressLogger(Callback):
    def __init__(self, verbose: bool = False):
        self._last = None
        self._verbose = verbose

    def on_epoch_end(self, state: dict) -> None:
        self._last = dict(state)
        if self._verbose:
            print(f"epoch {state['epoch']}: train {state['train_loss']:.4f} val {state['val_loss']:.4f}", flush=True)

    def last(self) -> Optional[dict]:
        return self._last


class _CallbackAdapter(_impl.train.callbacks.Callback):
    def __init__(self, cb: Callback):
        self.cb = cb

    def on_epoch_end(self, trainer, stats):
        self.cb.on_epoch_end({"epoch": stats.epoch, "train_loss": stats.train_loss, "val_loss": stats.val_loss,
                              "metrics": dict(stats.metrics), "lr": stats.lr})
        return not self.cb.stop()


class TrainerBuilder:
    """``TrainerBuilder(model).adamw(model, lr=...).loss(0.0).execution_policy_cpu().gradient_clip_norm(1.0)
    .accuracy().cosine(schedule).callback(cb).mixed_precision(False).build()``."""

    def __init__(self, model):
        self._model = model
        self._b = _impl.train.trainer.TrainerBuilder(_unwrap(model))

    def adamw(self, model=None, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
              weight_decay: float = 0.01):
        if isinstance(model, (int, float)):
            lr = float(model)
        self._b.adamw(lr, beta1, beta2, eps, weight_decay)
        return self

    def sgd(self, model=None, lr: float = 1e-2, momentum: float = 0.0, weight_decay: float = 0.0):
        if isinstance(model, (int, float)):
            lr = float(model)
        self._b.sgd(lr, momentum, weight_decay)
        return self

    def loss(self, label_smoothing: float = 0.0):
        self._b.loss(float(label_smoothing))
        return self

    def execution_policy_cpu(self):
        self._b.execution_policy("cpu")
        return self

    def execution_policy_cuda(self, device: int = 0):
        self._b.execution_policy(f"cuda:{device}")
        return self

    def gradient_clip_norm(self, c: float):
        self._b.gradient_clip_norm(float(c))
        return self

    def gradient_accumulation(self, n: int):
        self._b.gradient_accumulation(n)
        return self

    def accuracy(self):
        self._b.metric(_impl.metrics.Accuracy())
        return self

    def cosine(self, schedule: CosineAnnealing):
        self._b.learning_rate_schedule(schedule)
        return self

    def callback(self, cb):
        self._b.callback(_CallbackAdapter(cb) if isinstance(cb, Callback) else cb)
        return self

    def mixed_precision(self, on: bool = True):
        self._b.mixed_precision(bool(on))
        return self

    def build(self) -> "Trainer":
        return Trainer(self._b.build(), self._model)


class Trainer:
    def __init__(self, inner, model):
        self._t, self._model = inner, model

    def fit(self, train: DataLoader, val: Optional[DataLoader] = None, epochs: int = 1):
        self._t.fit(train, val, int(epochs))
        return self.history()

    def history(self):
        return list(self._t.history)

    def epochs_ran(self) -> int:
        return len(self._t.history)

    def evaluate(self, loader: DataLoader) -> dict:
        loss, mets = self._t.evaluate(loader)
        return {"loss": float(loss), **{k: float(v) for k, v in mets.items()}}

    def save_nxs(self, path: str) -> None:
        self._t.save_nxs(path)

    def load_nxs(self, path: str) -> None:
        self._t.load_nxs(path)


class LanguageTrainer:
    """``LanguageTrainer(model, lr).fit(rows, epochs)`` on next-token prediction; ``rows`` is a list of equally long
    token lists.  Returns the mean loss of the last epoch."""

    def __init__(self, model, lr: float = 3e-4, weight_decay: float = 0.0):
        self._t = _impl.train.language.LanguageTrainer(_unwrap(model), lr, weight_decay)

    def fit(self, rows, epochs: int = 1) -> float:
        arr = np.asarray(rows, dtype=np.int32)
        tr = _impl.train.language.TokenRows(arr.reshape(-1), arr.shape[0], arr.shape[1])
        return float(self._t.fit(tr, int(epochs))[-1])


def all_reduce_mean(ranks):
    """Mean over the ranks of equally shaped flat lists; every rank receives the same result."""
    arr = np.asarray(ranks, dtype=np.float64)
    mean = arr.mean(axis=0).tolist()
    return [list(mean) for _ in range(arr.shape[0])]


# ===================================================================================================== custom
class MicroTape:
    """Scalar reverse-mode tape addressed by node index."""

    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self._tape = _impl.custom.MicroTape()
        self._vars = []
        self._grads = None

    def _push(self, var) -> int:
        self._vars.append(var)
        return len(self._vars) - 1

    def input(self, value: float) -> int:
        make = getattr(self._tape, "input", None) or getattr(self._tape, "var", None) or self._tape.const
        return self._push(make(float(value)))

    def const(self, value: float) -> int:
        return self._push(self._tape.const(float(value)))

    def add(self, a: int, b: int) -> int: return self._push(self._vars[a] + self._vars[b])
    def sub(self, a: int, b: int) -> int: return self._push(self._vars[a] - self._vars[b])
    def mul(self, a: int, b: int) -> int: return self._push(self._vars[a] * self._vars[b])
    def div(self, a: int, b: int) -> int: return self._push(self._vars[a] / self._vars[b])
    def square(self, a: int) -> int: return self._push(self._tape.square(self._vars[a]))
    def exp(self, a: int) -> int: return self._push(self._tape.exp(self._vars[a]))
    def log(self, a: int) -> int: return self._push(self._tape.log(self._vars[a]))

    def backward(self, out: int) -> None:
        self._grads = self._tape.gradient(self._vars[out])

    def value(self, i: int) -> float:
        return float(self._vars[i].value)

    def grad(self, i: int) -> float:
        if self._grads is None:
            raise RuntimeError("MicroTape.grad before backward")
        return float(self._grads[self._vars[i].idx])

    def size(self) -> int:
        return len(self._vars)


class Tape:
    """Tensor tape over shell layers: `input(tensor)`, `apply(layer, node)`, `relu(node)`, `backward(node)`
    (accumulates into the layers' parameter gradients)."""

    def __init__(self):
        self._nodes: List[torch.Tensor] = []

    def input(self, values) -> int:
        self._nodes.append(_as_torch(values).detach().clone().requires_grad_(True))
        return len(self._nodes) - 1

    def apply(self, layer, node: int) -> int:
        self._nodes.append(_unwrap(layer)(self._nodes[node]))
        return len(self._nodes) - 1

    def relu(self, node: int) -> int:
        self._nodes.append(torch.relu(self._nodes[node]))
        return len(self._nodes) - 1

    def add(self, a: int, b: int) -> int:
        self._nodes.append(self._nodes[a] + self._nodes[b])
        return len(self._nodes) - 1

    def value(self, node: int) -> Tensor:
        return Tensor.wrap(self._nodes[node].detach())

    def backward(self, node: int, grad=None) -> None:
        out = self._nodes[node]
        out.backward(torch.ones_like(out) if grad is None else _as_torch(grad).reshape(out.shape))

    def size(self) -> int:
        return len(self._nodes)

    def reset(self) -> None:
        self._nodes = []


# ========================================================================================================= rl
class Environment:
    """Base class for environments written in Python: ``super().__init__(observation_dim, action_count, discrete)``,
    then override `reset(seed) -> observation` and `step(action) -> {"observation", "reward", "terminated",
    "truncated", "info"}`."""

    def __init__(self, observation_dim: int, action_count: int, discrete: bool = True):
        self._obs_dim, self._actions, self._discrete = int(observation_dim), int(action_count), bool(discrete)

    def observation_dim(self) -> int:
        return self._obs_dim

    def action_count(self) -> int:
        return self._actions

    def discrete(self) -> bool:
        return self._discrete

    def reset(self, seed: int = 0):
        raise NotImplementedError

    def step(self, action):
        raise NotImplementedError


class _NativeEnvironment(Environment):
    def __init__(self, env):
        self._e = env
        super().__init__(env.observation_space.n, env.action_space.n, env.action_space.kind == "discrete")

    def reset(self, seed: int = 0):
        return [float(v) for v in self._e.reset(int(seed))]

    def step(self, action) -> dict:
        obs, r, term, trunc = self._e.step(action)
        return {"observation": [float(v) for v in obs], "reward": float(r), "terminated": bool(term),
                "truncated": bool(trunc), "info": ""}


def LineWorld(length: int = 5, horizon: int = 12) -> Environment:
    return _NativeEnvironment(_impl.rl.LineWorld(length, horizon))


def GridWorld(size: int = 4, horizon: int = 24) -> Environment:
    return _NativeEnvironment(_impl.rl.GridWorld(size, horizon))


def CartPole() -> Environment:
    return _NativeEnvironment(_impl.rl.CartPole())


def PointMass() -> Environment:
    return _NativeEnvironment(_impl.rl.PointMass())


class VectorEnv:
    def __init__(self, inner, obs_dim: int):
        self._v, self._obs_dim = inner, obs_dim

    @staticmethod
    def line_worlds(count: int, length: int = 5, horizon: int = 12) -> "VectorEnv":
        v = _impl.rl.VectorEnv("LineWorld", int(count), length, horizon)
        return VectorEnv(v, v.obs_dim)

    def size(self) -> int:
        return self._v.size

    def reset(self, seed: int = 0) -> List[float]:
        return np.asarray(self._v.reset(), dtype=np.float32).reshape(-1).tolist()

    def step(self, actions) -> dict:
        out = self._v.step(actions)
        obs, rew, term, trunc = out[0], out[1], out[2], out[3]
        return {"observations": np.asarray(obs, np.float32).reshape(-1).tolist(),
                "rewards": [float(r) for r in np.asarray(rew).reshape(-1)],
                "terminated": [bool(t) for t in np.asarray(term).reshape(-1)],
                "truncated": [bool(t) for t in np.asarray(trunc).reshape(-1)]}


class PPOConfig:
    def __init__(self):
        d = _impl.rl.PpoConfig()
        self.hidden, self.lr, self.gamma, self.lam, self.clip = d.hidden, d.lr, d.gamma, d.lam, d.clip
        self.value_coef, self.entropy_coef, self.epochs, self.minibatch = d.value_coef, d.entropy_coef, d.epochs, d.minibatch
        self.seed = d.seed


class PPOAgent:
    def __init__(self, observation_dim: int, action_count: int, config: Optional[PPOConfig] = None, _inner=None):
        if _inner is not None:
            self._a = _inner
            return
        c = config or PPOConfig()
        self._a = _impl.rl.Ppo(_impl.rl.PpoConfig(obs_dim=int(observation_dim), actions=int(action_count), hidden=c.hidden,
                                                  lr=c.lr, gamma=c.gamma, lam=c.lam, clip=c.clip, value_coef=c.value_coef,
                                                  entropy_coef=c.entropy_coef, epochs=c.epochs, minibatch=c.minibatch,
                                                  seed=c.seed))

    def act(self, observation, deterministic: bool = False):
        return self._a.act(np.asarray(observation, np.float32), bool(deterministic))

    def learn(self, env: Environment, iterations: int, steps: int) -> dict:
        """``iterations`` rounds of ``steps`` environment steps followed by one PPO update each."""
        stats = {}
        obs = env.reset(self._a.cfg.seed)
        for _ in range(int(iterations)):
            last_done, nxt = False, obs
            for _s in range(int(steps)):
                a, logp, val = self._a.act(np.asarray(obs, np.float32))
                st = env.step(a)
                nxt, done = st["observation"], bool(st["terminated"] or st["truncated"])
                self._a.buf.add(obs, [a], logp, st["reward"], val, done)
                obs, last_done = (env.reset(self._a.cfg.seed) if done else nxt), done
            with torch.no_grad():
                last = 0.0 if last_done else float(self._a.v(torch.as_tensor(np.asarray(obs, np.float32))[None]))
            stats = self._a.update(last)
        return stats

    def save_nxs(self, path: str) -> None:
        self._a.save_nxs(path)

    @staticmethod
    def load_nxs(path: str) -> "PPOAgent":
        return PPOAgent(0, 0, _inner=_impl.rl.Ppo.load_nxs(path))


class ActorCriticAgent:
    def __init__(self, inner):
        self._a = inner

    @staticmethod
    def discrete(observation_dim: int, action_count: int, seed: int = 0) -> "ActorCriticAgent":
        return ActorCriticAgent(_impl.rl.ActorCritic(_impl.rl.ActorCriticConfig(obs_dim=int(observation_dim),
                                                                                  actions=int(action_count), seed=int(seed))))

    def act(self, observation, deterministic: bool = False):
        o = torch.as_tensor(np.asarray(observation, np.float32))[None]
        a = self._a.act(np.asarray(observation, np.float32), bool(deterministic))
        with torch.no_grad():
            logp = float(torch.log_softmax(self._a.pi(o)[0], -1)[int(a)])
            val = float(self._a.v(o))
        return int(a), logp, val

    def observe(self, obs, action, reward, next_obs, done) -> float:
        return self._a.observe(obs, action, reward, next_obs, done)

    def save_nxs(self, path: str) -> None:
        self._a.save_nxs(path)


class ContinuousActorCritic:
    def __init__(self, observation_dim: int, action_dim: int, seed: int = 0):
        self._a = _impl.rl.ContinuousActorCritic(_impl.rl.ActorCriticConfig(obs_dim=int(observation_dim),
                                                                            actions=int(action_dim), seed=int(seed)))

    def act(self, observation, deterministic: bool = False):
        a = np.tanh(np.asarray(self._a.act(np.asarray(observation, np.float32), bool(deterministic)), dtype=np.float64))
        return float(a[0]) if a.size == 1 else [float(v) for v in a]

    def observe(self, obs, action, reward, next_obs, done) -> float:
        return self._a.observe(obs, action, reward, next_obs, done)


class ReplayBuffer:
    def __init__(self, capacity: int, observation_dim: int):
        self._b = _impl.rl.ReplayBuffer(int(capacity), int(observation_dim))

    def add(self, obs, action, reward, next_obs, done) -> int:
        return self._b.add(obs, action, reward, next_obs, done)

    def size(self) -> int:
        return len(self._b)

    @staticmethod
    def _lists(d: dict) -> dict:
        return {"observations": d["obs"].reshape(-1).tolist(), "actions": [int(a) for a in d["act"].reshape(-1)],
                "rewards": d["rew"].tolist(), "next_observations": d["next_obs"].reshape(-1).tolist(),
                "dones": [bool(x) for x in d["done"]]}

    def sample(self, indices) -> dict:
        idx = np.asarray(indices, dtype=np.int64) if not isinstance(indices, int) else \
            self._b.rng.integers(0, len(self._b), size=indices)
        return self._lists(self._b._batch(idx))


class PrioritizedReplayBuffer:
    def __init__(self, capacity: int, observation_dim: int, alpha: float = 0.6):
        self._b = _impl.rl.PrioritizedReplayBuffer(int(capacity), int(observation_dim), alpha=float(alpha))

    def add(self, obs, action, reward, next_obs, done, priority: float = 1.0) -> int:
        i = self._b.add(obs, action, reward, next_obs, done)
        self._b.update_priorities([i], [float(priority)])
        return i

    def sample(self, batch: int, beta: float = 0.4, seed: int = 0) -> dict:
        self._b.beta = float(beta)
        self._b.rng = np.random.default_rng(int(seed))
        d = self._b.sample(int(batch))
        out = ReplayBuffer._lists(d)
        out["weights"] = d["weight"].tolist()
        out["indices"] = [int(i) for i in d["idx"]]
        return out

    def update_priorities(self, indices, td_errors) -> None:
        self._b.update_priorities(indices, td_errors)


class RolloutBuffer:
    """``reset(envs, observation_dim)``, ``add(obs, action, log_prob, value, reward, done)``, ``finish(gamma, lam,
    last_value)``; then `actions()`, `advantages()`, `returns()`."""

    def __init__(self):
        self._b = _impl.rl.RolloutBuffer()
        self._out = None

    def reset(self, envs: int = 1, observation_dim: int = 0) -> None:
        self._b.clear()
        self._out = None

    def add(self, obs, action, log_prob, value, reward, done) -> None:
        self._b.add(obs, [action], log_prob, reward, value, done)

    def finish(self, gamma: float = 0.99, lam: float = 0.95, last_value: float = 0.0) -> None:
        self._out = self._b.finish(float(last_value), float(gamma), float(lam), normalize=False)

    def size(self) -> int:
        return len(self._b)

    def actions(self) -> List[int]:
        return [int(a[0]) for a in self._b.act]

    def advantages(self) -> List[float]:
        return self._out["adv"].tolist()

    def returns(self) -> List[float]:
        return self._out["ret"].tolist()


class League:
    def __init__(self, _inner=None):
        self._l = _inner or _impl.rl.League()

    def add_player(self, elo: float = 1000.0) -> int:
        return self._l.add_player(elo)

    def save(self, player: int, weights) -> None:
        self._l.save(player, weights)

    def weights(self, player: int) -> List[float]:
        return [float(v) for v in self._l.weights(player)]

    def elo(self, player: int) -> float:
        return float(self._l.elo(player))

    def result(self, first: int, second: int, score_first: float, k: float = 32.0) -> None:
        self._l.result(first, second, score_first, k)

    def size(self) -> int:
        return self._l.size()

    def save_nxs(self, path: str) -> None:
        self._l.save_nxs(path)

    @staticmethod
    def load_nxs(path: str) -> "League":
        return League(_impl.rl.League.load_nxs(path))
