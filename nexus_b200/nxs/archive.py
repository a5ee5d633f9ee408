"""NXS2 archives of models, optimizers, trainers, RL agents and language models.

The byte-level codec is native (`_native.nxs2_encode/decode`); this module maps framework objects
to the archive dict and back.  Catalog models store their parameters in order under decimal names
("0", "1", ...); language models store a root node of type 35 with the config JSON embedded
(attrs ``config`` and ``format=1``), one child of type 34 per block (type 36 grand-children for MoE
layers) and weights under their real names.

Parity: include/nexus/model/nxs_format.hpp:217-233, src/model/nxs.cpp:535-660 and
`LanguageModel::save_nxs` in src/lm/model.cpp of the reference.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from .. import _native


class NxsError(RuntimeError):
    pass


def save_archive(path: str, archive: dict) -> None:
    data = _native.nxs2_encode(archive)
    with open(path, "wb") as f:
        f.write(data)


def load_archive(path: str) -> dict:
    with open(path, "rb") as f:
        data = f.read()
    try:
        return _native.nxs2_decode(data)
    except RuntimeError as e:
        raise NxsError(str(e)) from e


# ------------------------------------------------------------------------------- catalog models
def _weights_of(model: torch.nn.Module) -> list:
    out = []
    for i, p in enumerate(model.parameters()):
        out.append((str(i), list(p.shape), p.detach().float().cpu().numpy().reshape(-1)))
    for j, (name, b) in enumerate(model.named_buffers()):
        if b is not None and b.is_floating_point():
            out.append((f"buffer.{name}", list(b.shape), b.detach().float().cpu().numpy().reshape(-1)))
    return out


def _load_weights(model: torch.nn.Module, weights: list) -> None:
    params = list(model.parameters())
    bufs = dict(model.named_buffers())
    plain = [w for w in weights if not w[0].startswith("buffer.")]
    if len(plain) != len(params):
        raise NxsError(f"archive holds {len(plain)} weight tensors, the model has {len(params)}")
    with torch.no_grad():
        for p, (name, dims, vals) in zip(params, plain):
            if list(p.shape) != [int(d) for d in dims]:
                raise NxsError(f"weight {name}: shape {list(dims)} does not match {list(p.shape)}")
            p.copy_(torch.from_numpy(np.asarray(vals, dtype=np.float32)).view(p.shape))
        for name, dims, vals in weights:
            if name.startswith("buffer.") and name[7:] in bufs:
                bufs[name[7:]].copy_(torch.from_numpy(np.asarray(vals, dtype=np.float32)).view(bufs[name[7:]].shape))


def model_archive(model, optim: Optional[dict] = None, trainer: Optional[dict] = None, rl: Optional[dict] = None,
                  python: Optional[bytes] = None) -> dict:
    from ..nn.modules import KIND, Sequential
    from .. import fnstore
    if isinstance(model, Sequential):
        layers = [c.nxs_spec() for c in model.layers]
    else:
        layers = [model.nxs_spec()]
    if python is None:
        python = fnstore.payload_for(model)
    return {"layers": layers, "weights": _weights_of(model), "optim": optim, "trainer": trainer, "rl": rl,
            "python": python}


def save_model(model, path: str, **extra) -> None:
    save_archive(path, model_archive(model, **extra))


def load_model(path: str):
    """Rebuilds the network described by the archive and loads its weights."""
    from ..nn.modules import KIND, Sequential, make_one
    from .. import fnstore
    a = load_archive(path)
    if a.get("python"):
        fnstore.restore_payload(a["python"])
    layers = a["layers"]
    if len(layers) == 1 and layers[0]["type"] in (KIND["Graph"], KIND["Sequential"]):
        model = make_one(layers[0])
    elif len(layers) == 1 and layers[0]["type"] == KIND["LanguageModel"]:
        return load_language_model(path)
    else:
        model = Sequential(*[make_one(l) for l in layers])
    _load_weights(model, a["weights"])
    return model


# ----------------------------------------------------------------------------- language models
def save_language_model(model, path: str, optim: Optional[dict] = None) -> None:
    from ..lm.config import to_json
    from ..nn.modules import I32, KIND, STR
    cfg = model.config
    children = []
    for l, blk in enumerate(model.h):
        kids = []
        if blk.moe is not None:
            kids.append({"type": KIND["MoEFFN"], "name": f"h{l}.moe", "attrs": [
                ("experts", I32, cfg.moe_experts), ("top_k", I32, cfg.moe_top_k)], "children": []})
        children.append({"type": KIND["DecoderBlock"], "name": f"h{l}", "attrs": [("layer", I32, l)], "children": kids})
    root = {"type": KIND["LanguageModel"], "name": cfg.name, "attrs": [("config", STR, to_json(cfg)), ("format", I32, 1)],
            "children": children}
    weights = [(n, list(p.shape), p.detach().float().cpu().numpy().reshape(-1)) for n, p in model.named_parameters()]
    save_archive(path, {"layers": [root], "weights": weights, "optim": optim})


def load_language_model(path: str):
    from ..lm.config import from_json
    from ..lm.model import LanguageModel
    from ..nn.modules import KIND
    a = load_archive(path)
    if len(a["layers"]) != 1 or a["layers"][0]["type"] != KIND["LanguageModel"]:
        raise NxsError("archive does not hold a language model")
    attrs = {k: v for k, _, v in a["layers"][0]["attrs"]}
    if attrs.get("format") != 1:
        raise NxsError("unsupported language-model archive format")
    model = LanguageModel(from_json(attrs["config"]))
    named = dict(model.named_parameters())
    seen = set()
    with torch.no_grad():
        for name, dims, vals in a["weights"]:
            if name not in named:
                raise NxsError(f"archive weight '{name}' has no counterpart in the model")
            p = named[name]
            if list(p.shape) != [int(d) for d in dims]:
                raise NxsError(f"weight {name}: shape mismatch")
            p.copy_(torch.from_numpy(np.asarray(vals, dtype=np.float32)).view(p.shape))
            seen.add(name)
    missing = set(named) - seen
    if missing:
        raise NxsError(f"archive lacks weights: {sorted(missing)[:4]}")
    return model


# --------------------------------------------------------------------------- optimizer / trainer
def optim_record(algorithm: str, step: int, lrs: List[float], state_tensors: List[torch.Tensor],
                 scalars: List[float]) -> dict:
    return {"algorithm": algorithm, "step": int(step), "lr": [float(x) for x in lrs],
            "blobs": [t.detach().float().cpu().numpy().tobytes() for t in state_tensors],
            "scalars": [float(s) for s in scalars]}


def trainer_record(epoch: int, global_step: int, loss: float, best: float, stop: bool, metrics: Dict[str, float]) -> dict:
    return {"epoch": int(epoch), "global_step": int(global_step), "loss": float(loss), "best": float(best),
            "stop": bool(stop), "metrics": [(k, float(v)) for k, v in metrics.items()]}
