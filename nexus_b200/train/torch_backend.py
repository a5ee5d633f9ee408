"""`LmBackend` for any ``torch.nn.Module`` language model (``model.loss(tokens)``): CPU FP32 or CUDA
with BF16 autocast; the fused ops dispatch to the sm_100a kernels on CUDA.  AdamW follows the
shared op order (`fused.ops.adamw_multi_tensor`), with per-parameter decay / LR scales, data-parallel
gradient reduction (bucketed, overlapped) and ZeRO/FSDP sharding through the attached engine.

Parity: the CPU module backend of src/train/lm_trainer.cpp:133-760 of the reference.
"""
from __future__ import annotations

import io
import math
from typing import List, Optional

import numpy as np
import torch

from ..fused import ops as F_
from .lm_trainer import AdamW, LmBackend, LmNonFinite, LmParamInfo, LmStepResult


class TorchLmBackend(LmBackend):
    def __init__(self, model: torch.nn.Module, micro_batch: int, seq_len: int, device="cpu", precision="f32",
                 recompute="none", seed: int = 1234):
        self.dev = torch.device(device)
        self.model = model.to(self.dev)
        self.precision = precision if self.dev.type == "cuda" else "f32"
        if self.precision in ("bf16", "f16") and self.dev.type == "cuda":
            self.compute = torch.bfloat16 if self.precision == "bf16" else torch.float16
            self.shadow = None  # parameters stay FP32 masters; narrow copies are made per forward
        else:
            self.compute = torch.float32
        if hasattr(model, "recompute") and recompute != "none":
            model.recompute = "full" if recompute in ("full", "selective") else recompute
        self.B, self.T = micro_batch, seq_len
        self.names = [n for n, _ in self.model.named_parameters()]
        self.params = [p for _, p in self.model.named_parameters()]
        self.m = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.v = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.wd = [1.0 if p.dim() >= 2 else 0.0 for p in self.params]
        self.lrs = [1.0] * len(self.params)
        self.steps = 0
        self._loss = 0.0
        self._micro_losses: List[float] = []
        self._gnorm = float("nan")
        self._skipped = False
        self._pg = None
        self._ddp = None
        self._fsdp = None
        self.h2d_bytes = self.d2h_bytes = 0

    def device(self) -> str: return str(self.dev)
    def micro_batch(self) -> int: return self.B
    def seq_len(self) -> int: return self.T
    def vocab(self) -> int: return getattr(getattr(self.model, "config", None), "vocab_size", 0)
    def reshape(self, micro_batch: int, seq_len: int) -> None: self.B, self.T = micro_batch, seq_len

    def parameters(self) -> List[LmParamInfo]:
        return [LmParamInfo(n, p.numel(), p.dim(), n in ("wte", "wpe") or "embed" in n.lower())
                for n, p in zip(self.names, self.params)]

    def set_param_scales(self, weight_decay, lr) -> None:
        self.wd, self.lrs = [float(x) for x in weight_decay], [float(x) for x in lr]

    def set_rng(self, seed: int, offset: int) -> None:
        if hasattr(self.model, "set_rng"):
            self.model.set_rng(seed, offset)

    def _tokens(self, tokens: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(np.ascontiguousarray(tokens, dtype=np.int32))
        if self.dev.type == "cuda":
            t = t.pin_memory().to(self.dev, non_blocking=True)
            self.h2d_bytes += t.numel() * 4
        return t.long() if self.dev.type == "cpu" else t

    def _loss_of(self, t: torch.Tensor) -> torch.Tensor:
        if self.compute != torch.float32:
            with torch.autocast("cuda", dtype=self.compute):
                return self.model.loss(t)
        return self.model.loss(t)

    def micro_step(self, tokens: np.ndarray, grad_weight: float, index: int, count: int) -> None:
        if index == 0:
            self._loss, self._micro_losses = 0.0, []
        self.model.train()
        t = self._tokens(tokens)
        if self._fsdp is not None:
            loss = self._fsdp.forward_backward(lambda: self._loss_of(t), grad_weight, sync=index == count - 1)
        else:
            loss = self._loss_of(t)
            sync = index == count - 1
            if self._ddp is not None:
                with self._ddp.backward_context(sync):
                    (loss * grad_weight).backward()
            else:
                (loss * grad_weight).backward()
        lv = float(loss.detach())
        self.d2h_bytes += 4
        self._micro_losses.append(lv)
        self._loss += lv * grad_weight

    def optimizer_step(self, optimizer: AdamW, lr: float, clip: float) -> None:
        if self._fsdp is not None:
            self._gnorm, self._skipped = self._fsdp.step(optimizer, lr, clip, self.wd, self.lrs)
            return
        if self._ddp is not None:
            self._ddp.finish()
        idx = [i for i, p in enumerate(self.params) if p.grad is not None]
        grads = [self.params[i].grad for i in idx]
        self.steps += 1
        norm = F_.adamw_multi_tensor([self.params[i].data for i in idx], grads, [self.m[i] for i in idx],
                                     [self.v[i] for i in idx], self.steps, lr, optimizer.beta1, optimizer.beta2,
                                     optimizer.eps, optimizer.weight_decay, clip, [self.wd[i] for i in idx],
                                     [self.lrs[i] for i in idx])
        self._gnorm = norm
        self._skipped = not math.isfinite(norm)
        if self._skipped:
            self.steps -= 1
        for p in self.params:
            p.grad = None

    def finish_step(self) -> LmStepResult:
        if self.dev.type == "cuda":
            torch.cuda.synchronize(self.dev)
        return LmStepResult(loss=self._loss, grad_norm=self._gnorm, skipped=self._skipped,
                            micro_losses=list(self._micro_losses))

    @torch.no_grad()
    def eval_loss(self, tokens: np.ndarray) -> float:
        self.model.eval()
        return float(self._loss_of(self._tokens(tokens)))

    @torch.no_grad()
    def token_losses(self, tokens: np.ndarray) -> np.ndarray:
        self.model.eval()
        t = self._tokens(tokens)
        V = self.vocab() or None
        lg = self.model.logits(t).float()
        lg = lg[..., :V] if V else lg
        tgt = torch.roll(t.long(), -1, dims=1)
        l = torch.nn.functional.cross_entropy(lg.reshape(-1, lg.shape[-1]), tgt.reshape(-1), reduction="none").view(t.shape)
        l[:, -1] = 0.0
        return l.reshape(-1).cpu().numpy()

    def diagnose(self, tokens: np.ndarray) -> LmNonFinite:
        for n, p in zip(self.names, self.params):
            if not torch.isfinite(p).all():
                return LmNonFinite(True, f"param:{n}")
            if p.grad is not None and not torch.isfinite(p.grad).all():
                return LmNonFinite(True, f"grad:{n}")
        found = {}

        def hook(name):
            def f(mod, inp, out):
                o = out[0] if isinstance(out, tuple) else out
                if isinstance(o, torch.Tensor) and "where" not in found and not torch.isfinite(o).all():
                    found["where"] = f"activation:{name}"
            return f
        hs = [m.register_forward_hook(hook(n)) for n, m in self.model.named_modules() if n]
        try:
            with torch.no_grad():
                self._loss_of(self._tokens(tokens))
        finally:
            for h in hs:
                h.remove()
        return LmNonFinite("where" in found, found.get("where", ""))

    def layer_norms(self):
        return [(n, float(p.detach().float().norm()), float(p.grad.float().norm()) if p.grad is not None else 0.0)
                for n, p in zip(self.names, self.params)]

    # ------------------------------------------------------------------------------------ state
    def save_state(self) -> bytes:
        if self._fsdp is not None:
            return self._fsdp.save_state()
        buf = io.BytesIO()
        torch.save({"params": [p.detach().cpu() for p in self.params], "m": [x.cpu() for x in self.m],
                    "v": [x.cpu() for x in self.v], "steps": self.steps}, buf)
        return buf.getvalue()

    def load_state(self, blob: bytes) -> None:
        if self._fsdp is not None:
            return self._fsdp.load_state(blob)
        d = torch.load(io.BytesIO(blob), map_location="cpu")
        with torch.no_grad():
            for p, q in zip(self.params, d["params"]):
                p.copy_(q)
            for a, b in zip(self.m, d["m"]):
                a.copy_(b)
            for a, b in zip(self.v, d["v"]):
                a.copy_(b)
        self.steps = d["steps"]

    def load_resharded_state(self, blobs) -> None:
        if self._fsdp is not None:
            return self._fsdp.load_resharded(blobs)
        self.load_state(blobs[0])

    def state_layout(self) -> str:
        return self._fsdp.layout() if self._fsdp is not None else "replicated"

    def peak_memory_bytes(self) -> int:
        return int(torch.cuda.max_memory_allocated(self.dev)) if self.dev.type == "cuda" else 0

    def reset_peak_memory(self) -> None:
        if self.dev.type == "cuda":
            torch.cuda.reset_peak_memory_stats(self.dev)

    def peak_flops(self) -> float:
        if self.dev.type != "cuda":
            return 0.0
        from .gpt_backend import PEAK_BF16_FLOPS
        return PEAK_BF16_FLOPS.get(torch.cuda.get_device_capability(self.dev)[0], 0.0)

    def flops_per_token(self, seq_len: int) -> float:
        cfg = getattr(self.model, "config", None)
        n = sum(p.numel() for p in self.params)
        if cfg is None:
            return 6.0 * n
        if getattr(cfg, "pos", "") == "learned":
            n -= cfg.max_position * cfg.d_model
        return 6.0 * n + 12.0 * cfg.n_layer * cfg.n_head * cfg.hdim() * seq_len

    # ------------------------------------------------------------------------------ parallelism
    def attach_process_group(self, group, options=None) -> None:
        from ..parallel.ddp import DdpEngine, DdpOptions
        self._pg = group
        self._ddp = DdpEngine(self.params, group, options or DdpOptions())

    def broadcast_parameters(self) -> None:
        if self._pg is not None:
            for p in self.params:
                self._pg.broadcast_tensor(p.data, 0)

    def ddp_stats(self):
        return self._ddp.stats if self._ddp is not None else None

    def attach_fsdp(self, group, options=None) -> None:
        from ..parallel.fsdp import FsdpEngine, FsdpOptions
        self._pg = group
        self._fsdp = FsdpEngine(self.model, group, options or FsdpOptions())

    def fsdp(self):
        return self._fsdp

    def data_parallel_group(self):
        return self._pg
