"""GPT-2 training on one B200 with hand-written sm_100a kernels only (no autograd, no library GEMM).

All parameters live in ONE flat FP32 master buffer with a BF16 shadow copy, one flat FP32 gradient
buffer and flat AdamW moments; the layer loop launches tcgen05 GEMMs with fused epilogues
(bias, bias+GELU with saved pre-activation, dGELU, residual add, beta=1 accumulate), the tcgen05
flash-attention kernels on the packed QKV tensor, fused LayerNorm forward/backward, the in-place
shifted cross-entropy and the multi-tensor AdamW.  A whole step (micro-steps + optimizer) can be
captured into one CUDA graph; the learning rate lives in device memory so replay never bakes it in.

Parity: include/nexus/cuda/gpt.hpp:80-343 and src/cuda/gpt.cpp:664-1526 of the reference
(`GptModel`: 16 flat parameter tensors in the same order, pre-norm blocks, tied head, in-place CE,
FP32 master + narrow shadow, accumulation through beta=1 GEMMs, on-device optimizer state).
Weights are stored [out, in] here (the reference stores [in, out]); archives transpose on the way.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..lm.config import LmConfig, preset
from ..ops import _cuda as K

PARAM_ORDER = ("wte", "wpe", "qkv_w", "attproj_w", "fc_w", "fcproj_w", "ln1_w", "ln1_b", "qkv_b", "attproj_b",
               "ln2_w", "ln2_b", "fc_b", "fcproj_b", "lnf_w", "lnf_b")
DECAY = {"wte", "wpe", "qkv_w", "attproj_w", "fc_w", "fcproj_w"}


@dataclass
class AdamWConfig:
    lr: float = 6e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    grad_clip: float = 1.0


def _align(n: int, a: int = 64) -> int:
    return (n + a - 1) // a * a


class GptModel:
    """Flat-buffer GPT-2 (pre-norm, learned positions, tied head, GELU-tanh) for one CUDA device."""

    RECOMPUTE = ("none", "selective", "full", "every_k")
    OPTIMIZERS = ("adamw", "adamw8bit", "zero_offload")
    MASTERS = ("fp32", "cast_per_forward")

    def __init__(self, config: LmConfig, device="cuda", seed: Optional[int] = None, vocab_pad: int = 128,
                 recompute: str = "none", recompute_every: int = 2, optimizer: str = "adamw", master: str = "fp32",
                 compute_dtype: str = "bf16", offload_grad_dtype: str = "bf16", dynamic_loss_scale: bool = False,
                 loss_scale_init: float = 65536.0, loss_scale_growth_interval: int = 2000, ce_chunk_rows: Optional[int] = None):
        """``recompute`` (activation memory against recomputation in the backward pass; include/nexus/cuda/gpt.hpp:66 of
        the reference): "none" keeps every activation; "selective" keeps the GEMM outputs (qkv, attention output,
        MLP pre-activation) and recomputes the norm outputs and the GELU output; "full" keeps only the residual stream
        and re-runs the layer's forward; "every_k" treats layers with ``l % recompute_every == 0`` as "full".
        ``optimizer``: "adamw" (FP32 moments on the device), "adamw8bit" (block-wise 8-bit moments for the matrices,
        FP32 moments for norms and biases), "zero_offload" (FP32 master and moments in pinned host memory, gradients
        copied to the host, AdamW on the CPU, BF16 weights copied back).  ``master``: "fp32" (BF16 working copy written
        by the optimizer kernel) or "cast_per_forward" (the working copy is re-cast from the FP32 parameters at the
        start of every forward pass).  Anything else the reference's model offers (FP16 with a loss scale, BF16-only
        weights with stochastic rounding, the 8-bit optimizer applied layer by layer inside the backward pass) is
        refused here with an error rather than ignored.
        ``ce_chunk_rows`` (`GptConfig::ce_chunk_rows` of include/nexus/cuda/gpt.hpp; default from
        ``NEXUS_B200_CE_CHUNK_ROWS``, else 0): 0 keeps one [B*T, V] logits
        buffer; a positive value runs the LM head, the fused cross-entropy and the head's two backward GEMMs over
        groups of whole sequences of at most that many rows, so that only one group's logits exist at a time."""
        if recompute not in self.RECOMPUTE:
            raise ValueError(f"GptModel: recompute must be one of {self.RECOMPUTE}, got {recompute!r}")
        if optimizer not in self.OPTIMIZERS:
            raise ValueError(f"GptModel: optimizer must be one of {self.OPTIMIZERS}, got {optimizer!r} "
                             "(the layer-wise fused 8-bit optimizer is not implemented)")
        if master not in self.MASTERS:
            raise ValueError(f"GptModel: master must be one of {self.MASTERS}, got {master!r} "
                             "(BF16-only weights with stochastic rounding are not implemented)")
        if compute_dtype != "bf16":
            raise ValueError("GptModel computes in BF16; FP16 with a dynamic loss scale is not implemented "
                             "(the attention kernels take BF16 only)")
        if recompute == "every_k" and recompute_every < 1:
            raise ValueError("GptModel: recompute_every must be >= 1")
        if optimizer == "zero_offload" and master != "fp32":
            raise ValueError("GptModel: zero_offload keeps the FP32 master on the host (master must be 'fp32')")
        if ce_chunk_rows is None:
            ce_chunk_rows = int(os.environ.get("NEXUS_B200_CE_CHUNK_ROWS", "0"))
        if ce_chunk_rows < 0:
            raise ValueError("GptModel: ce_chunk_rows must be >= 0")
        self.ce_chunk_rows = int(ce_chunk_rows)
        self.recompute, self.recompute_every = recompute, recompute_every
        self.optimizer_kind, self.master_mode = optimizer, master
        self.offload_grad_dtype = torch.bfloat16 if offload_grad_dtype == "bf16" else torch.float32
        if config.norm != "layernorm" or config.mlp != "gelu" or config.pos != "learned" or not config.bias:
            raise ValueError("GptModel implements the GPT-2 architecture (LayerNorm, GELU, learned positions, bias)")
        if not config.tie_embeddings:
            raise ValueError("GptModel ties the LM head to the token embedding")
        if config.hdim() not in (64, 128):
            raise ValueError("head_dim must be 64 or 128")
        self.config = config
        self.device = torch.device(device)
        self.L, self.C, self.H = config.n_layer, config.d_model, config.n_head
        self.V = config.vocab_size
        self.Vp = _align(config.vocab_size, vocab_pad)
        self.P = config.max_position
        self.F = config.d_ff
        L, C, F = self.L, self.C, self.F
        shapes = {
            "wte": (self.Vp, C), "wpe": (self.P, C),
            "qkv_w": (L, 3 * C, C), "attproj_w": (L, C, C), "fc_w": (L, F, C), "fcproj_w": (L, C, F),
            "ln1_w": (L, C), "ln1_b": (L, C), "qkv_b": (L, 3 * C), "attproj_b": (L, C),
            "ln2_w": (L, C), "ln2_b": (L, C), "fc_b": (L, F), "fcproj_b": (L, C),
            "lnf_w": (C,), "lnf_b": (C,),
        }
        self.shapes = shapes
        self.offsets: Dict[str, int] = {}
        off = 0
        for name in PARAM_ORDER:
            off = _align(off)
            self.offsets[name] = off
            off += math.prod(shapes[name])
        self.num_params = _align(off)
        dev = self.device
        self.params = torch.zeros(self.num_params, dtype=torch.float32, device=dev)     # FP32 master
        self.params_lp = torch.zeros(self.num_params, dtype=torch.bfloat16, device=dev)  # BF16 shadow
        self.grads = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
        self._tail = self.offsets["ln1_w"]      # matrices (and embeddings) before, 1-D parameters after
        self._q8 = None
        self._host = None
        if optimizer == "adamw":
            self.m = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
            self.v = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
        elif optimizer == "adamw8bit":
            from ..ops import _lowp
            self._q8 = _lowp.AdamW8bitState(self._tail, dev)                 # 8-bit moments of the matrices
            self.m = torch.zeros(self.num_params - self._tail, dtype=torch.float32, device=dev)   # FP32 for the 1-D tail
            self.v = torch.zeros(self.num_params - self._tail, dtype=torch.float32, device=dev)
        else:  # zero_offload: master, moments and the gradient landing buffer live in pinned host memory
            self.m = self.v = None
            self._host = {"p": torch.zeros(self.num_params, dtype=torch.float32).pin_memory(),
                          "m": torch.zeros(self.num_params, dtype=torch.float32).pin_memory(),
                          "v": torch.zeros(self.num_params, dtype=torch.float32).pin_memory(),
                          "g": torch.zeros(self.num_params, dtype=self.offload_grad_dtype).pin_memory(),
                          "lp": torch.zeros(self.num_params, dtype=torch.bfloat16).pin_memory()}
            self.last_cpu_update_ms = 0.0
        self.p = {n: self._view(self.params, n) for n in PARAM_ORDER}
        self.w = {n: self._view(self.params_lp, n) for n in PARAM_ORDER}
        self.g = {n: self._view(self.grads, n) for n in PARAM_ORDER}
        self.opt_state = K.opt_state_tensor(dev)
        off = K.OptState.loss_scale.offset             # the loss-scale field, as the 1-element tensor the CE kernel reads
        self._loss_scale_dev = self.opt_state[off: off + 4].view(torch.float32)
        self._opt_host = torch.zeros(self.opt_state.numel(), dtype=torch.uint8).pin_memory()
        self._lr_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self.chunks = K.make_chunks(
            [(self.offsets[n], math.prod(shapes[n]), 1.0 if n in DECAY else 0.0, 1.0) for n in PARAM_ORDER],
            device=dev)
        self._tail_chunks = K.make_chunks(
            [(self.offsets[n] - self._tail, math.prod(shapes[n]), 0.0, 1.0) for n in PARAM_ORDER
             if self.offsets[n] >= self._tail], device=dev)
        self.loss_buf = torch.zeros(1, dtype=torch.float32, device=dev)
        self._acts = None
        self._acts_key = None
        self.step_count = 0
        # Dynamic loss scale (include/nexus/cuda/gpt.hpp:30,91 of the reference): the scale lives in the device-resident
        # optimizer state; the loss gradient is multiplied by it on the device, the norm kernel unscales and flags
        # non-finite gradients, AdamW skips such a step, and one tiny kernel halves / doubles the scale.  No host read.
        self.dynamic_loss_scale = bool(dynamic_loss_scale)
        self.loss_scale_init = float(loss_scale_init)
        self.loss_scale_growth_interval = int(loss_scale_growth_interval)
        if self.dynamic_loss_scale and optimizer != "adamw":
            raise ValueError("dynamic_loss_scale is implemented for optimizer='adamw'")
        self.backward_hook = None     # callable(stage): see set_backward_hook
        # the bias-gradient column sums of fc / qkv are bandwidth-bound side work: they run on a second stream under the
        # two GEMMs that follow them (NEXUS_B200_OVERLAP_COLSUM=0 keeps them in line)
        self.overlap_colsum = os.environ.get("NEXUS_B200_OVERLAP_COLSUM", "1") != "0" and torch.device(device).type == "cuda"
        self._side = None
        self.deterministic_embedding = False
        self.init_weights(config.seed if seed is None else seed)

    # ---------------------------------------------------------------------------------------- setup
    def _view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        n = math.prod(self.shapes[name])
        return flat[self.offsets[name]: self.offsets[name] + n].view(self.shapes[name])

    def init_weights(self, seed: int) -> None:
        """GPT-2 init: N(0, 0.02), residual projections 0.02/sqrt(2L), LayerNorm 1/0, biases 0."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        std = self.config.init_std
        self.params.zero_()
        for name in ("wte", "wpe", "qkv_w", "fc_w", "attproj_w", "fcproj_w"):
            t = self.p[name]
            s = std / math.sqrt(2 * self.L) if name in ("attproj_w", "fcproj_w") else std
            t.copy_(torch.randn(t.shape, generator=g, dtype=torch.float32) * s)
        self.p["wte"][self.V:].zero_()  # padded vocabulary rows stay zero (their gradient is zero)
        for name in ("ln1_w", "ln2_w", "lnf_w"):
            self.p[name].fill_(1.0)
        if self._host is not None:
            self._host["p"].copy_(self.params)
        self.refresh_shadow()

    def rebind_buffers(self, params_lp: Optional[torch.Tensor] = None, grads: Optional[torch.Tensor] = None) -> None:
        """Re-points the BF16 shadow and/or the gradient buffer at caller-provided storage (e.g. symmetric
        memory that peers can reach) and rebuilds the per-tensor views."""
        if params_lp is not None:
            self.params_lp = params_lp
            self.w = {n: self._view(self.params_lp, n) for n in PARAM_ORDER}
        if grads is not None:
            self.grads = grads
            self.g = {n: self._view(self.grads, n) for n in PARAM_ORDER}

    def fp32_tail_offset(self) -> int:
        """Offset of the first 1-D parameter (norm scales and biases follow the matrices in the flat
        buffer); everything from here on is read by the kernels in FP32."""
        return self.offsets["ln1_w"]

    def rebind_fp32_tail(self, tail: torch.Tensor) -> None:
        """Re-points the FP32 views of the 1-D parameters at ``tail`` (same layout as
        ``params[fp32_tail_offset():]``), e.g. symmetric memory filled by a sharded optimizer."""
        base = self.fp32_tail_offset()
        for n in PARAM_ORDER:
            if self.offsets[n] >= base:
                o, cnt = self.offsets[n] - base, math.prod(self.shapes[n])
                self.p[n] = tail[o: o + cnt].view(self.shapes[n])

    def refresh_shadow(self) -> None:
        self.params_lp.copy_(self.params)

    def named_parameters(self):
        return [(n, self.p[n]) for n in PARAM_ORDER]

    def count_parameters(self) -> int:
        return sum(math.prod(self.shapes[n]) for n in PARAM_ORDER) - (self.Vp - self.V) * self.C

    # ------------------------------------------------------------------------------------ buffers
    _LAYER_KEYS = ("ln1", "qkv", "atty", "lse", "ln2", "fch_pre", "fch")
    _KEPT = {"none": set(_LAYER_KEYS), "selective": {"qkv", "atty", "lse", "fch_pre"}, "full": set()}

    def layer_mode(self, l: int) -> str:
        """How layer ``l`` treats its activations: "none" (kept), "selective" or "full" (recomputed)."""
        if self.recompute == "every_k":
            return "full" if l % self.recompute_every == 0 else "none"
        return self.recompute

    def _plan_slots(self):
        """Per activation kind: the buffer index of every layer.  Kept activations get an index of their own; the
        ones a layer recomputes share one scratch index."""
        slots, counts = {}, {}
        for key in self._LAYER_KEYS:
            idx, nxt = [], 0
            for l in range(self.L):
                if key in self._KEPT[self.layer_mode(l)]:
                    idx.append(nxt)
                    nxt += 1
                else:
                    idx.append(-1)
            shared = nxt if any(i < 0 for i in idx) else -1
            slots[key] = [shared if i < 0 else i for i in idx]
            counts[key] = nxt + (1 if shared >= 0 else 0)
        return slots, counts

    def activation_bytes(self) -> int:
        a = self._acts or {}
        return sum(t.numel() * t.element_size() for t in a.values() if isinstance(t, torch.Tensor))

    def _alloc_acts(self, B: int, T: int):
        key = (B, T)
        if self._acts_key == key:
            return self._acts
        dev, L, C, F, H = self.device, self.L, self.C, self.F, self.H
        N = B * T
        bf, f32 = torch.bfloat16, torch.float32
        self._slots, cnt = self._plan_slots()
        a = {
            "res": torch.empty((2 * L + 1, N, C), dtype=f32, device=dev),   # residual stream checkpoints
            "ln1": torch.empty((cnt["ln1"], N, C), dtype=bf, device=dev),
            "ln1_mean": torch.empty((L, N), dtype=f32, device=dev), "ln1_rstd": torch.empty((L, N), dtype=f32, device=dev),
            "qkv": torch.empty((cnt["qkv"], B, T, 3, H, C // H), dtype=bf, device=dev),
            "atty": torch.empty((cnt["atty"], B, T, H, C // H), dtype=bf, device=dev),
            "lse": torch.empty((cnt["lse"], B, H, T), dtype=f32, device=dev),
            "ln2": torch.empty((cnt["ln2"], N, C), dtype=bf, device=dev),
            "ln2_mean": torch.empty((L, N), dtype=f32, device=dev), "ln2_rstd": torch.empty((L, N), dtype=f32, device=dev),
            "fch_pre": torch.empty((cnt["fch_pre"], N, F), dtype=bf, device=dev),
            "fch": torch.empty((cnt["fch"], N, F), dtype=bf, device=dev),
            "lnf": torch.empty((N, C), dtype=bf, device=dev),
            "lnf_mean": torch.empty(N, dtype=f32, device=dev), "lnf_rstd": torch.empty(N, dtype=f32, device=dev),
            "logits": torch.empty((self._head_group(B, T) * T, self.Vp), dtype=bf, device=dev),
            # backward scratch (reused by every layer)
            "dres_a": torch.empty((N, C), dtype=f32, device=dev), "dres_b": torch.empty((N, C), dtype=f32, device=dev),
            "dres_lp": torch.empty((N, C), dtype=bf, device=dev),
            "dlnf": torch.empty((N, C), dtype=bf, device=dev),
            "dfch": torch.empty((N, F), dtype=bf, device=dev),
            "dln": torch.empty((N, C), dtype=bf, device=dev),
            "datty": torch.empty((B, T, H, C // H), dtype=bf, device=dev),
            "dqkv": torch.empty((B, T, 3, H, C // H), dtype=bf, device=dev),
        }
        self._acts, self._acts_key = a, key
        return a

    def _head_group(self, B: int, T: int) -> int:
        """Sequences per pass of the LM head and the loss: all of them unless ``ce_chunk_rows`` asks for less; always a
        divisor of B, so that every group has the same number of targets and the mean of the group means is the mean."""
        if self.ce_chunk_rows <= 0 or self.ce_chunk_rows >= B * T:
            return B
        k = max(1, self.ce_chunk_rows // T)
        while B % k:
            k -= 1
        return k

    # ------------------------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor, *, want_logits: bool = True):
        """tokens [B, T] int32 on the device.  Fills the activation buffers; returns logits [B*T, Vp]."""
        B, T = tokens.shape
        a = self._alloc_acts(B, T)
        w, L, C = self.w, self.L, self.C
        N = B * T
        if self.master_mode == "cast_per_forward":
            self.refresh_shadow()
        res = a["res"]
        _embedding_into(res[0], tokens, w["wte"], w["wpe"], T)
        for l in range(L):
            self._layer_forward(a, l, B, T, output=True)
        _norm_into(a["lnf"], a["lnf_mean"], a["lnf_rstd"], res[2 * L], self.p["lnf_w"], self.p["lnf_b"])
        if not want_logits:
            return None
        if a["logits"].shape[0] != N:     # the training buffer holds one group only: whole logits on request
            full = a.get("logits_full")
            if full is None:
                full = a["logits_full"] = torch.empty((N, self.Vp), dtype=torch.bfloat16, device=self.device)
            K.gemm(a["lnf"], w["wte"], out=full)
            return full
        K.gemm(a["lnf"], w["wte"], out=a["logits"])
        return a["logits"]

    STAGE_HEAD, STAGE_EMBEDDING = -1, -2

    def set_backward_hook(self, hook) -> None:
        """``hook(stage)`` is called on the host while the backward pass is being enqueued, right after the kernels
        that complete a stage's gradients: STAGE_HEAD (final norm), then layer L-1 ... 0 (every per-layer slice of
        that layer), then STAGE_EMBEDDING (wte, wpe).  A data-parallel backend records an event there and starts
        reducing the stage's gradients on another stream.  Parity: GptModel::set_backward_hook of the reference
        (include/nexus/cuda/gpt.hpp, kStageHead / kStageEmbedding)."""
        self.backward_hook = hook

    def layer_grad_ranges(self, l0: int, l1: int):
        """(offset, count) of the gradient slices of layers [l0, l1) in the flat buffer, one per per-layer tensor."""
        out = []
        for name in PARAM_ORDER:
            shp = self.shapes[name]
            if name in ("wte", "wpe", "lnf_w", "lnf_b"):
                continue
            per = math.prod(shp[1:])
            out.append((self.offsets[name] + l0 * per, (l1 - l0) * per))
        return out

    def _layer_forward(self, a, l: int, B: int, T: int, output: bool, only: Optional[set] = None) -> None:
        """Forward of layer ``l`` into its activation buffers.  ``output``: also form the residual outputs (the
        forward pass); the recomputation of the backward pass only refills the activations named in ``only``."""
        w, C = self.w, self.C
        N = B * T
        S = self._slots
        res = a["res"]
        x_in, x_mid, x_out = res[2 * l], res[2 * l + 1], res[2 * l + 2]
        want = (lambda k: True) if only is None else (lambda k: k in only)
        ln1, qkv, atty, lse = a["ln1"][S["ln1"][l]], a["qkv"][S["qkv"][l]], a["atty"][S["atty"][l]], a["lse"][S["lse"][l]]
        ln2, fch_pre, fch = a["ln2"][S["ln2"][l]], a["fch_pre"][S["fch_pre"][l]], a["fch"][S["fch"][l]]
        if want("ln1"):
            _norm_into(ln1, a["ln1_mean"][l], a["ln1_rstd"][l], x_in, self.p["ln1_w"][l], self.p["ln1_b"][l])
        if want("qkv"):
            K.gemm(ln1, w["qkv_w"][l], bias=w["qkv_b"][l], out=qkv.view(N, 3 * C))
        if want("atty"):
            _attn_fwd_into(atty, lse, qkv)
        if output:
            K.gemm(atty.view(N, C), w["attproj_w"][l], bias=w["attproj_b"][l], residual=x_in, out=x_mid)
        if want("ln2"):
            _norm_into(ln2, a["ln2_mean"][l], a["ln2_rstd"][l], x_mid, self.p["ln2_w"][l], self.p["ln2_b"][l])
        if want("fch_pre"):
            K.gemm(ln2, w["fc_w"][l], bias=w["fc_b"][l], act="gelu", aux_out=fch_pre, out=fch)
        elif want("fch"):   # the pre-activation was kept: only the GELU is redone
            K._check(K.lib().nx_gelu(K._p(fch_pre), K._p(None), K._p(fch), _C.c_int(K._DT[fch.dtype]),
                                     _C.c_int64(fch.numel()), K._stream()), "nx_gelu")
        if output:
            K.gemm(fch, w["fcproj_w"][l], bias=w["fcproj_b"][l], residual=x_mid, out=x_out)

    # --------------------------------------------------------------------------- forward + backward
    def forward_backward(self, tokens: torch.Tensor, grad_scale: float = 1.0, accumulate_loss: bool = False,
                         loss_weight: float = 1.0, smoothing: float = 0.0, z_loss: float = 0.0) -> torch.Tensor:
        """One micro-step.  Gradients accumulate into ``self.grads`` (zeroed by the optimizer step).
        Returns the device tensor holding the (weighted, accumulated) loss."""
        B, T = tokens.shape
        N = B * T
        a = self._alloc_acts(B, T)
        w, g, L, C, F = self.w, self.g, self.L, self.C, self.F
        self.forward(tokens, want_logits=False)
        res = a["res"]
        # head, per group of whole sequences (one group unless ce_chunk_rows is set):
        # logits = lnf @ wte^T ; CE turns them into dlogits ; dlnf = dlogits @ wte ; dwte += dlogits^T @ lnf
        k = self._head_group(B, T)
        groups, rows = B // k, k * T
        dlogits = a["logits"]
        for c in range(groups):
            r0 = c * rows
            lnf_c = a["lnf"][r0:r0 + rows]
            K.gemm(lnf_c, w["wte"], out=dlogits)
            K.cross_entropy_shifted(dlogits, tokens[c * k:(c + 1) * k], vocab=self.V, smoothing=smoothing, z_loss=z_loss,
                                    grad_scale=grad_scale / groups, loss_out=self.loss_buf,
                                    loss_weight=loss_weight / groups, accumulate_loss=accumulate_loss or c > 0, seq_len=T,
                                    grad_scale_dev=self._loss_scale_dev if self.dynamic_loss_scale else None)
            K.gemm(dlogits, w["wte"], b_mn=True, out=a["dlnf"][r0:r0 + rows])
            K.gemm(dlogits, lnf_c, a_mn=True, b_mn=True, out=g["wte"], accumulate=True)
        dres, dres_other, dres_lp = a["dres_a"], a["dres_b"], a["dres_lp"]
        # each norm backward also sums the columns of its BF16 dx: the bias gradient of the projection that follows
        K.norm_bwd(a["dlnf"], res[2 * L], self.p["lnf_w"], a["lnf_mean"], a["lnf_rstd"], dx=dres, dx_lp=dres_lp,
                   dgamma=g["lnf_w"], dbeta=g["lnf_b"], accumulate_params=True, dx_colsum=g["fcproj_b"][L - 1])
        hook = self.backward_hook
        if hook is not None:
            hook(self.STAGE_HEAD)
        S = self._slots
        side = None
        if self.overlap_colsum:
            if self._side is None:
                self._side = torch.cuda.Stream(device=self.device)
                self._side_evt = [torch.cuda.Event() for _ in range(4)]   # fork / join, for dfch and dqkv
            side = self._side
        main = torch.cuda.current_stream() if side is not None else None
        pending = [False, False]      # a column sum of dfch / dqkv is still running on the side stream

        def side_colsum(which, src, dst):
            """Column sums of ``src`` into ``dst`` on the side stream, ordered after what the main stream has enqueued."""
            fork = self._side_evt[2 * which]
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                K.colsum(src, out=dst, accumulate=True)
                self._side_evt[2 * which + 1].record(side)
            pending[which] = True

        def side_join(which):
            """The main stream waits for the side stream's last use of dfch / dqkv (before the buffer is overwritten)."""
            if side is not None and pending[which]:
                main.wait_event(self._side_evt[2 * which + 1])
                pending[which] = False
        for l in range(L - 1, -1, -1):
            x_in, x_mid = res[2 * l], res[2 * l + 1]
            mode = self.layer_mode(l)
            if mode != "none":   # refill what this layer did not keep (the residual stream is always kept)
                self._layer_forward(a, l, B, T, output=False, only=set(self._LAYER_KEYS) - self._KEPT[mode])
            ln1_l, qkv_l, atty_l, lse_l = (a[k][S[k][l]] for k in ("ln1", "qkv", "atty", "lse"))
            ln2_l, fch_pre_l, fch_l = (a[k][S[k][l]] for k in ("ln2", "fch_pre", "fch"))
            # ---- MLP
            side_join(0)
            K.gemm(dres_lp, w["fcproj_w"][l], b_mn=True, act="dgelu", aux_in=fch_pre_l, out=a["dfch"])
            K.gemm(dres_lp, fch_l, a_mn=True, b_mn=True, out=g["fcproj_w"][l], accumulate=True, split_k=0)
            K.gemm(a["dfch"], w["fc_w"][l], b_mn=True, out=a["dln"])
            K.gemm(a["dfch"], ln2_l, a_mn=True, b_mn=True, out=g["fc_w"][l], accumulate=True, split_k=0)
            if side is not None:
                side_colsum(0, a["dfch"], g["fc_b"][l])
            else:
                K.colsum(a["dfch"], out=g["fc_b"][l], accumulate=True)
            K.norm_bwd(a["dln"], x_mid, self.p["ln2_w"][l], a["ln2_mean"][l], a["ln2_rstd"][l], add=dres,
                       dx=dres_other, dx_lp=dres_lp, dgamma=g["ln2_w"][l], dbeta=g["ln2_b"][l], accumulate_params=True,
                       dx_colsum=g["attproj_b"][l])
            dres, dres_other = dres_other, dres
            # ---- attention
            K.gemm(dres_lp, w["attproj_w"][l], b_mn=True, out=a["datty"].view(N, C))
            K.gemm(dres_lp, atty_l.view(N, C), a_mn=True, b_mn=True, out=g["attproj_w"][l], accumulate=True,
                   split_k=0)
            qkv, dqkv = qkv_l, a["dqkv"]
            side_join(1)
            K.attention_bwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], atty_l, lse_l, a["datty"],
                            causal=True, dq=dqkv[:, :, 0], dk=dqkv[:, :, 1], dv=dqkv[:, :, 2])
            dq2 = dqkv.view(N, 3 * C)
            K.gemm(dq2, w["qkv_w"][l], b_mn=True, out=a["dln"])
            K.gemm(dq2, ln1_l, a_mn=True, b_mn=True, out=g["qkv_w"][l], accumulate=True, split_k=0)
            if side is not None:
                side_colsum(1, dq2, g["qkv_b"][l])
            else:
                K.colsum(dq2, out=g["qkv_b"][l], accumulate=True)
            K.norm_bwd(a["dln"], x_in, self.p["ln1_w"][l], a["ln1_mean"][l], a["ln1_rstd"][l], add=dres,
                       dx=dres_other, dx_lp=dres_lp, dgamma=g["ln1_w"][l], dbeta=g["ln1_b"][l], accumulate_params=True,
                       dx_colsum=g["fcproj_b"][l - 1] if l > 0 else None)
            dres, dres_other = dres_other, dres
            if hook is not None:
                side_join(0)          # the stage's bias gradients are complete before the hook looks at them
                side_join(1)
                hook(l)
        side_join(0)
        side_join(1)
        K.embedding_bwd(tokens, dres.view(B, T, C), g["wte"], g["wpe"][:T], B, T,
                        deterministic=self.deterministic_embedding)
        if hook is not None:
            hook(self.STAGE_EMBEDDING)
        return self.loss_buf

    # ---------------------------------------------------------------------------------- optimizer
    def set_optimizer(self, cfg: AdamWConfig, lr: Optional[float] = None, loss_scale: Optional[float] = None) -> None:
        """Writes hyper-parameters into the device-resident optimizer state (keeps step counters and, under
        ``dynamic_loss_scale``, the current scale)."""
        cur = K.unpack_opt_state(bytes(self.opt_state.cpu().numpy().tobytes()))
        if loss_scale is None:
            if not self.dynamic_loss_scale:
                loss_scale = 1.0
            else:
                loss_scale = cur.loss_scale if getattr(self, "_loss_scale_set", False) else self.loss_scale_init
        self._loss_scale_set = True
        raw = K.pack_opt_state(lr=cfg.lr if lr is None else lr, weight_decay=cfg.weight_decay, beta1=cfg.beta1,
                               beta2=cfg.beta2, eps=cfg.eps, max_grad_norm=cfg.grad_clip, loss_scale=loss_scale,
                               step=cur.step, skipped=cur.skipped, good_steps=cur.good_steps,
                               inv_bias1=cur.inv_bias1, inv_bias2=cur.inv_bias2)
        self._opt_host.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
        self.opt_state.copy_(self._opt_host, non_blocking=True)

    def set_lr(self, lr: float) -> None:
        """Updates only the learning-rate field on the device (4-byte async copy; graph friendly)."""
        off = K.OptState.lr.offset
        self._lr_host[0] = lr
        self.opt_state[off: off + 4].view(torch.float32).copy_(self._lr_host, non_blocking=True)

    def optimizer_step(self) -> None:
        """Global-norm clip + AdamW on the flat buffers, refreshes the BF16 shadow, zeroes the gradients."""
        K.grad_norm(self.grads, self.opt_state)
        shadow = None if self.master_mode == "cast_per_forward" else self.params_lp
        if self.optimizer_kind == "adamw":
            K.adamw(self.params, self.grads, self.m, self.v, shadow, self.chunks, self.opt_state, zero_grad=True)
            if self.dynamic_loss_scale:
                K.loss_scale_update(self.opt_state, interval=self.loss_scale_growth_interval)
        elif self.optimizer_kind == "adamw8bit":
            from ..ops import _lowp
            t = self._tail
            _lowp.adamw8(self.params[:t], shadow[:t] if shadow is not None else None, self.grads[:t], self._q8,
                         self.opt_state, wd_scale=1.0, lr_scale=1.0, zero_grad=True)
            K.adamw(self.params[t:], self.grads[t:], self.m, self.v, shadow[t:] if shadow is not None else None,
                    self._tail_chunks, self.opt_state, zero_grad=True)
        else:
            self._offload_step()
        self.step_count += 1

    def _offload_step(self) -> None:
        """ZeRO-Offload: gradients -> pinned host memory (BF16 by default), AdamW on the CPU with the device's clip
        factor and bias corrections, BF16 weights -> device.  One synchronisation per step."""
        import time
        import numpy as np
        from .. import _native
        h = self._host
        h["g"].copy_(self.grads.to(h["g"].dtype), non_blocking=True)
        st_host = self.opt_state.cpu()          # synchronises: the gradient copy and the norm are complete
        st = K.unpack_opt_state(bytes(st_host.numpy().tobytes()))
        self.grads.zero_()
        if st.found_inf:
            return
        t0 = time.perf_counter()
        g32 = h["g"].float().numpy() if h["g"].dtype != torch.float32 else h["g"].numpy()
        pn, mn, vn = h["p"].numpy(), h["m"].numpy(), h["v"].numpy()
        for name in PARAM_ORDER:
            lo = self.offsets[name]
            hi = lo + math.prod(self.shapes[name])
            wd = st.weight_decay if name in DECAY else 0.0
            _native.adamw_range(pn[lo:hi], np.ascontiguousarray(g32[lo:hi]), mn[lo:hi], vn[lo:hi], st.lr, wd, st.beta1,
                                st.beta2, st.eps, st.inv_bias1, st.inv_bias2, st.clip_coef)
        h["lp"].copy_(h["p"])
        self.last_cpu_update_ms = (time.perf_counter() - t0) * 1e3
        self.params_lp.copy_(h["lp"], non_blocking=True)
        self.params[self._tail:].copy_(h["p"][self._tail:], non_blocking=True)   # the kernels read norms / biases in FP32

    def optimizer_tensors(self) -> Dict[str, torch.Tensor]:
        """Every tensor that, with the device optimizer state, makes up the training state (host copies)."""
        if self.optimizer_kind == "adamw":
            return {"params": self.params.cpu(), "m": self.m.cpu(), "v": self.v.cpu()}
        if self.optimizer_kind == "adamw8bit":
            q = self._q8
            return {"params": self.params.cpu(), "m_tail": self.m.cpu(), "v_tail": self.v.cpu(), "qm": q.qm.cpu(),
                    "qv": q.qv.cpu(), "absmax_m": q.absmax_m.cpu(), "absmax_v": q.absmax_v.cpu()}
        h = self._host
        return {"params": h["p"].clone(), "m": h["m"].clone(), "v": h["v"].clone()}

    def load_optimizer_tensors(self, d: Dict[str, torch.Tensor]) -> None:
        if self.optimizer_kind == "adamw":
            self.params.copy_(d["params"]); self.m.copy_(d["m"]); self.v.copy_(d["v"])
        elif self.optimizer_kind == "adamw8bit":
            q = self._q8
            self.params.copy_(d["params"]); self.m.copy_(d["m_tail"]); self.v.copy_(d["v_tail"])
            q.qm.copy_(d["qm"]); q.qv.copy_(d["qv"]); q.absmax_m.copy_(d["absmax_m"]); q.absmax_v.copy_(d["absmax_v"])
        else:
            h = self._host
            h["p"].copy_(d["params"]); h["m"].copy_(d["m"]); h["v"].copy_(d["v"])
            self.params.copy_(h["p"])
        self.refresh_shadow()

    def optimizer_state_bytes(self) -> Tuple[int, int]:
        """(device bytes, host bytes) of master weights + moments (the working copy and gradients excluded)."""
        if self.optimizer_kind == "adamw":
            return 12 * self.num_params, 0
        if self.optimizer_kind == "adamw8bit":
            return 4 * self.num_params + self._q8.nbytes() + 8 * (self.num_params - self._tail), 0
        return 4 * self.num_params, 12 * self.num_params + self._host["g"].numel() * self._host["g"].element_size()

    def read_opt_state(self) -> "K.OptState":
        return K.unpack_opt_state(bytes(self.opt_state.cpu().numpy().tobytes()))

    # ---------------------------------------------------------------------------------- utilities
    def loss(self, tokens: torch.Tensor) -> float:
        self.forward(tokens, want_logits=False)
        B, T = tokens.shape
        a = self._acts
        k = self._head_group(B, T)
        groups, rows = B // k, k * T
        out = torch.zeros(1, dtype=torch.float32, device=self.device)
        for c in range(groups):
            K.gemm(a["lnf"][c * rows:(c + 1) * rows], self.w["wte"], out=a["logits"])
            K.cross_entropy_shifted(a["logits"], tokens[c * k:(c + 1) * k], vocab=self.V, write_grad=False, loss_out=out,
                                    loss_weight=1.0 / groups, accumulate_loss=c > 0, seq_len=T)
        return float(out.item())

    def state_dict(self) -> Dict[str, torch.Tensor]:
        sd = {n: self.p[n].detach().clone() for n in PARAM_ORDER}
        sd["wte"] = sd["wte"][: self.V].clone()
        return sd

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for n in PARAM_ORDER:
            t = sd[n].to(self.device, torch.float32)
            if n == "wte":
                self.p[n][: self.V].copy_(t[: self.V])
            else:
                self.p[n].copy_(t)
        self.refresh_shadow()

    def flops_per_token(self, T: int) -> float:
        """MFU numerator of the reference: 6 * N_nopos + 12 * L * H * d_h * T."""
        n_nopos = self.count_parameters() - self.P * self.C
        return 6.0 * n_nopos + 12.0 * self.L * self.H * (self.C // self.H) * T


# ---- thin "write into a preallocated buffer" helpers around the kernel bindings -------------------
import ctypes as _C  # noqa: E402


def _embedding_into(out, tokens, wte, wpe, T):
    L = K.lib()
    K._check(L.nx_embedding_pos_fwd(K._p(tokens), K._p(None), K._p(wte), K._p(wpe), _C.c_int(K._DT[wte.dtype]),
                                    K._p(out), _C.c_int(K._DT[out.dtype]), _C.c_int64(tokens.numel()), _C.c_int(T),
                                    _C.c_int(wte.shape[1]), K._stream()), "nx_embedding_pos_fwd")


def _norm_into(y, mean, rstd, x, gamma, beta, eps=1e-5, rms=False):
    rows, cols = x.shape[0], x.shape[1]
    K._check(K.lib().nx_norm_fwd(_C.c_int(int(rms)), K._p(x), _C.c_int(K._DT[x.dtype]), K._p(None), K._p(None),
                                 K._p(gamma), K._p(beta), _C.c_int(K._DT[gamma.dtype]), K._p(y),
                                 _C.c_int(K._DT[y.dtype]), K._p(mean), K._p(rstd), _C.c_int(rows), _C.c_int(cols),
                                 _C.c_float(eps), K._stream()), "nx_norm_fwd")


def _attn_fwd_into(o, lse, qkv, causal=True):
    B, T, _, H, D = qkv.shape
    a = K.AttnArgs()
    a.q, a.k, a.v, a.o = K._view(qkv[:, :, 0]), K._view(qkv[:, :, 1]), K._view(qkv[:, :, 2]), K._view(o)
    a.lse = lse.data_ptr()
    a.status = K.status_word(qkv.device).data_ptr()
    a.batch, a.heads, a.kv_heads, a.tq, a.tk, a.head_dim = B, H, H, T, T, D
    a.causal, a.window, a.scale = int(causal), 0, D ** -0.5
    K._check(K.lib().nx_attention_fwd(_C.byref(a), K._stream()), "nx_attention_fwd")
