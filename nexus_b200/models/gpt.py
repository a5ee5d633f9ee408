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

    def __init__(self, config: LmConfig, device="cuda", seed: Optional[int] = None, vocab_pad: int = 128):
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
        self.m = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
        self.p = {n: self._view(self.params, n) for n in PARAM_ORDER}
        self.w = {n: self._view(self.params_lp, n) for n in PARAM_ORDER}
        self.g = {n: self._view(self.grads, n) for n in PARAM_ORDER}
        self.opt_state = K.opt_state_tensor(dev)
        self._opt_host = torch.zeros(self.opt_state.numel(), dtype=torch.uint8).pin_memory()
        self._lr_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self.chunks = K.make_chunks(
            [(self.offsets[n], math.prod(shapes[n]), 1.0 if n in DECAY else 0.0, 1.0) for n in PARAM_ORDER],
            device=dev)
        self.loss_buf = torch.zeros(1, dtype=torch.float32, device=dev)
        self._acts = None
        self._acts_key = None
        self.step_count = 0
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
    def _alloc_acts(self, B: int, T: int):
        key = (B, T)
        if self._acts_key == key:
            return self._acts
        dev, L, C, F, H = self.device, self.L, self.C, self.F, self.H
        N = B * T
        bf, f32 = torch.bfloat16, torch.float32
        a = {
            "res": torch.empty((2 * L + 1, N, C), dtype=f32, device=dev),   # residual stream checkpoints
            "ln1": torch.empty((L, N, C), dtype=bf, device=dev),
            "ln1_mean": torch.empty((L, N), dtype=f32, device=dev), "ln1_rstd": torch.empty((L, N), dtype=f32, device=dev),
            "qkv": torch.empty((L, B, T, 3, H, C // H), dtype=bf, device=dev),
            "atty": torch.empty((L, B, T, H, C // H), dtype=bf, device=dev),
            "lse": torch.empty((L, B, H, T), dtype=f32, device=dev),
            "ln2": torch.empty((L, N, C), dtype=bf, device=dev),
            "ln2_mean": torch.empty((L, N), dtype=f32, device=dev), "ln2_rstd": torch.empty((L, N), dtype=f32, device=dev),
            "fch_pre": torch.empty((L, N, F), dtype=bf, device=dev),
            "fch": torch.empty((L, N, F), dtype=bf, device=dev),
            "lnf": torch.empty((N, C), dtype=bf, device=dev),
            "lnf_mean": torch.empty(N, dtype=f32, device=dev), "lnf_rstd": torch.empty(N, dtype=f32, device=dev),
            "logits": torch.empty((N, self.Vp), dtype=bf, device=dev),
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

    # ------------------------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor, *, want_logits: bool = True):
        """tokens [B, T] int32 on the device.  Fills the activation buffers; returns logits [B*T, Vp]."""
        B, T = tokens.shape
        a = self._alloc_acts(B, T)
        w, L, C = self.w, self.L, self.C
        N = B * T
        res = a["res"]
        _embedding_into(res[0], tokens, w["wte"], w["wpe"], T)
        for l in range(L):
            x_in, x_mid, x_out = res[2 * l], res[2 * l + 1], res[2 * l + 2]
            _norm_into(a["ln1"][l], a["ln1_mean"][l], a["ln1_rstd"][l], x_in, self.p["ln1_w"][l], self.p["ln1_b"][l])
            qkv = a["qkv"][l]
            K.gemm(a["ln1"][l], w["qkv_w"][l], bias=w["qkv_b"][l], out=qkv.view(N, 3 * C))
            _attn_fwd_into(a["atty"][l], a["lse"][l], qkv)
            K.gemm(a["atty"][l].view(N, C), w["attproj_w"][l], bias=w["attproj_b"][l], residual=x_in, out=x_mid)
            _norm_into(a["ln2"][l], a["ln2_mean"][l], a["ln2_rstd"][l], x_mid, self.p["ln2_w"][l], self.p["ln2_b"][l])
            K.gemm(a["ln2"][l], w["fc_w"][l], bias=w["fc_b"][l], act="gelu", aux_out=a["fch_pre"][l], out=a["fch"][l])
            K.gemm(a["fch"][l], w["fcproj_w"][l], bias=w["fcproj_b"][l], residual=x_mid, out=x_out)
        _norm_into(a["lnf"], a["lnf_mean"], a["lnf_rstd"], res[2 * L], self.p["lnf_w"], self.p["lnf_b"])
        if want_logits:
            K.gemm(a["lnf"], w["wte"], out=a["logits"])
        return a["logits"]

    # --------------------------------------------------------------------------- forward + backward
    def forward_backward(self, tokens: torch.Tensor, grad_scale: float = 1.0, accumulate_loss: bool = False,
                         loss_weight: float = 1.0, smoothing: float = 0.0, z_loss: float = 0.0) -> torch.Tensor:
        """One micro-step.  Gradients accumulate into ``self.grads`` (zeroed by the optimizer step).
        Returns the device tensor holding the (weighted, accumulated) loss."""
        B, T = tokens.shape
        N = B * T
        a = self._alloc_acts(B, T)
        w, g, L, C, F = self.w, self.g, self.L, self.C, self.F
        logits = self.forward(tokens)
        K.cross_entropy_shifted(logits, tokens, vocab=self.V, smoothing=smoothing, z_loss=z_loss,
                                grad_scale=grad_scale, loss_out=self.loss_buf, loss_weight=loss_weight,
                                accumulate_loss=accumulate_loss, seq_len=T)
        dlogits = logits
        res = a["res"]
        # head: dlnf = dlogits @ wte ; dwte += dlogits^T @ lnf
        K.gemm(dlogits, w["wte"], b_mn=True, out=a["dlnf"])
        K.gemm(dlogits, a["lnf"], a_mn=True, b_mn=True, out=g["wte"], accumulate=True)
        dres, dres_other, dres_lp = a["dres_a"], a["dres_b"], a["dres_lp"]
        # each norm backward also sums the columns of its BF16 dx: the bias gradient of the projection that follows
        K.norm_bwd(a["dlnf"], res[2 * L], self.p["lnf_w"], a["lnf_mean"], a["lnf_rstd"], dx=dres, dx_lp=dres_lp,
                   dgamma=g["lnf_w"], dbeta=g["lnf_b"], accumulate_params=True, dx_colsum=g["fcproj_b"][L - 1])
        for l in range(L - 1, -1, -1):
            x_in, x_mid = res[2 * l], res[2 * l + 1]
            # ---- MLP
            K.gemm(dres_lp, w["fcproj_w"][l], b_mn=True, act="dgelu", aux_in=a["fch_pre"][l], out=a["dfch"])
            K.gemm(dres_lp, a["fch"][l], a_mn=True, b_mn=True, out=g["fcproj_w"][l], accumulate=True, split_k=0)
            K.gemm(a["dfch"], w["fc_w"][l], b_mn=True, out=a["dln"])
            K.gemm(a["dfch"], a["ln2"][l], a_mn=True, b_mn=True, out=g["fc_w"][l], accumulate=True, split_k=0)
            K.colsum(a["dfch"], out=g["fc_b"][l], accumulate=True)
            K.norm_bwd(a["dln"], x_mid, self.p["ln2_w"][l], a["ln2_mean"][l], a["ln2_rstd"][l], add=dres,
                       dx=dres_other, dx_lp=dres_lp, dgamma=g["ln2_w"][l], dbeta=g["ln2_b"][l], accumulate_params=True,
                       dx_colsum=g["attproj_b"][l])
            dres, dres_other = dres_other, dres
            # ---- attention
            K.gemm(dres_lp, w["attproj_w"][l], b_mn=True, out=a["datty"].view(N, C))
            K.gemm(dres_lp, a["atty"][l].view(N, C), a_mn=True, b_mn=True, out=g["attproj_w"][l], accumulate=True,
                   split_k=0)
            qkv, dqkv = a["qkv"][l], a["dqkv"]
            K.attention_bwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], a["atty"][l], a["lse"][l], a["datty"],
                            causal=True, dq=dqkv[:, :, 0], dk=dqkv[:, :, 1], dv=dqkv[:, :, 2])
            dq2 = dqkv.view(N, 3 * C)
            K.gemm(dq2, w["qkv_w"][l], b_mn=True, out=a["dln"])
            K.gemm(dq2, a["ln1"][l], a_mn=True, b_mn=True, out=g["qkv_w"][l], accumulate=True, split_k=0)
            K.colsum(dq2, out=g["qkv_b"][l], accumulate=True)
            K.norm_bwd(a["dln"], x_in, self.p["ln1_w"][l], a["ln1_mean"][l], a["ln1_rstd"][l], add=dres,
                       dx=dres_other, dx_lp=dres_lp, dgamma=g["ln1_w"][l], dbeta=g["ln1_b"][l], accumulate_params=True,
                       dx_colsum=g["fcproj_b"][l - 1] if l > 0 else None)
            dres, dres_other = dres_other, dres
        K.embedding_bwd(tokens, dres.view(B, T, C), g["wte"], g["wpe"][:T], B, T,
                        deterministic=self.deterministic_embedding)
        return self.loss_buf

    # ---------------------------------------------------------------------------------- optimizer
    def set_optimizer(self, cfg: AdamWConfig, lr: Optional[float] = None, loss_scale: float = 1.0) -> None:
        """Writes hyper-parameters into the device-resident optimizer state (keeps step counters)."""
        cur = K.unpack_opt_state(bytes(self.opt_state.cpu().numpy().tobytes()))
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
        K.adamw(self.params, self.grads, self.m, self.v, self.params_lp, self.chunks, self.opt_state, zero_grad=True)
        self.step_count += 1

    def read_opt_state(self) -> "K.OptState":
        return K.unpack_opt_state(bytes(self.opt_state.cpu().numpy().tobytes()))

    # ---------------------------------------------------------------------------------- utilities
    def loss(self, tokens: torch.Tensor) -> float:
        logits = self.forward(tokens)
        B, T = tokens.shape
        out = torch.zeros(1, dtype=torch.float32, device=self.device)
        K.cross_entropy_shifted(logits, tokens, vocab=self.V, write_grad=False, loss_out=out, seq_len=T)
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
