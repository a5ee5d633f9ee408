"""Llama-style decoder trained tensor-parallel + sequence-parallel over the GPUs of one node, with hand-scheduled
forward and backward passes on the sm_100a kernels (no autograd, no library GEMM, no NCCL in the layer loop).

One process per GPU; rank r of n holds 1/n of every projection (attention heads, SwiGLU columns, vocabulary rows)
and 1/n of the token rows of the residual stream (sequence parallel).  The communication of a layer lives inside
the tensor-core kernels:

* column-parallel projections (QKV, gate/up, LM head) and the row-parallel backward products run as
  all-gather -> GEMM in ONE kernel (`symm.gemm_ag`): copier CTAs push this rank's normalised rows into every peer's
  gather buffer while the tcgen05 CTAs consume rows in their order of arrival; the gathered activations stay local
  and feed the weight-gradient GEMMs;
* row-parallel projections (attention output, MLP down) and the column-parallel backward products run as
  GEMM -> reduce-scatter in ONE kernel (`symm.gemm_rs`): copier CTAs push every finished 256-row block of BF16 partial
  sums into the owner's slots over NVLink while the tcgen05 CTAs work on the next blocks, and the owner adds the
  slots, in rank order, to its FP32 residual rows (`symm.sum_slots`);
* the embedding table and the LM head are split by vocabulary rows: lookups read the owner's rows through peer
  pointers, and the loss exchanges three numbers per row (`nx_vocab_ce_exchange`) instead of logits;
* replicated norm-weight gradients are summed with the fused peer-memory all-reduce and the global gradient norm
  is exchanged by the same kernel the sharded optimizer uses; AdamW is the multi-tensor kernel on the local shard.

With one rank the same code runs on local GEMMs, which is the oracle of the multi-rank tests.

Parity (behaviour): ParallelLm with tensor + sequence parallelism of the reference (include/nexus/dist/parallel_lm.hpp,
src/dist/parallel_lm.cpp:225-291 chunked all-gather/GEMM and GEMM/reduce-scatter forms, :560-665 vocabulary-parallel
embedding and loss), which runs FP32 on CPU ranks there.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Optional

import torch

from ..lm.config import LmConfig
from ..lm.rope import RopeCache
from ..ops import _cuda as K
from ..ops import _infer as KI
from .gpt import AdamWConfig, _align, _norm_into

MATRICES = ("wte", "head", "qkv_w", "o_w", "up_w", "down_w")
VECTORS = ("norm1", "norm2", "normf")


class LlamaTpModel:
    def __init__(self, config: LmConfig, pg=None, device="cuda", seed: Optional[int] = None, copier_ctas: int = 0,
                 full_weights: Optional[Dict[str, torch.Tensor]] = None):
        c = config
        if c.norm != "rmsnorm" or c.mlp != "swiglu" or c.pos != "rope" or c.bias or c.qkv_bias or c.tie_embeddings:
            raise ValueError("LlamaTpModel implements RMSNorm + SwiGLU + RoPE decoders with an untied head and no biases")
        if c.hdim() not in (64, 128):
            raise ValueError("head_dim must be 64 or 128")
        if c.padded_vocab() != c.vocab_size:
            raise ValueError("LlamaTpModel needs vocab_pad_multiple = 1 (choose a vocabulary that divides by the ranks)")
        self.config = c
        self.device = torch.device(device)
        self.pg = pg
        self.n = pg.size() if pg is not None else 1
        self.r = pg.rank() if pg is not None else 0
        n = self.n
        if c.n_head % n or c.kv_heads() % n or c.d_ff % n or c.padded_vocab() % n:
            raise ValueError("heads, kv heads, d_ff and the padded vocabulary must divide by the tensor-parallel degree")
        self.L, self.d, self.D = c.n_layer, c.d_model, c.hdim()
        self.Hl, self.Hkvl, self.Fl = c.n_head // n, c.kv_heads() // n, c.d_ff // n
        if self.Fl % 8 or (c.padded_vocab() // n) % 8:
            raise ValueError("d_ff / tp and vocab / tp must be multiples of 8")
        self.V, self.Vl = c.vocab_size, c.padded_vocab() // n
        self.v0 = self.r * self.Vl
        self.Nqkv = (self.Hl + 2 * self.Hkvl) * self.D
        # copier CTAs of the fused GEMMs: 8 fill the link between two ranks; at more ranks every projection is
        # link-bound and more copiers win although they take CTAs from the GEMM (Llama-7B, 8 ranks: 357 / 280 / 257 ms
        # per step with 8 / 16 / 32)
        self.copier_ctas = copier_ctas if copier_ctas > 0 else (32 if (pg.size() if pg is not None else 1) > 2 else 8)
        L, d, D = self.L, self.d, self.D
        shapes = {"wte": (self.Vl, d), "head": (self.Vl, d), "qkv_w": (L, self.Nqkv, d), "o_w": (L, d, self.Hl * D),
                  "up_w": (L, 2 * self.Fl, d), "down_w": (L, d, self.Fl),
                  "norm1": (L, d), "norm2": (L, d), "normf": (d,)}
        self.shapes = shapes
        self.offsets: Dict[str, int] = {}
        off = 0
        for name in MATRICES + VECTORS:
            off = _align(off)
            self.offsets[name] = off
            off += math.prod(shapes[name])
        self.num_params = _align(off)
        self.vec_off = self.offsets["norm1"]               # replicated 1-D parameters start here
        dev = self.device
        self.ws = None
        if n > 1:
            from ..parallel.symm import SymmetricWorkspace
            self.ws = SymmetricWorkspace(pg)
            self._lp_sym = self.ws.alloc(self.num_params, torch.bfloat16)   # peers read embedding rows from it
            self.params_lp = self._lp_sym.local
        else:
            self.params_lp = torch.zeros(self.num_params, dtype=torch.bfloat16, device=dev)
        self.params = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
        self.grads = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
        self.m = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.num_params, dtype=torch.float32, device=dev)
        names = MATRICES + VECTORS
        self.p = {k: self._view(self.params, k) for k in names}
        self.w = {k: self._view(self.params_lp, k) for k in names}
        self.g = {k: self._view(self.grads, k) for k in names}
        self.opt_state = K.opt_state_tensor(dev)
        self._opt_host = torch.zeros(self.opt_state.numel(), dtype=torch.uint8).pin_memory()
        self._lr_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self.chunks = K.make_chunks([(self.offsets[k], math.prod(shapes[k]), 1.0 if k in MATRICES else 0.0, 1.0)
                                     for k in names], device=dev)
        self.loss_buf = torch.zeros(1, dtype=torch.float32, device=dev)
        self.ce_scale = torch.ones(1, dtype=torch.float32, device=dev)
        self.rope = RopeCache(c, device=dev)
        self._acts = None
        self._acts_key = None
        self.step_count = 0
        self.init_weights(c.seed if seed is None else seed, full_weights)

    # ------------------------------------------------------------------------------------------ parameters
    def _view(self, flat, name):
        cnt = math.prod(self.shapes[name])
        return flat[self.offsets[name]: self.offsets[name] + cnt].view(self.shapes[name])

    @staticmethod
    def full_shapes(c: LmConfig) -> Dict[str, tuple]:
        """Shapes of the unsharded parameters (`full_weights` of the constructor, and what `gather_full` returns)."""
        H, Hk, D, d, F, L = c.n_head, c.kv_heads(), c.hdim(), c.d_model, c.d_ff, c.n_layer
        return {"wte": (c.padded_vocab(), d), "head": (c.padded_vocab(), d), "q_w": (L, H * D, d), "k_w": (L, Hk * D, d),
                "v_w": (L, Hk * D, d), "o_w": (L, d, H * D), "gate_w": (L, F, d), "up_w": (L, F, d), "down_w": (L, d, F),
                "norm1": (L, d), "norm2": (L, d), "normf": (d,)}

    @staticmethod
    def random_full_weights(c: LmConfig, seed: int, device="cpu") -> Dict[str, torch.Tensor]:
        g = torch.Generator(device="cpu").manual_seed(seed)
        out = {}
        for k, shp in LlamaTpModel.full_shapes(c).items():
            if k.startswith("norm"):
                out[k] = torch.ones(shp)
            else:
                std = c.init_std / math.sqrt(2 * c.n_layer) if k in ("o_w", "down_w") else c.init_std
                out[k] = torch.randn(shp, generator=g) * std
        out["wte"][c.vocab_size:].zero_()
        out["head"][c.vocab_size:].zero_()
        return {k: v.to(device) for k, v in out.items()}

    def init_weights(self, seed: int, full: Optional[Dict[str, torch.Tensor]] = None) -> None:
        """From ``full`` (unsharded tensors; every rank slices its part), else random per-rank slices drawn on the
        device (throughput runs: the full model is never materialised)."""
        c, r = self.config, self.r
        Hl, Hkvl, D, Fl, Vl = self.Hl, self.Hkvl, self.D, self.Fl, self.Vl
        self.params.zero_()
        if full is None:
            g = torch.Generator(device=self.device).manual_seed(seed * 1000 + r)
            for k in MATRICES:
                t = self.p[k]
                std = c.init_std / math.sqrt(2 * c.n_layer) if k in ("o_w", "down_w") else c.init_std
                t.copy_(torch.randn(t.shape, generator=g, device=self.device) * std)
            for k in VECTORS:
                self.p[k].fill_(1.0)
        else:
            f = {k: v.to(self.device, torch.float32) for k, v in full.items()}
            self.p["wte"].copy_(f["wte"][r * Vl: (r + 1) * Vl])
            self.p["head"].copy_(f["head"][r * Vl: (r + 1) * Vl])
            q = f["q_w"][:, r * Hl * D: (r + 1) * Hl * D]
            k_ = f["k_w"][:, r * Hkvl * D: (r + 1) * Hkvl * D]
            v_ = f["v_w"][:, r * Hkvl * D: (r + 1) * Hkvl * D]
            self.p["qkv_w"].copy_(torch.cat([q, k_, v_], dim=1))
            self.p["o_w"].copy_(f["o_w"][:, :, r * Hl * D: (r + 1) * Hl * D])
            self.p["up_w"].copy_(torch.cat([f["gate_w"][:, r * Fl: (r + 1) * Fl], f["up_w"][:, r * Fl: (r + 1) * Fl]], dim=1))
            self.p["down_w"].copy_(f["down_w"][:, :, r * Fl: (r + 1) * Fl])
            for k in VECTORS:
                self.p[k].copy_(f[k])
        self.refresh_shadow()

    def refresh_shadow(self) -> None:
        self.params_lp.copy_(self.params)
        if self.ws is not None:
            torch.cuda.synchronize()
            self.pg.barrier()

    def gather_full(self, what: str = "params") -> Dict[str, torch.Tensor]:
        """Unsharded FP32 tensors (``what``: "params" or "grads") on every rank, through NCCL (tests / export)."""
        src = {"params": self.p, "grads": self.g}[what]
        n, Hl, Hkvl, D, Fl = self.n, self.Hl, self.Hkvl, self.D, self.Fl

        def cat(t, dim):
            if n == 1:
                return t.clone()
            parts = [torch.empty_like(t) for _ in range(n)]
            torch.distributed.all_gather(parts, t.contiguous(), group=self.pg.group)
            return torch.cat(parts, dim=dim)

        qkv = src["qkv_w"]
        up = src["up_w"]
        out = {"wte": cat(src["wte"], 0), "head": cat(src["head"], 0),
               "q_w": cat(qkv[:, : Hl * D], 1), "k_w": cat(qkv[:, Hl * D: (Hl + Hkvl) * D], 1),
               "v_w": cat(qkv[:, (Hl + Hkvl) * D:], 1), "o_w": cat(src["o_w"], 2),
               "gate_w": cat(up[:, :Fl], 1), "up_w": cat(up[:, Fl:], 1), "down_w": cat(src["down_w"], 2)}
        for k in VECTORS:
            out[k] = src[k].clone()
        return out

    def count_parameters(self) -> int:
        c = self.config
        return sum(math.prod(s) for s in self.full_shapes(c).values()) - 2 * (c.padded_vocab() - c.vocab_size) * c.d_model

    def flops_per_token(self, T: int) -> float:
        c = self.config
        return 6.0 * (self.count_parameters() - c.padded_vocab() * c.d_model) + 12.0 * c.n_layer * c.n_head * c.hdim() * T

    # --------------------------------------------------------------------------------------------- buffers
    def _alloc(self, B: int, T: int):
        key = (B, T)
        if self._acts_key == key:
            return self._acts
        n, dev, L, d, D = self.n, self.device, self.L, self.d, self.D
        M = B * T
        if M % n or (n > 1 and (M // n) % 256):
            raise ValueError("batch * seq_len must divide by the tensor-parallel degree into multiples of 256 rows")
        Ml = M // n
        bf, f32 = torch.bfloat16, torch.float32
        a = {"M": M, "Ml": Ml}
        if n > 1:
            from ..parallel.symm import GatherSite
            ws = self.ws
            self._site = GatherSite(ws, Ml)
            # per layer: gathered norm outputs [M, d] (this rank writes its block, the all-gather GEMM fills the rest)
            a["xn1_sym"] = [ws.alloc(M * d, bf) for _ in range(L)]
            a["xn2_sym"] = [ws.alloc(M * d, bf) for _ in range(L)]
            a["xnf_sym"] = ws.alloc(M * d, bf)
            a["dz_sym"] = ws.alloc(M * d, bf)            # gathered gradient of a row-parallel output
            a["slots_sym"] = ws.alloc(n * Ml * d, bf)    # [source rank][Ml][d] partial sums of a reduce-scatter
            a["dh_sym"] = ws.alloc(Ml * d, bf)           # gradient of the embedding output (read by the vocabulary owners)
            a["partial"] = torch.empty((M, d), dtype=bf, device=dev)   # this rank's partial sums of a row-parallel product
            a["rs_done"] = torch.zeros(M // 256, dtype=torch.int32, device=dev)
            a["xn1"] = [s.local.view(M, d) for s in a["xn1_sym"]]
            a["xn2"] = [s.local.view(M, d) for s in a["xn2_sym"]]
            a["xnf"] = a["xnf_sym"].local.view(M, d)
            a["dz"] = a["dz_sym"].local.view(M, d)
            a["slots"] = a["slots_sym"].local
            a["dh"] = a["dh_sym"].local.view(Ml, d)
            rows = M
            a["ce_table"] = ws.alloc(n * rows * 3, f32)
            a["vec_src"] = ws.alloc(_align(self.num_params - self.vec_off, 8), f32)
            a["vec_dst"] = ws.alloc(_align(self.num_params - self.vec_off, 8), f32)
        else:
            a["xn1"] = [torch.empty((M, d), dtype=bf, device=dev) for _ in range(L)]
            a["xn2"] = [torch.empty((M, d), dtype=bf, device=dev) for _ in range(L)]
            a["xnf"] = torch.empty((M, d), dtype=bf, device=dev)
            a["dz"] = torch.empty((M, d), dtype=bf, device=dev)
            a["dh"] = torch.empty((Ml, d), dtype=bf, device=dev)
        a["res"] = torch.empty((2 * L + 1, Ml, d), dtype=f32, device=dev)      # residual stream checkpoints (local rows)
        a["rstd1"] = torch.empty((L, Ml), dtype=f32, device=dev)
        a["rstd2"] = torch.empty((L, Ml), dtype=f32, device=dev)
        a["rstdf"] = torch.empty(Ml, dtype=f32, device=dev)
        a["qkv"] = torch.empty((L, M, self.Nqkv), dtype=bf, device=dev)
        a["atty"] = torch.empty((L, M, self.Hl * D), dtype=bf, device=dev)
        a["lse"] = torch.empty((L, B, self.Hl, T), dtype=f32, device=dev)
        a["ug"] = torch.empty((L, M, 2 * self.Fl), dtype=bf, device=dev)
        a["act"] = torch.empty((M, self.Fl), dtype=bf, device=dev)            # recomputed in the backward pass
        a["logits"] = torch.empty((M, self.Vl), dtype=bf, device=dev)
        a["stats"] = torch.empty((M, 3), dtype=f32, device=dev)
        a["merged"] = torch.empty((M, 3), dtype=f32, device=dev)
        a["targets"] = torch.empty(M, dtype=torch.int32, device=dev)
        a["positions"] = torch.arange(T, dtype=torch.int32, device=dev).repeat(B)
        # backward scratch
        a["dres_a"] = torch.empty((Ml, d), dtype=f32, device=dev)
        a["dres_b"] = torch.empty((Ml, d), dtype=f32, device=dev)
        a["dxn"] = torch.empty((Ml, d), dtype=bf, device=dev)
        a["dact"] = torch.empty((M, self.Fl), dtype=bf, device=dev)
        a["dug"] = torch.empty((M, 2 * self.Fl), dtype=bf, device=dev)
        a["datty"] = torch.empty((M, self.Hl * D), dtype=bf, device=dev)
        a["dqkv"] = torch.empty((M, self.Nqkv), dtype=bf, device=dev)
        self._acts, self._acts_key = a, key
        if n > 1:
            torch.cuda.synchronize()
            self.pg.barrier()
        return a

    # ---------------------------------------------------------------------------- distributed building blocks
    def _col_gemm(self, gather_sym, x_full, w, out, b_mn=False):
        """out[M, N] = all-gather(x)[M, d] @ w^T, x's local block already in place."""
        if self.n == 1:
            K.gemm(x_full, w, b_mn=b_mn, out=out)
            return
        from ..parallel.symm import gemm_ag
        self.ws.barrier()   # every rank has left the previous user of this gather buffer and of the flags
        gemm_ag(self._site, gather_sym, w, out, k=self.d, b_mn=b_mn, copier_ctas=self.copier_ctas)

    def _row_gemm_rs(self, a_mat, w, b_mn, residual, out, out_lp=None):
        """out[Ml, d] = residual + reduce-scatter(a_mat[M, k] @ w^T)[own rows]   (FP32 out, optional BF16 copy)."""
        A = self._acts
        if self.n == 1:
            tmp = K.gemm(a_mat, w, b_mn=b_mn, out_dtype=torch.float32, residual=residual,
                         out=out if out.dtype == torch.float32 else None)
            if out.dtype != torch.float32:
                out.copy_(tmp)
            if out_lp is not None:
                out_lp.copy_(out)
            return
        from ..parallel.symm import gemm_rs, sum_slots
        n, Ml, d = self.n, A["Ml"], self.d
        self.ws.barrier()   # the owners have consumed the previous contents of their slots
        gemm_rs(self.ws, a_mat, w, A["partial"], A["slots_sym"], A["rs_done"], b_mn=b_mn, copier_ctas=self.copier_ctas)
        self.ws.barrier()   # every rank's partial blocks have landed
        sum_slots(A["slots"], n, Ml, d, out, residual=residual, out_lp=out_lp, own=self._own(A["partial"]), own_rank=self.r)

    def _own(self, full_rows):
        """This rank's row block of a gathered [M, d] buffer."""
        Ml = self._acts["Ml"]
        return full_rows[self.r * Ml: (self.r + 1) * Ml]

    # --------------------------------------------------------------------------------------------- forward
    def forward(self, tokens: torch.Tensor):
        """tokens [B, T] int32 (the same on every rank).  Returns this rank's logits columns [B*T, V/n]."""
        B, T = tokens.shape
        A = self._alloc(B, T)
        n, r, L, d, D = self.n, self.r, self.L, self.d, self.D
        M, Ml = A["M"], A["Ml"]
        w, p = self.w, self.p
        Hl, Hkvl = self.Hl, self.Hkvl
        flat = tokens.reshape(-1)
        res = A["res"]
        # ---- vocabulary-parallel embedding of this rank's rows
        if n == 1:
            res[0].copy_(w["wte"][flat.long()])
        else:
            K._check(K.lib().nx_tp_embed_gather(K._p(flat[r * Ml: (r + 1) * Ml]), C.byref(self._lp_sym.offset_table(
                self.offsets["wte"] * 2)), C.c_int(n), C.c_int(self.Vl), C.c_int(d), K._p(res[0]), C.c_int(Ml),
                K._stream()), "nx_tp_embed_gather")
        eps = self.config.norm_eps
        for l in range(L):
            x_in, x_mid, x_out = res[2 * l], res[2 * l + 1], res[2 * l + 2]
            _norm_into(self._own(A["xn1"][l]), None, A["rstd1"][l], x_in, p["norm1"][l], None, eps=eps, rms=True)
            qkv = A["qkv"][l]
            self._col_gemm(A["xn1_sym"][l] if n > 1 else None, A["xn1"][l], w["qkv_w"][l], qkv)
            q = qkv[:, : Hl * D].view(M, Hl, D)
            k = qkv[:, Hl * D: (Hl + Hkvl) * D].view(M, Hkvl, D)
            v = qkv[:, (Hl + Hkvl) * D:].view(M, Hkvl, D)
            KI.rope_(q, A["positions"], self.rope.cos, self.rope.sin)
            KI.rope_(k, A["positions"], self.rope.cos, self.rope.sin)
            K.attention_fwd(q.view(B, T, Hl, D), k.view(B, T, Hkvl, D), v.view(B, T, Hkvl, D), causal=True,
                            out=A["atty"][l].view(B, T, Hl, D), lse=A["lse"][l])
            self._row_gemm_rs(A["atty"][l], w["o_w"][l], False, x_in, x_mid)
            _norm_into(self._own(A["xn2"][l]), None, A["rstd2"][l], x_mid, p["norm2"][l], None, eps=eps, rms=True)
            self._col_gemm(A["xn2_sym"][l] if n > 1 else None, A["xn2"][l], w["up_w"][l], A["ug"][l])
            K._check(K.lib().nx_gated_fwd(K._p(A["ug"][l]), K._p(A["act"]), C.c_int64(M), C.c_int(self.Fl), C.c_int(0),
                                          K._stream()), "nx_gated_fwd")
            self._row_gemm_rs(A["act"], w["down_w"][l], False, x_mid, x_out)
        _norm_into(self._own(A["xnf"]), None, A["rstdf"], res[2 * L], p["normf"], None, eps=eps, rms=True)
        self._col_gemm(A["xnf_sym"] if n > 1 else None, A["xnf"], w["head"], A["logits"])
        return A["logits"]

    # --------------------------------------------------------------------------------------- loss + backward
    def _loss_and_dlogits(self, tokens, grad_scale: float, loss_weight: float, accumulate_loss: bool):
        """Vocabulary-parallel shifted cross-entropy on the local logits columns; leaves d(logits) in place."""
        A = self._acts
        B, T = tokens.shape
        M, n = A["M"], self.n
        tg = A["targets"].view(B, T)
        tg[:, :-1].copy_(tokens[:, 1:])
        tg[:, -1].fill_(-100)
        L_ = K.lib()
        logits = A["logits"]
        K._check(L_.nx_tp_ce_stats(K._p(logits), C.c_int64(logits.stride(0)), C.c_int(M), C.c_int(self.Vl),
                                   K._p(A["targets"]), C.c_int(self.v0), K._p(A["stats"]), K._stream()), "nx_tp_ce_stats")
        if n == 1:
            merged = A["stats"]
        else:
            ws = self.ws
            ws.barrier()     # the previous call's tables have been read by everyone
            K._check(L_.nx_vocab_ce_exchange(K._p(A["stats"]), C.byref(A["ce_table"].table), C.byref(ws.flags.table),
                                             C.c_int(ws.rank), C.c_int(n), C.c_int(M), K._p(ws.counter),
                                             K._p(A["merged"]), K._p(K.status_word(self.device)), K._stream()),
                     "nx_vocab_ce_exchange")
            merged = A["merged"]
        valid = B * (T - 1)
        K._check(L_.nx_tp_ce_loss(K._p(merged), K._p(A["targets"]), C.c_int(M), C.c_float(1.0 / valid),
                                  C.c_float(loss_weight), C.c_int(int(accumulate_loss)), K._p(self.loss_buf),
                                  K._stream()), "nx_tp_ce_loss")
        self.ce_scale.fill_(grad_scale / valid)
        K._check(L_.nx_tp_ce_grad(K._p(logits), C.c_int64(logits.stride(0)), C.c_int(M), C.c_int(self.Vl),
                                  K._p(A["targets"]), C.c_int(self.v0), K._p(merged), K._p(self.ce_scale), K._stream()),
                 "nx_tp_ce_grad")

    def forward_backward(self, tokens: torch.Tensor, grad_scale: float = 1.0, accumulate_loss: bool = False,
                         loss_weight: float = 1.0) -> torch.Tensor:
        """One micro-step: gradients accumulate into ``self.grads`` (cleared by the optimizer step)."""
        B, T = tokens.shape
        self.forward(tokens)
        A = self._acts
        n, r, L, d, D = self.n, self.r, self.L, self.d, self.D
        M, Ml = A["M"], A["Ml"]
        w, p, g = self.w, self.p, self.g
        Hl, Hkvl, Fl = self.Hl, self.Hkvl, self.Fl
        res = A["res"]
        self._loss_and_dlogits(tokens, grad_scale, loss_weight, accumulate_loss)
        dlogits = A["logits"]
        dres, dres_other = A["dres_a"], A["dres_b"]
        # ---- head: d(xnf) = RS(dlogits @ head) ; d(head) += dlogits^T @ gathered xnf
        self._row_gemm_rs(dlogits, w["head"], True, None, dres, out_lp=A["dxn"])
        K.gemm(dlogits, A["xnf"], a_mn=True, b_mn=True, out=g["head"], accumulate=True, split_k=0)
        K.norm_bwd(A["dxn"], res[2 * L], p["normf"], None, A["rstdf"], rms=True, dx=dres_other,
                   dx_lp=self._own(A["dz"]), dgamma=g["normf"], accumulate_params=True)
        dres, dres_other = dres_other, dres
        for l in range(L - 1, -1, -1):
            x_in, x_mid = res[2 * l], res[2 * l + 1]
            # ---- MLP.  dz (gathered) = d(x_out) rows of every rank; act is recomputed from the saved gate/up
            K._check(K.lib().nx_gated_fwd(K._p(A["ug"][l]), K._p(A["act"]), C.c_int64(M), C.c_int(Fl), C.c_int(0),
                                          K._stream()), "nx_gated_fwd")
            self._col_gemm(A["dz_sym"] if n > 1 else None, A["dz"], w["down_w"][l], A["dact"], b_mn=True)
            K.gemm(A["dz"], A["act"], a_mn=True, b_mn=True, out=g["down_w"][l], accumulate=True, split_k=0)
            K._check(K.lib().nx_gated_bwd(K._p(A["ug"][l]), K._p(A["dact"]), K._p(A["dug"]), C.c_int64(M), C.c_int(Fl),
                                          C.c_int(0), K._stream()), "nx_gated_bwd")
            self._row_gemm_rs(A["dug"], w["up_w"][l], True, None, dres_other, out_lp=A["dxn"])
            K.gemm(A["dug"], A["xn2"][l], a_mn=True, b_mn=True, out=g["up_w"][l], accumulate=True, split_k=0)
            K.norm_bwd(A["dxn"], x_mid, p["norm2"][l], None, A["rstd2"][l], rms=True, add=dres, dx=dres_other,
                       dx_lp=self._own(A["dz"]), dgamma=g["norm2"][l], accumulate_params=True)
            dres, dres_other = dres_other, dres
            # ---- attention
            self._col_gemm(A["dz_sym"] if n > 1 else None, A["dz"], w["o_w"][l], A["datty"], b_mn=True)
            K.gemm(A["dz"], A["atty"][l], a_mn=True, b_mn=True, out=g["o_w"][l], accumulate=True, split_k=0)
            qkv, dqkv = A["qkv"][l], A["dqkv"]
            q = qkv[:, : Hl * D].view(B, T, Hl, D)
            k = qkv[:, Hl * D: (Hl + Hkvl) * D].view(B, T, Hkvl, D)
            v = qkv[:, (Hl + Hkvl) * D:].view(B, T, Hkvl, D)
            dq = dqkv[:, : Hl * D].view(B, T, Hl, D)
            dk = dqkv[:, Hl * D: (Hl + Hkvl) * D].view(B, T, Hkvl, D)
            dv = dqkv[:, (Hl + Hkvl) * D:].view(B, T, Hkvl, D)
            K.attention_bwd(q, k, v, A["atty"][l].view(B, T, Hl, D), A["lse"][l], A["datty"].view(B, T, Hl, D),
                            causal=True, dq=dq, dk=dk, dv=dv)
            KI.rope_(dq.view(M, Hl, D), A["positions"], self.rope.cos, self.rope.sin, inverse=True)
            KI.rope_(dk.view(M, Hkvl, D), A["positions"], self.rope.cos, self.rope.sin, inverse=True)
            self._row_gemm_rs(dqkv, w["qkv_w"][l], True, None, dres_other, out_lp=A["dxn"])
            K.gemm(dqkv, A["xn1"][l], a_mn=True, b_mn=True, out=g["qkv_w"][l], accumulate=True, split_k=0)
            K.norm_bwd(A["dxn"], x_in, p["norm1"][l], None, A["rstd1"][l], rms=True, add=dres, dx=dres_other,
                       dx_lp=self._own(A["dz"]) if l > 0 else A["dh"], dgamma=g["norm1"][l], accumulate_params=True)
            dres, dres_other = dres_other, dres
        # ---- embedding gradient for this rank's vocabulary rows (rows of every rank's d(h0))
        flat = tokens.reshape(-1)
        if n == 1:
            g["wte"].index_add_(0, flat.long(), A["dh"].float())
        else:
            self.ws.barrier()   # every rank's d(h0) is complete
            K._check(K.lib().nx_tp_embed_bwd(K._p(flat), C.c_int(M), C.byref(A["dh_sym"].table), C.c_int(Ml),
                                             C.c_int(self.v0), C.c_int(self.Vl), C.c_int(d), K._p(g["wte"]), K._stream()),
                     "nx_tp_embed_bwd")
        return self.loss_buf

    # ------------------------------------------------------------------------------------------- optimizer
    def set_optimizer(self, cfg: AdamWConfig, lr: Optional[float] = None) -> None:
        cur = K.unpack_opt_state(bytes(self.opt_state.cpu().numpy().tobytes()))
        raw = K.pack_opt_state(lr=cfg.lr if lr is None else lr, weight_decay=cfg.weight_decay, beta1=cfg.beta1,
                               beta2=cfg.beta2, eps=cfg.eps, max_grad_norm=cfg.grad_clip, loss_scale=1.0, step=cur.step,
                               skipped=cur.skipped, good_steps=cur.good_steps, inv_bias1=cur.inv_bias1,
                               inv_bias2=cur.inv_bias2)
        self._opt_host.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
        self.opt_state.copy_(self._opt_host, non_blocking=True)

    def set_lr(self, lr: float) -> None:
        off = K.OptState.lr.offset
        self._lr_host[0] = lr
        self.opt_state[off: off + 4].view(torch.float32).copy_(self._lr_host, non_blocking=True)

    def optimizer_step(self) -> None:
        """Sums the replicated (norm) gradients over the ranks, exchanges the global gradient norm, clips and applies
        AdamW to the local shard, refreshes the BF16 shadow and clears the gradients."""
        n = self.n
        if n == 1:
            K.grad_norm(self.grads, self.opt_state)
        else:
            from ..parallel.symm import fused_all_reduce
            A, ws = self._acts, self.ws
            cnt = self.num_params - self.vec_off
            cnt8 = A["vec_src"].local.numel()
            A["vec_src"].local[:cnt].copy_(self.grads[self.vec_off:])
            if cnt8 > cnt:
                A["vec_src"].local[cnt:].zero_()
            fused_all_reduce(ws, A["vec_src"], A["vec_dst"], cnt8)
            self.grads[self.vec_off:].copy_(A["vec_dst"].local[:cnt])
            # local square sum of the sharded part + 1/n of the replicated part (it is identical on every rank)
            K.grad_norm(self.grads[: self.vec_off], self.opt_state, local_only=True)
            off = K.OptState.local_sq.offset
            parts = torch.empty(2, dtype=torch.float64, device=self.device)
            parts[0:1].copy_(self.opt_state[off: off + 8].view(torch.float64))
            parts[1:2].copy_((A["vec_dst"].local[:cnt].double() ** 2).sum().reshape(1) / n)
            K._check(K.lib().nx_comm_norm_exchange(K._p(parts), C.c_int(2), C.byref(ws.slots.table),
                                                   C.byref(ws.flags.table), C.c_int(ws.rank), C.c_int(n),
                                                   K._p(ws.counter), K._p(self.opt_state),
                                                   K._p(K.status_word(self.device)), K._stream()), "nx_comm_norm_exchange")
        K.adamw(self.params, self.grads, self.m, self.v, self.params_lp, self.chunks, self.opt_state, zero_grad=True)
        self.step_count += 1
        if n > 1:
            self.ws.barrier()   # the new embedding rows are visible before any peer looks them up

    def read_opt_state(self):
        return K.unpack_opt_state(bytes(self.opt_state.cpu().numpy().tobytes()))
