"""`ParallelLm`: one language model trained on a 4-D mesh ``dp x pp x cp x tp`` (tp varies fastest),
sliced from a full `lm.LanguageModel` that every rank builds with the same seed.

* **TP (Megatron)**: QKV and MLP-up are column-parallel (heads / matched ``W1|W3`` slices), attention
  output and MLP-down are row-parallel; the token embedding and the LM head are vocabulary-parallel
  and the cross-entropy never gathers logits (local max -> all-reduce(max); [sum-exp | target logit]
  -> all-reduce(sum)).
* **SP**: the norm / residual regions are sharded over tokens inside the tp group: all-gather on
  region entry, reduce-scatter on exit; gradients of replicated parameters are all-reduced over tp.
* **Async TP**: all-gather+GEMM and GEMM+reduce-scatter run as a ring of chunk GEMMs, the next chunk
  travelling while the current one is multiplied.
* **PP**: layers are cost-balanced into ``pp * v`` chunks (chunk g on rank g % pp) and driven by the
  GPipe / 1F1B / interleaved-1F1B / ZB-H1 action lists with point-to-point activation transfers;
  tied embeddings are reconciled by an all-reduce between the first and last stage.
* **CP**: ring attention (zigzag or contiguous) or Ulysses inside every block.
* **DP x CP** gradient sync on one flat buffer (reduce-scatter + all-gather); ``zero = 1`` shards the
  AdamW state over that group and all-gathers the updated parameters.

Parity: include/nexus/dist/parallel_lm.hpp:15-163 and src/dist/parallel_lm.cpp:219-1350 of the reference.
"""
from __future__ import annotations

import io
import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from ..fused import ops as F_
from ..lm.config import LmConfig
from ..lm.rope import RopeCache, apply_rope
from . import collectives as C
from .context_parallel import chunk_ids, ring_attention, shard_sequence, ulysses_attention
from .dtensor import DeviceMesh
from .pipeline import PipeAction, balance_partition, make_schedule, theoretical_bubble


@dataclass
class ParallelConfig:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    cp: int = 1
    zero: int = 0
    sp: bool = False
    async_tp: bool = False
    pp_schedule: str = "1f1b"
    virtual_stages: int = 1
    cp_algorithm: str = "ring"     # "ring" | "ulysses"
    cp_comm: str = "fused"         # on GPUs: "fused" = ring / Ulysses over peer memory (the attention kernels read the
                                   # owners' K / V by TMA, head <-> sequence exchange by peer stores); "nccl" = send_recv
    cp_layout: str = "zigzag"      # "zigzag" | "contiguous"

    def world(self) -> int:
        return self.dp * self.tp * self.pp * self.cp


@dataclass
class ParallelStepStats:
    loss: float = 0.0
    grad_norm: float = 0.0
    bubble_theory: float = 0.0
    p2p_messages: int = 0
    p2p_bytes: int = 0


# ------------------------------------------------------------------------------ async-TP rings
class _RingAllGatherMatmul(torch.autograd.Function):
    """y = all_gather_rows(x) @ w.T computed chunk by chunk while the next chunk moves round the ring."""

    @staticmethod
    def forward(ctx, x, w, pg):
        n, r = pg.size(), pg.rank()
        rows = x.shape[0]
        out = x.new_empty((rows * n, w.shape[0]))
        cur = x.contiguous()
        for s in range(n):
            src = (r - s) % n
            nxt = torch.empty_like(cur)
            if s + 1 < n:
                pg.send_recv(cur, (r + 1) % n, nxt, (r - 1) % n, tag=300 + s)
            out[src * rows: (src + 1) * rows] = cur @ w.t()
            cur = nxt
        ctx.save_for_backward(x, w)
        ctx.pg = pg
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        pg = ctx.pg
        n = pg.size()
        full = x.new_empty((x.shape[0] * n, x.shape[1]))
        pg.all_gather_tensor(full, x.contiguous())
        dw = dy.t() @ full
        dfull = (dy @ w).contiguous()
        dx = torch.empty_like(x)
        pg.reduce_scatter_tensor(dx, dfull, "sum")
        return dx, dw, None


class _MatmulRingReduceScatter(torch.autograd.Function):
    """y = reduce_scatter_rows(a @ w.T): each step adds the local chunk product to the incoming
    accumulator and forwards it; after tp-1 hops every rank holds its fully reduced row block."""

    @staticmethod
    def forward(ctx, a, w, pg):
        n, r = pg.size(), pg.rank()
        rows = a.shape[0] // n
        acc = None
        for s in range(n):
            blk = (r - s - 1) % n  # block whose accumulator is at this rank in step s
            part = a[blk * rows: (blk + 1) * rows] @ w.t()
            acc = part if acc is None else acc + part
            if s + 1 < n:
                nxt = torch.empty_like(acc)
                pg.send_recv(acc.contiguous(), (r + 1) % n, nxt, (r - 1) % n, tag=400 + s)
                acc = nxt
        ctx.save_for_backward(a, w)
        ctx.pg = pg
        return acc

    @staticmethod
    def backward(ctx, dy):
        a, w = ctx.saved_tensors
        pg = ctx.pg
        n = pg.size()
        full = dy.new_empty((dy.shape[0] * n, dy.shape[1]))
        pg.all_gather_tensor(full, dy.contiguous())
        return full @ w, full.t() @ a, None


# --------------------------------------------------------------------------- vocab-parallel CE
class _VocabParallelCE(torch.autograd.Function):
    """Sum over rows of -log softmax(target) with the vocabulary split over ``pg``; rows whose target
    is ``ignore`` contribute zero.  logits [N, V/tp] local; ``lo`` = first vocabulary id of this rank."""

    @staticmethod
    def forward(ctx, logits, targets, pg, lo, vocab, ignore):
        lf = logits.float()
        Vl = lf.shape[1]
        col = torch.arange(Vl, device=lf.device) + lo
        lf = lf.masked_fill(col[None] >= vocab, float("-inf"))
        mx = lf.max(-1).values
        if pg is not None and pg.size() > 1:
            pg.all_reduce_tensor(mx, "max")
        e = torch.exp(lf - mx[:, None])
        local_t = targets - lo
        mine = (local_t >= 0) & (local_t < Vl)
        tl = torch.where(mine, lf.gather(1, local_t.clamp(0, Vl - 1)[:, None])[:, 0], torch.zeros_like(mx))
        st = torch.cat([e.sum(-1), tl])
        if pg is not None and pg.size() > 1:
            pg.all_reduce_tensor(st, "sum")
        N = lf.shape[0]
        sumexp, tlogit = st[:N], st[N:]
        valid = targets != ignore
        loss_rows = (mx + torch.log(sumexp) - tlogit) * valid
        ctx.save_for_backward(e / sumexp[:, None], local_t, mine & valid, valid)
        return loss_rows.sum()

    @staticmethod
    def backward(ctx, dl):
        p, local_t, mine, valid = ctx.saved_tensors
        g = p * valid[:, None]
        idx = local_t.clamp(0, p.shape[1] - 1)
        g[torch.arange(p.shape[0], device=p.device)[mine], idx[mine]] -= 1.0
        return g * dl, None, None, None, None, None


# ------------------------------------------------------------------------------------- engine
class ParallelLm:
    def __init__(self, model, pg, cfg: ParallelConfig, device=None, compute_dtype: Optional[torch.dtype] = None):
        """``device``: where this rank's parameter slices, optimizer state and activations live (default: CPU).
        ``compute_dtype``: dtype of activations and of the weights as the GEMMs see them (default: FP32); the FP32
        slices stay the master copy that AdamW updates.  On a CUDA device the linear layers run on the tcgen05 GEMM
        kernels (``fused_linear``; block-scaled FP8 under ``fused.ops.linear_precision("mxfp8")``)."""
        self.cfg, self.pg = cfg, pg
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.cd = compute_dtype or torch.float32
        if cfg.world() != pg.size():
            raise ValueError(f"dp*pp*cp*tp = {cfg.world()} but the group has {pg.size()} ranks")
        mc: LmConfig = model.config
        self.mc = mc
        if mc.moe_experts > 0 or not mc.prenorm or mc.parallel_block:
            raise ValueError("ParallelLm supports dense pre-norm sequential blocks")
        if mc.n_head % cfg.tp or mc.kv_heads() % cfg.tp or mc.d_ff % cfg.tp:
            raise ValueError("heads, kv heads and d_ff must be divisible by tp")
        if cfg.cp > 1 and cfg.cp_algorithm == "ulysses" and ((mc.n_head // cfg.tp) % cfg.cp or (mc.kv_heads() // cfg.tp) % cfg.cp):
            raise ValueError("ulysses needs (heads / tp) divisible by cp")
        self.mesh = DeviceMesh(pg, (cfg.dp, cfg.pp, cfg.cp, cfg.tp), ("dp", "pp", "cp", "tp"))
        self.tp_g, self.cp_g, self.dp_g = self.mesh.group("tp"), self.mesh.group("cp"), self.mesh.group("dp")
        self.dpcp_g = self.mesh.flatten(["dp", "cp"])
        self.tppp_g = self.mesh.flatten(["pp", "tp"])
        self.tp_r, self.cp_r, self.pp_r, self.dp_r = (self.mesh.index(n) for n in ("tp", "cp", "pp", "dp"))
        self.pp_g = self.mesh.group("pp")
        # context parallelism on GPUs: symmetric workspace over the cp group for the peer-memory attention paths
        self._cp_ws = None
        if cfg.cp > 1 and self.device.type == "cuda" and cfg.cp_comm == "fused" and mc.window <= 0 and \
                self.cd == torch.bfloat16 and hasattr(self.cp_g, "dist"):      # a torch (NCCL) process group
            from .symm import SymmetricWorkspace
            self._cp_ws = SymmetricWorkspace(self.cp_g)
        # embedding group {first, last} pipeline stage for the tied weight
        self.tie_g = None
        if cfg.pp > 1 and mc.tie_embeddings:
            self.tie_g = self.pp_g.new_group([0, cfg.pp - 1]) if self.pp_g is not None else None
        nchunks = cfg.pp * cfg.virtual_stages
        if nchunks > mc.n_layer:
            raise ValueError("more pipeline chunks than layers")
        self.ranges = balance_partition([1.0] * mc.n_layer, nchunks)
        self.my_chunks = [g for g in range(nchunks) if g % cfg.pp == self.pp_r]
        self.nchunks = nchunks
        self.Vp = (mc.padded_vocab() + cfg.tp - 1) // cfg.tp * cfg.tp
        self.params: Dict[str, torch.nn.Parameter] = {}
        self.kind: Dict[str, str] = {}   # "sharded" (tp-split) | "replicated"
        self._slice_model(model)
        self.rope = RopeCache(mc) if mc.pos == "rope" else None
        if self.rope is not None and self.device.type != "cpu":
            self.rope.to(self.device)
        self.names = list(self.params.keys())
        self.m = {n: torch.zeros_like(p) for n, p in self.params.items()}
        self.v = {n: torch.zeros_like(p) for n, p in self.params.items()}
        self.steps = 0
        self.stats = ParallelStepStats()
        self._zero_shards = None
        self._sends = []

    # ------------------------------------------------------------------------------- slicing
    def _add(self, name: str, t: torch.Tensor, kind: str) -> None:
        self.params[name] = torch.nn.Parameter(t.detach().to(device=self.device, dtype=torch.float32, copy=True))
        self.kind[name] = kind

    def _slice_model(self, model) -> None:
        mc, tp, r = self.mc, self.cfg.tp, self.tp_r
        H, Hk, D, Fd = mc.n_head, mc.kv_heads(), mc.hdim(), mc.d_ff
        first = 0 in self.my_chunks
        last = (self.nchunks - 1) in self.my_chunks
        sd = {n: p.detach() for n, p in model.named_parameters()}
        wdev = sd["wte"].device
        Vl = self.Vp // tp
        if first or (last and mc.tie_embeddings):
            w = torch.zeros(self.Vp, mc.d_model, device=wdev, dtype=sd["wte"].dtype)
            w[: sd["wte"].shape[0]] = sd["wte"]
            self._add("wte", w[r * Vl: (r + 1) * Vl], "sharded")
        if first and mc.pos == "learned":
            self._add("wpe", sd["wpe"], "replicated")
        for g in self.my_chunks:
            lo, hi = self.ranges[g]
            for l in range(lo, hi):
                p = f"h.{l}."
                for nm in ("norm1", "norm2"):
                    self._add(p + nm + ".weight", sd[p + nm + ".weight"], "replicated")
                    if p + nm + ".bias" in sd:
                        self._add(p + nm + ".bias", sd[p + nm + ".bias"], "replicated")
                wq = sd[p + "attn.qkv.weight"]
                q, k, v = wq[: H * D], wq[H * D: (H + Hk) * D], wq[(H + Hk) * D:]
                hq, hk = H // tp * D, Hk // tp * D
                self._add(p + "attn.qkv.weight", torch.cat([q[r * hq: (r + 1) * hq], k[r * hk: (r + 1) * hk],
                                                             v[r * hk: (r + 1) * hk]]), "sharded")
                if p + "attn.qkv.bias" in sd:
                    b = sd[p + "attn.qkv.bias"]
                    bq, bk, bv = b[: H * D], b[H * D: (H + Hk) * D], b[(H + Hk) * D:]
                    self._add(p + "attn.qkv.bias", torch.cat([bq[r * hq: (r + 1) * hq], bk[r * hk: (r + 1) * hk],
                                                               bv[r * hk: (r + 1) * hk]]), "sharded")
                self._add(p + "attn.o.weight", sd[p + "attn.o.weight"][:, r * hq: (r + 1) * hq], "sharded")
                if p + "attn.o.bias" in sd:
                    self._add(p + "attn.o.bias", sd[p + "attn.o.bias"], "replicated")
                up = sd[p + "mlp.up.weight"]
                fl = Fd // tp
                if mc.gated_mlp():
                    self._add(p + "mlp.up.weight", torch.cat([up[:Fd][r * fl: (r + 1) * fl], up[Fd:][r * fl: (r + 1) * fl]]), "sharded")
                else:
                    self._add(p + "mlp.up.weight", up[r * fl: (r + 1) * fl], "sharded")
                if p + "mlp.up.bias" in sd:
                    ub = sd[p + "mlp.up.bias"]
                    if mc.gated_mlp():
                        self._add(p + "mlp.up.bias", torch.cat([ub[:Fd][r * fl: (r + 1) * fl], ub[Fd:][r * fl: (r + 1) * fl]]), "sharded")
                    else:
                        self._add(p + "mlp.up.bias", ub[r * fl: (r + 1) * fl], "sharded")
                self._add(p + "mlp.down.weight", sd[p + "mlp.down.weight"][:, r * fl: (r + 1) * fl], "sharded")
                if p + "mlp.down.bias" in sd:
                    self._add(p + "mlp.down.bias", sd[p + "mlp.down.bias"], "replicated")
        if last:
            self._add("norm_f.weight", sd["norm_f.weight"], "replicated")
            if "norm_f.bias" in sd:
                self._add("norm_f.bias", sd["norm_f.bias"], "replicated")
            if not mc.tie_embeddings:
                w = torch.zeros(self.Vp, mc.d_model, device=wdev, dtype=sd["lm_head"].dtype)
                w[: sd["lm_head"].shape[0]] = sd["lm_head"]
                self._add("lm_head", w[r * Vl: (r + 1) * Vl], "sharded")

    # ------------------------------------------------------------------------------ forward
    def _norm(self, x, prefix):
        w = self.params[prefix + ".weight"]
        b = self.params.get(prefix + ".bias")
        if self.mc.norm == "rmsnorm":
            return F_.rms_norm(x, w, self.mc.norm_eps)
        return F_.fused_layernorm(x, w, b, self.mc.norm_eps)

    def _w(self, w):
        """The weight as the GEMM sees it: the FP32 master slice cast to the compute dtype (the cast is part of the
        graph, so the gradient arrives in FP32)."""
        return w if w.dtype == self.cd else w.to(self.cd)

    def _col_linear(self, h, w, b):
        """Column-parallel linear on the region input (replicated, or token-sharded under SP)."""
        w = self._w(w)
        if self.cfg.sp and self.cfg.tp > 1:
            if self.cfg.async_tp:
                y = _RingAllGatherMatmul.apply(h, w, self.tp_g)
            else:
                y = F_.fused_linear(C.all_gather_rows(h, self.tp_g), w)
        else:
            y = F_.fused_linear(C.copy_to_group(h, self.tp_g), w)
        return y if b is None else y + b.to(y.dtype)

    def _row_linear(self, a, w, b):
        """Row-parallel linear back into the region output."""
        w = self._w(w)
        if self.cfg.sp and self.cfg.tp > 1:
            y = _MatmulRingReduceScatter.apply(a, w, self.tp_g) if self.cfg.async_tp else \
                C.reduce_scatter_rows(F_.fused_linear(a, w), self.tp_g)
        else:
            y = C.all_reduce(F_.fused_linear(a, w), self.tp_g)
        return y if b is None else y + b.to(y.dtype)

    def _block(self, x, l: int, B: int, Tl: int, positions):
        mc, tp = self.mc, self.cfg.tp
        p = f"h.{l}."
        H, Hk, D = mc.n_head // tp, mc.kv_heads() // tp, mc.hdim()
        h = self._norm(x, p + "norm1")
        qkv = self._col_linear(h, self.params[p + "attn.qkv.weight"], self.params.get(p + "attn.qkv.bias"))
        qkv = qkv.view(B, Tl, (H + 2 * Hk) * D)
        q = qkv[..., : H * D].reshape(B, Tl, H, D)
        k = qkv[..., H * D: (H + Hk) * D].reshape(B, Tl, Hk, D)
        v = qkv[..., (H + Hk) * D:].reshape(B, Tl, Hk, D)
        if self.rope is not None:
            q = apply_rope(q, self.rope.cos, self.rope.sin, positions)
            k = apply_rope(k, self.rope.cos, self.rope.sin, positions)
        if self.cfg.cp > 1 and self._cp_ws is not None:
            from . import symm
            if self.cfg.cp_algorithm == "ulysses":
                a = symm.ulysses_attention(self._cp_ws, q, k, v, causal=True)
            else:
                a = symm.ring_attention_autograd(self._cp_ws, q, k, v, layout=self.cfg.cp_layout, causal=True)
        elif self.cfg.cp > 1:
            if self.cfg.cp_algorithm == "ulysses":
                a = ulysses_attention(q, k, v, self.cp_g)
            else:
                a = ring_attention(q, k, v, self.cp_g, self.cfg.cp_layout)
        else:
            a = F_.attention(q, k, v, causal=True, window=mc.window)
        a = a.reshape(B * Tl, H * D)
        x = x + self._row_linear(a, self.params[p + "attn.o.weight"], self.params.get(p + "attn.o.bias"))
        h = self._norm(x, p + "norm2")
        u = self._col_linear(h, self.params[p + "mlp.up.weight"], self.params.get(p + "mlp.up.bias"))
        if mc.mlp == "gelu":
            act = F_.gelu_tanh(u)
        else:
            act = F_.gated_activation(u, "swiglu" if mc.mlp == "swiglu" else "geglu")
        return x + self._row_linear(act, self.params[p + "mlp.down.weight"], self.params.get(p + "mlp.down.bias"))

    def _embed(self, tokens, positions):
        tp, r = self.cfg.tp, self.tp_r
        Vl = self.Vp // tp
        ids = tokens.reshape(-1).long() - r * Vl
        ok = (ids >= 0) & (ids < Vl)
        x = (self.params["wte"][ids.clamp(0, Vl - 1)] * ok[:, None]).to(self.cd)
        if self.mc.pos == "learned":
            # added once (not once per tp rank): only tp rank 0 contributes before the reduction
            pe = self.params["wpe"][positions.reshape(-1)]
            x = x + (pe if r == 0 else torch.zeros_like(pe)).to(self.cd)
        if self.cfg.sp and tp > 1:
            return C.reduce_scatter_rows(x, self.tp_g)
        return C.all_reduce(x, self.tp_g)

    def _head_loss(self, x, targets):
        """x region output -> summed next-token loss over the local tokens."""
        h = self._norm(x, "norm_f")
        if self.cfg.sp and self.cfg.tp > 1:
            h = C.all_gather_rows(h, self.tp_g)
        else:
            h = C.copy_to_group(h, self.tp_g)
        w = self.params["wte"] if self.mc.tie_embeddings else self.params["lm_head"]
        logits = F_.fused_linear(h, self._w(w)).float()
        return _VocabParallelCE.apply(logits, targets.reshape(-1), self.tp_g, self.tp_r * (self.Vp // self.cfg.tp),
                                      self.mc.vocab_size, -100)

    def _run_chunk(self, g: int, x, tokens, positions, targets, B, Tl):
        if g == 0:
            x = self._embed(tokens, positions)
        lo, hi = self.ranges[g]
        for l in range(lo, hi):
            x = self._block(x, l, B, Tl, positions)
        if g == self.nchunks - 1:
            return self._head_loss(x, targets)
        return x

    # ------------------------------------------------------------------------------ data prep
    def _prepare(self, tokens: torch.Tensor):
        """Shard one micro-batch over cp: local tokens, global positions, shifted targets."""
        B, T = tokens.shape
        tg = torch.full_like(tokens, -100, dtype=torch.long)
        tg[:, :-1] = tokens[:, 1:].long()
        pos = torch.arange(T, device=tokens.device)[None].expand(B, T)
        cp = self.cfg.cp
        if cp > 1:
            layout = "contiguous" if self.cfg.cp_algorithm == "ulysses" else self.cfg.cp_layout
            tokens = shard_sequence(tokens, cp, self.cp_r, layout)
            tg = shard_sequence(tg, cp, self.cp_r, layout)
            pos = shard_sequence(pos, cp, self.cp_r, layout)
        return tokens.contiguous(), pos.contiguous(), tg.contiguous()

    # ------------------------------------------------------------------- pipeline executor
    def _region_rows(self, B, Tl):
        n = B * Tl
        return n // self.cfg.tp if (self.cfg.sp and self.cfg.tp > 1) else n

    def forward_backward(self, micro: List[torch.Tensor], weights: Optional[List[float]] = None) -> float:
        """Runs every micro-batch through the pipeline schedule; gradients accumulate into ``.grad``.
        ``weights[i]`` scales micro-batch i (token-weighted accumulation); the loss of a micro-batch is
        its summed token loss divided by its global number of valid targets."""
        cfg = self.cfg
        m = len(micro)
        weights = weights or [1.0 / m] * m
        acts = make_schedule(cfg.pp_schedule, cfg.pp, self.pp_r, m, cfg.virtual_stages)
        self.stats = ParallelStepStats(bubble_theory=theoretical_bubble(cfg.pp_schedule, cfg.pp, m, cfg.virtual_stages))
        prep = [self._prepare(t) for t in micro]
        B, Tl = prep[0][0].shape
        rows, d = self._region_rows(B, Tl), self.mc.d_model
        valid = [max(1, int((t.shape[0]) * (t.shape[1] - 1))) for t in micro]
        saved: Dict[Tuple[int, int], Tuple] = {}
        pending_w: List[Tuple] = []
        split_w = cfg.pp_schedule == "zb_h1"
        total_loss = 0.0
        params = [p for p in self.params.values()]

        def run_w(entry):
            out, gout, inp = entry
            grads = torch.autograd.grad(out, params, gout, allow_unused=True)
            for p, g in zip(params, grads):
                if g is not None:
                    p.grad = g if p.grad is None else p.grad + g

        for a in acts:
            g, mb = a.chunk, a.mb
            tok, pos, tg = prep[mb]
            prev_rank, next_rank = (g - 1) % cfg.pp, (g + 1) % cfg.pp
            if a.kind == "F":
                x_in = None
                if g > 0:
                    x_in = torch.empty(rows, d, device=self.device, dtype=self.cd)
                    self._p2p_recv(x_in, prev_rank, tag=1000 + mb * 64 + g)
                    x_in.requires_grad_(True)
                out = self._run_chunk(g, x_in, tok, pos, tg, B, Tl)
                if g == self.nchunks - 1:
                    out = out / valid[mb]
                    total_loss += float(out.detach()) * weights[mb]
                else:
                    self._p2p_send(out.detach(), next_rank, tag=1000 + mb * 64 + g + 1)
                saved[(mb, g)] = (x_in, out)
            else:  # B
                x_in, out = saved.pop((mb, g))
                if g == self.nchunks - 1:
                    gout = torch.tensor(weights[mb], dtype=out.dtype, device=out.device)
                else:
                    gout = torch.empty(rows, d, device=self.device, dtype=self.cd)
                    self._p2p_recv(gout, next_rank, tag=5000 + mb * 64 + g)
                if split_w:
                    if x_in is not None:
                        (gx,) = torch.autograd.grad(out, [x_in], gout, retain_graph=True)
                        self._p2p_send(gx, prev_rank, tag=5000 + mb * 64 + g - 1)
                    pending_w.append((out, gout, x_in))
                    while len(pending_w) > cfg.pp - self.pp_r:
                        run_w(pending_w.pop(0))
                else:
                    torch.autograd.backward([out], [gout])
                    if x_in is not None:
                        self._p2p_send(x_in.grad, prev_rank, tag=5000 + mb * 64 + g - 1)
        for e in pending_w:
            run_w(e)
        for w, _ in self._sends:
            w.wait()
        self._sends = []
        self._sync_grads()
        # loss: sum over cp shards, known on the last stage -> broadcast over pp
        lt = torch.tensor([total_loss], dtype=torch.float64, device=self.device)
        if self.cp_g is not None:
            self.cp_g.all_reduce_tensor(lt, "sum")
        if self.pp_g is not None:
            self.pp_g.broadcast_tensor(lt, cfg.pp - 1)
        self.local_loss = float(lt)          # this data-parallel replica's share
        if self.dp_g is not None:
            self.dp_g.all_reduce_tensor(lt, "sum")
        self.stats.loss = float(lt)
        return self.stats.loss

    def _p2p_send(self, t, dst, tag):
        if hasattr(self.pp_g, "isend"):
            self._sends.append((self.pp_g.isend(t.contiguous(), dst, tag), t))  # keep the buffer alive
        else:
            self.pp_g.send(t.contiguous(), dst, tag)
        self.stats.p2p_messages += 1
        self.stats.p2p_bytes += t.numel() * 4

    def _p2p_recv(self, t, src, tag):
        self.pp_g.recv(t, src, tag)

    # ------------------------------------------------------------------------------ grad sync
    def _sync_grads(self) -> None:
        cfg = self.cfg
        for n, p in self.params.items():
            if p.grad is None:
                p.grad = torch.zeros_like(p)
        # replicated parameters inside a token-sharded (SP) region saw only their tokens
        if cfg.sp and cfg.tp > 1:
            for n, p in self.params.items():
                if self.kind[n] == "replicated" and n != "wpe":
                    self.tp_g.all_reduce_tensor(p.grad, "sum")
        elif cfg.tp > 1:
            pass  # copy_to_group / all_reduce already produced full gradients for replicated parameters
        if cfg.tp > 1 and "wpe" in self.params and not cfg.sp:
            # wpe was added on tp rank 0 only; its gradient is complete there: share it
            self.tp_g.broadcast_tensor(self.params["wpe"].grad, 0)
        if cfg.tp > 1 and "wpe" in self.params and cfg.sp:
            self.tp_g.all_reduce_tensor(self.params["wpe"].grad, "sum")
        if self.tie_g is not None and "wte" in self.params:
            self.tie_g.all_reduce_tensor(self.params["wte"].grad, "sum")
        if self.dpcp_g is not None:
            flat = torch.cat([p.grad.reshape(-1) for p in self.params.values()])
            n = self.dpcp_g.size()
            pad = (-flat.numel()) % n
            if pad:
                flat = torch.cat([flat, flat.new_zeros(pad)])
            shard = torch.empty(flat.numel() // n, device=flat.device, dtype=flat.dtype)
            self.dpcp_g.reduce_scatter_tensor(shard, flat, "sum")
            self.dpcp_g.all_gather_tensor(flat, shard)
            off = 0
            for p in self.params.values():
                p.grad.copy_(flat[off: off + p.numel()].view(p.shape))
                off += p.numel()

    # ------------------------------------------------------------------------------ optimizer
    def grad_norm(self) -> float:
        """Global norm: sharded parameters count on every tp rank, replicated ones once; summed over pp."""
        sq = 0.0
        for n, p in self.params.items():
            s = float(p.grad.double().pow(2).sum())
            if self.kind[n] == "replicated" and self.tp_r != 0:
                s = 0.0
            if n == "wte" and self.tie_g is not None and self.pp_r != 0:
                s = 0.0  # the tied table lives on two stages: count it once
            sq += s
        t = torch.tensor([sq], dtype=torch.float64, device=self.device)
        if self.tppp_g is not None:
            self.tppp_g.all_reduce_tensor(t, "sum")
        return math.sqrt(float(t))

    def step(self, opt, lr: float, clip: float = 0.0, wd_rule=None) -> float:
        norm = self.grad_norm()
        self.stats.grad_norm = norm
        if not math.isfinite(norm):
            self.zero_grad()
            return norm
        self.steps += 1
        names = self.names
        wd = [(1.0 if self.params[n].dim() >= 2 else 0.0) if wd_rule is None else wd_rule(n, self.params[n]) for n in names]
        if self.cfg.zero >= 1 and self.dpcp_g is not None:
            self._zero1_step(opt, lr, clip, wd, norm)
        else:
            F_.adamw_multi_tensor([self.params[n].data for n in names], [self.params[n].grad for n in names],
                                  [self.m[n] for n in names], [self.v[n] for n in names], self.steps, lr, opt.beta1,
                                  opt.beta2, opt.eps, opt.weight_decay, clip, wd, None, grad_sq_sum=norm * norm)
        self.zero_grad()
        return norm

    def _zero1_step(self, opt, lr, clip, wd, norm) -> None:
        """AdamW state sharded over dp x cp: each rank updates 1/n of the flat parameter vector and
        the updated parameters are all-gathered."""
        g = self.dpcp_g
        n, r = g.size(), g.rank()
        names = self.names
        flat_p = torch.cat([self.params[x].data.reshape(-1) for x in names])
        flat_g = torch.cat([self.params[x].grad.reshape(-1) for x in names])
        flat_wd = torch.cat([torch.full((self.params[x].numel(),), w, device=self.device) for x, w in zip(names, wd)])
        pad = (-flat_p.numel()) % n
        if pad:
            flat_p, flat_g, flat_wd = (torch.cat([t, t.new_zeros(pad)]) for t in (flat_p, flat_g, flat_wd))
        S = flat_p.numel() // n
        if self._zero_shards is None:
            self._zero_shards = (torch.zeros(S, device=self.device), torch.zeros(S, device=self.device))
        ms, vs = self._zero_shards
        sl = slice(r * S, (r + 1) * S)
        ps, gs, ws = flat_p[sl].clone(), flat_g[sl], flat_wd[sl]
        # decay / no-decay segments of the shard
        for val in (1.0, 0.0):
            idx = (ws == val).nonzero()[:, 0]
            if idx.numel() == 0:
                continue
            pp, mm, vv = ps[idx], ms[idx], vs[idx]
            F_.adamw_multi_tensor([pp], [gs[idx]], [mm], [vv], self.steps, lr, opt.beta1, opt.beta2, opt.eps,
                                  opt.weight_decay, clip, [val], None, grad_sq_sum=norm * norm)
            ps[idx], ms[idx], vs[idx] = pp, mm, vv
        g.all_gather_tensor(flat_p, ps)
        off = 0
        for x in names:
            p = self.params[x]
            p.data.copy_(flat_p[off: off + p.numel()].view(p.shape))
            off += p.numel()

    def zero_grad(self) -> None:
        for p in self.params.values():
            p.grad = None

    @torch.no_grad()
    def eval_loss(self, tokens: torch.Tensor) -> float:
        if self.cfg.pp > 1:
            raise RuntimeError("eval_loss with pp > 1: use forward_backward on a no-grad copy")
        tok, pos, tg = self._prepare(tokens)
        B, Tl = tok.shape
        loss = self._run_chunk(0, None, tok, pos, tg, B, Tl) if self.nchunks == 1 else None
        t = torch.tensor([float(loss)], dtype=torch.float64, device=self.device)
        if self.cp_g is not None:
            self.cp_g.all_reduce_tensor(t, "sum")
        return float(t) / max(1, tokens.shape[0] * (tokens.shape[1] - 1))

    # ---------------------------------------------------------------------------- test helper
    def assemble_full(self, what: str = "param") -> Dict[str, torch.Tensor]:
        """Gathers every tensor (or its gradient) over tp; each pipeline stage returns its own layers."""
        tp = self.cfg.tp
        mc = self.mc
        H, Hk, D, Fd = mc.n_head, mc.kv_heads(), mc.hdim(), mc.d_ff
        out = {}
        for n, p in self.params.items():
            t = (p.grad if what == "grad" else p.data).detach().clone()
            if self.kind[n] == "replicated" or tp == 1:
                out[n] = t
                continue
            parts = [torch.empty_like(t) for _ in range(tp)]
            buf = torch.empty((tp,) + tuple(t.shape))
            self.tp_g.all_gather_tensor(buf, t.contiguous())
            parts = list(buf)
            if n.endswith("attn.qkv.weight") or n.endswith("attn.qkv.bias"):
                hq, hk = H // tp * D, Hk // tp * D
                out[n] = torch.cat([torch.cat([x[:hq] for x in parts]), torch.cat([x[hq: hq + hk] for x in parts]),
                                    torch.cat([x[hq + hk:] for x in parts])])
            elif n.endswith("attn.o.weight") or n.endswith("mlp.down.weight"):
                out[n] = torch.cat(parts, dim=1)
            elif (n.endswith("mlp.up.weight") or n.endswith("mlp.up.bias")) and mc.gated_mlp():
                fl = Fd // tp
                out[n] = torch.cat([torch.cat([x[:fl] for x in parts]), torch.cat([x[fl:] for x in parts])])
            else:
                out[n] = torch.cat(parts, dim=0)
        return out

    # ------------------------------------------------------------------------------ persistence
    def save_state(self) -> bytes:
        buf = io.BytesIO()
        torch.save({"params": {n: p.data for n, p in self.params.items()}, "m": self.m, "v": self.v,
                    "steps": self.steps, "zero": self._zero_shards}, buf)
        return buf.getvalue()

    def load_state(self, blob: bytes) -> None:
        d = torch.load(io.BytesIO(blob), map_location="cpu")
        for n, p in self.params.items():
            p.data.copy_(d["params"][n])
            self.m[n].copy_(d["m"][n])
            self.v[n].copy_(d["v"][n])
        self.steps = d["steps"]
        self._zero_shards = d["zero"]
