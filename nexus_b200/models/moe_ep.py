"""Mixture-of-experts decoder trained with expert parallelism over the GPUs of one node.

Every rank holds its own sequences (data parallel for attention, norms, embeddings and the routers) and 1 / n of the
experts of every layer.  Routed rows travel through the peer-memory dispatch / combine kernels of
`moe.ep_gpu.MoeEpLayer`; the replicated gradients are summed by the fused peer-memory all-reduce (BF16 in, FP32 out,
the cast inside the reduction); the global gradient norm is exchanged by the kernel the sharded optimizer uses; AdamW
runs as the multi-tensor kernel on flat FP32 masters with BF16 working copies.  Layers are RMSNorm -> attention
(rotary, flash kernels) -> RMSNorm -> top-k SwiGLU MoE; untied LM head; loss = next-token cross-entropy + the
load-balancing auxiliary loss.

Parity (behaviour): MoeExpertParallel training of the reference (include/nexus/dist/moe_ep.hpp, src/dist/moe_ep.cpp:45-90,
the `moe-*` presets of src/lm/config.cpp), which runs FP32 on CPU ranks there.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional

import torch
import torch.nn as nn

from ..fused import ops as F_
from ..lm.config import LmConfig
from ..lm.rope import RopeCache
from ..moe.ep_gpu import EpContext, MoeEpLayer
from ..ops import _cuda as K
from ..ops import _infer as KI
from .gpt import AdamWConfig


class _Rope(torch.autograd.Function):
    """In-place rotary embedding kernel on q / k views [rows, heads, D]; the backward is the inverse rotation."""

    @staticmethod
    def forward(ctx, x, positions, cos, sin):
        ctx.save_for_backward(positions, cos, sin)
        y = x.contiguous().clone()
        KI.rope_(y.view(-1, y.shape[-2], y.shape[-1]), positions, cos, sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        positions, cos, sin = ctx.saved_tensors
        g = dy.contiguous().clone()
        KI.rope_(g.view(-1, g.shape[-2], g.shape[-1]), positions, cos, sin, inverse=True)
        return g, None, None, None


class _Block(nn.Module):
    def __init__(self, cfg: LmConfig, layer: int, ep: EpContext, gen: torch.Generator, device):
        super().__init__()
        H, Hk, D, d = cfg.n_head, cfg.kv_heads(), cfg.hdim(), cfg.d_model
        bf = torch.bfloat16

        def mat(rows, cols, std):
            return nn.Parameter((torch.randn(rows, cols, generator=gen) * std).to(device, bf))

        self.norm1 = nn.Parameter(torch.ones(d, device=device, dtype=bf))
        self.qkv = mat((H + 2 * Hk) * D, d, cfg.init_std)
        self.o = mat(d, H * D, cfg.init_std / math.sqrt(2 * cfg.n_layer))
        self.norm2 = nn.Parameter(torch.ones(d, device=device, dtype=bf))
        self.moe = MoeEpLayer(ep, cfg.expert_ff(), cfg.moe_aux_alpha, cfg.init_std, cfg.seed + 101 * layer)
        self.cfg = cfg

    def forward(self, x, positions, rope: RopeCache):
        cfg = self.cfg
        B, T, d = x.shape
        H, Hk, D = cfg.n_head, cfg.kv_heads(), cfg.hdim()
        h = F_.rms_norm(x, self.norm1, cfg.norm_eps)
        qkv = F_.fused_linear(h, self.qkv)
        q = _Rope.apply(qkv[..., : H * D].reshape(B, T, H, D), positions, rope.cos, rope.sin)
        k = _Rope.apply(qkv[..., H * D: (H + Hk) * D].reshape(B, T, Hk, D), positions, rope.cos, rope.sin)
        v = qkv[..., (H + Hk) * D:].reshape(B, T, Hk, D)
        o = F_.attention(q, k, v, causal=True)
        x = x + F_.fused_linear(o.reshape(B, T, H * D), self.o)
        h = F_.rms_norm(x, self.norm2, cfg.norm_eps)
        y, aux = self.moe(h.reshape(B * T, d))
        return x + y.view(B, T, d), aux


class MoeEpDecoder(nn.Module):
    def __init__(self, cfg: LmConfig, pg=None, device="cuda", micro_batch: int = 1, seq_len: int = 0):
        super().__init__()
        if cfg.moe_experts <= 0 or cfg.norm != "rmsnorm" or cfg.pos != "rope" or cfg.bias or cfg.tie_embeddings:
            raise ValueError("MoeEpDecoder: an MoE configuration with RMSNorm, RoPE, an untied head and no biases")
        if cfg.moe_every != 1 or cfg.moe_shared_expert or cfg.moe_reroute or cfg.moe_groups != 1 or cfg.moe_noisy:
            raise ValueError("MoeEpDecoder: every layer is a plain top-k MoE layer with the drop policy")
        self.cfg, self.pg = cfg, pg
        self.dev = torch.device(device)
        T = seq_len or cfg.max_position
        self.ep = EpContext(pg, cfg.moe_experts, cfg.d_model, micro_batch * T, cfg.moe_top_k, cfg.moe_capacity_factor,
                            self.dev, cfg.moe_min_capacity)
        g = torch.Generator(device="cpu").manual_seed(cfg.seed)      # the same stream on every rank: replicas agree
        bf = torch.bfloat16
        V, d = cfg.padded_vocab(), cfg.d_model
        self.wte = nn.Parameter((torch.randn(V, d, generator=g) * cfg.init_std).to(self.dev, bf))
        self.blocks = nn.ModuleList([_Block(cfg, l, self.ep, g, self.dev) for l in range(cfg.n_layer)])
        self.normf = nn.Parameter(torch.ones(d, device=self.dev, dtype=bf))
        self.head = nn.Parameter((torch.randn(V, d, generator=g) * cfg.init_std).to(self.dev, bf))
        self.rope = RopeCache(cfg, device=self.dev, seq_len=T)
        self._positions = None

    def expert_parameters(self) -> List[nn.Parameter]:
        return [p for b in self.blocks for p in (b.moe.up, b.moe.down)]

    def replicated_parameters(self) -> List[nn.Parameter]:
        mine = {id(p) for p in self.expert_parameters()}
        return [p for p in self.parameters() if id(p) not in mine]

    def loss(self, tokens: torch.Tensor):
        """tokens [B, T] int32/int64 (this rank's sequences).  Returns (cross-entropy, auxiliary loss)."""
        B, T = tokens.shape
        if self._positions is None or self._positions.numel() != B * T:
            self._positions = torch.arange(T, dtype=torch.int32, device=self.dev).repeat(B)
        x = self.wte[tokens.long()]
        aux_total = x.new_zeros((), dtype=torch.float32)
        for blk in self.blocks:
            x, aux = blk(x, self._positions, self.rope)
            aux_total = aux_total + aux
        h = F_.rms_norm(x, self.normf, self.cfg.norm_eps)
        logits = F_.fused_linear(h, self.head)
        ce = F_.cross_entropy_shifted(logits, tokens.to(torch.int32), vocab=self.cfg.vocab_size)
        return ce, aux_total

    def flops_per_token(self, T: int) -> float:
        """Active-parameter FLOPs: 6 x (attention + top-k experts + router + head) + attention scores."""
        c = self.cfg
        H, Hk, D, d, F = c.n_head, c.kv_heads(), c.hdim(), c.d_model, c.expert_ff()
        per_layer = (H + 2 * Hk) * D * d + d * H * D + c.moe_top_k * 3 * d * F + c.moe_experts * d
        return 6.0 * (c.n_layer * per_layer + c.padded_vocab() * d) + 12.0 * c.n_layer * H * D * T


class MoeEpTrainer:
    """Flat-buffer training state around a `MoeEpDecoder`: BF16 working weights and BF16 gradients live in two flat
    buffers (replicated / experts), FP32 masters and moments beside them; one optimizer step = backward, fused
    all-reduce of the replicated gradients, gradient-norm exchange, clip + AdamW kernels."""

    def __init__(self, model: MoeEpDecoder, opt: AdamWConfig):
        self.model, self.pg = model, model.pg
        self.n = self.pg.size() if self.pg is not None else 1
        dev = model.dev
        self.ws = model.ep.ws
        rep, exp = model.replicated_parameters(), model.expert_parameters()
        self.rep_count = self._total(rep)
        self.exp_count = self._total(exp)
        bf, f32 = torch.bfloat16, torch.float32
        if self.n > 1:
            self._g_src = self.ws.alloc(self.rep_count, bf)        # this rank's replicated gradients (BF16)
            self._g_dst = self.ws.alloc(self.rep_count, f32)       # their sum over the ranks (FP32)
            rep_grad_lp, self.rep_grad = self._g_src.local, self._g_dst.local
            rep_grad_lp.zero_()
            self.rep_grad.zero_()
        else:
            rep_grad_lp = torch.zeros(self.rep_count, dtype=bf, device=dev)
            self.rep_grad = rep_grad_lp
        self.rep_grad_lp = rep_grad_lp
        self.rep_lp = torch.zeros(self.rep_count, dtype=bf, device=dev)
        self.exp_lp = torch.zeros(self.exp_count, dtype=bf, device=dev)
        self.exp_grad = torch.zeros(self.exp_count, dtype=bf, device=dev)
        self.rep_chunks = self._bind(rep, self.rep_lp, rep_grad_lp)
        self.exp_chunks = self._bind(exp, self.exp_lp, self.exp_grad)
        self.rep_master, self.exp_master = self.rep_lp.float(), self.exp_lp.float()
        self.rep_m, self.rep_v = torch.zeros_like(self.rep_master), torch.zeros_like(self.rep_master)
        self.exp_m, self.exp_v = torch.zeros_like(self.exp_master), torch.zeros_like(self.exp_master)
        self.opt_state = K.opt_state_tensor(dev)
        raw = K.pack_opt_state(lr=opt.lr, weight_decay=opt.weight_decay, beta1=opt.beta1, beta2=opt.beta2, eps=opt.eps,
                               max_grad_norm=opt.grad_clip, loss_scale=1.0)
        self.opt_state.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
        self._parts = torch.zeros(2, dtype=torch.float64, device=dev)
        self.last_loss = torch.zeros(2, dtype=torch.float32, device=dev)

    @staticmethod
    def _total(params) -> int:
        off = 0
        for p in params:
            off = (off + 63) // 64 * 64 + p.numel()
        return (off + 63) // 64 * 64

    def _bind(self, params, flat_lp, flat_grad):
        """Re-points every parameter (and its gradient) at a 64-element-aligned view of the flat buffers."""
        segs, off = [], 0
        for p in params:
            off = (off + 63) // 64 * 64
            n = p.numel()
            flat_lp[off: off + n].copy_(p.data.reshape(-1))
            p.data = flat_lp[off: off + n].view(p.shape)
            p.grad = flat_grad[off: off + n].view(p.shape)
            segs.append((off, n, 1.0 if p.dim() >= 2 else 0.0, 1.0))
            off += n
        return K.make_chunks(segs, device=flat_lp.device)

    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """One optimizer step on this rank's ``tokens`` [B, T].  Returns a device tensor (cross-entropy, aux loss)."""
        return self.step_accumulate([tokens])

    def step_accumulate(self, micro_batches) -> torch.Tensor:
        """One optimizer step over several micro-batches (gradients accumulate in the flat BF16 buffers)."""
        m, n = self.model, self.n
        k = len(micro_batches)
        self.last_loss.zero_()
        for tokens in micro_batches:
            ce, aux = m.loss(tokens)
            ((ce + aux) / (n * k)).backward()    # the global loss is the mean over ranks and micro-batches
            self.last_loss[0].add_(ce.detach() / k)
            self.last_loss[1].add_(aux.detach() / k)
        off = K.OptState.local_sq.offset
        sq = self.opt_state[off: off + 8].view(torch.float64)
        if n > 1:
            from ..parallel.symm import fused_all_reduce
            fused_all_reduce(self.ws, self._g_src, self._g_dst, self.rep_count)
        K.grad_norm(self.rep_grad, self.opt_state, local_only=True)
        self._parts[0:1].copy_(sq)
        self._parts[0:1].div_(n)             # identical on every rank after the all-reduce: count it once
        K.grad_norm(self.exp_grad, self.opt_state, local_only=True)
        self._parts[1:2].copy_(sq)
        if n > 1:
            ws = self.ws
            K._check(K.lib().nx_comm_norm_exchange(K._p(self._parts), C.c_int(2), C.byref(ws.slots.table),
                                                   C.byref(ws.flags.table), C.c_int(ws.rank), C.c_int(n), K._p(ws.counter),
                                                   K._p(self.opt_state), K._p(K.status_word(m.dev)), K._stream()),
                     "nx_comm_norm_exchange")
        else:
            total = self._parts.sum().reshape(1)
            K.grad_norm(self.exp_grad, self.opt_state, extra_sq=total)
        K.adamw(self.rep_master, self.rep_grad, self.rep_m, self.rep_v, self.rep_lp, self.rep_chunks, self.opt_state,
                zero_grad=True)
        K.adamw(self.exp_master, self.exp_grad, self.exp_m, self.exp_v, self.exp_lp, self.exp_chunks, self.opt_state,
                zero_grad=True)
        if n > 1:
            self.rep_grad_lp.zero_()
        return self.last_loss

    def read_opt_state(self):
        return K.unpack_opt_state(bytes(self.opt_state.cpu().numpy().tobytes()))
