"""Config-driven decoder language model (GPT-2 / LLaMA / Mistral / Qwen2 / MoE families) on the fused
operators: every Linear / norm / attention / cross-entropy goes through :mod:`nexus_b200.fused.ops`,
so on CUDA BF16 it runs the sm_100a kernels and on CPU the PyTorch reference math.

Parameter names follow the reference (`wte`, `wpe`, `h{l}.norm1.weight`, `h{l}.attn.qkv.weight`,
`h{l}.attn.o.weight`, `h{l}.mlp.up.weight`, `h{l}.mlp.down.weight`, `norm_f.weight`,
`lm_head.weight`); weights are stored [out, in].

Parity: include/nexus/lm/model.hpp:14-224 and src/lm/model.cpp of the reference (`LanguageModel`:
logits/loss, named parameters, KV-cache incremental decode, NXS archive with embedded config).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..fused import ops as F_
from ..moe.moe import MoEFFN, Spec as MoeSpec
from .config import LmConfig, validate
from .rope import RopeCache, alibi_slopes, apply_rope


def _trunc_normal_(t: torch.Tensor, std: float, gen: torch.Generator, truncated: bool) -> None:
    with torch.no_grad():
        t.copy_(torch.randn(t.shape, generator=gen) * std)
        if truncated:
            bad = t.abs() > 2 * std
            while bad.any():
                t[bad] = (torch.randn(int(bad.sum()), generator=gen) * std)
                bad = t.abs() > 2 * std


class Norm(nn.Module):
    def __init__(self, cfg: LmConfig, dim: Optional[int] = None):
        super().__init__()
        d = dim or cfg.d_model
        self.rms = cfg.norm == "rmsnorm" or dim is not None
        self.eps = cfg.norm_eps
        self.weight = nn.Parameter(torch.ones(d))
        self.bias = nn.Parameter(torch.zeros(d)) if (not self.rms and cfg.bias) else None

    def forward(self, x):
        if self.rms:
            return F_.rms_norm(x, self.weight, self.eps)
        return F_.fused_layernorm(x, self.weight, self.bias, self.eps)


CPU_WEIGHT_MODES = ("auto", "f32", "bf16", "int8", "int4")


class Linear(nn.Module):
    def __init__(self, d_in: int, d_out: int, bias: bool):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(d_out, d_in))
        self.bias = nn.Parameter(torch.zeros(d_out)) if bias else None
        self._cpu_pack = None      # (mode, packed weights) after LanguageModel.prepare_cpu_inference

    def pack_for_cpu(self, mode: str) -> int:
        """Prepares the inference form of the weights on the CPU; returns the bytes it occupies."""
        from .. import cpu as _cpu
        w = self.weight.detach().float().cpu().numpy()
        if mode in ("auto", "f32"):
            self._cpu_pack = ("f32", w.copy())
            return w.nbytes
        if mode == "bf16":
            bits = _cpu.to_bf16_bits(w)
            self._cpu_pack = ("bf16", bits)
            return bits.nbytes
        bits_n = 8 if mode == "int8" else 4
        group = 32 if w.shape[1] % 32 == 0 else 0
        if bits_n == 4 and not group:
            raise ValueError("int4 CPU inference needs in-features divisible by 32")
        self._cpu_pack = (mode, _cpu.pack_weights(w, bits_n, group or 32))
        return w.size * bits_n // 8 + w.shape[0] * 4 * (1 if bits_n == 8 else w.shape[1] // 32)

    def _cpu_fast(self, x, act: str):
        from .. import cpu as _cpu
        mode, pack = self._cpu_pack
        x2 = x.detach().reshape(-1, x.shape[-1]).float().numpy()
        bias = None if self.bias is None else self.bias.detach().float().numpy()
        if mode == "f32":
            y = _cpu.gemm_nt(x2, pack, bias)
        elif mode == "bf16":
            y = _cpu.gemm_nt_bf16(x2, pack, bias)
        else:
            y = _cpu.quant_gemm(x2, pack)
            if bias is not None:
                y = y + bias
        out = torch.from_numpy(y).view(*x.shape[:-1], y.shape[-1])
        return F_._act_fwd(out, act) if act != "identity" else out

    def forward(self, x, act: str = "identity"):
        if self._cpu_pack is not None and not x.is_cuda and not torch.is_grad_enabled():
            return self._cpu_fast(x, act)
        return F_.fused_linear(x, self.weight, self.bias, act)


class Attention(nn.Module):
    def __init__(self, cfg: LmConfig):
        super().__init__()
        self.cfg = cfg
        H, Hk, D = cfg.n_head, cfg.kv_heads(), cfg.hdim()
        self.qkv = Linear(cfg.d_model, (H + 2 * Hk) * D, cfg.bias or cfg.qkv_bias)
        self.o = Linear(H * D, cfg.d_model, cfg.bias)
        self.q_norm = Norm(cfg, D) if cfg.qk_norm else None
        self.k_norm = Norm(cfg, D) if cfg.qk_norm else None

    def forward(self, x, rope: Optional[RopeCache], slopes, positions=None, cache=None, rng=None):
        cfg = self.cfg
        B, T, _ = x.shape
        H, Hk, D = cfg.n_head, cfg.kv_heads(), cfg.hdim()
        qkv = self.qkv(x)
        if H == Hk:
            qkv5 = qkv.view(B, T, 3, H, D)
            q, k, v = qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2]
        else:
            q = qkv[..., : H * D].view(B, T, H, D)
            k = qkv[..., H * D: (H + Hk) * D].view(B, T, Hk, D)
            v = qkv[..., (H + Hk) * D:].view(B, T, Hk, D)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        if rope is not None:
            q = apply_rope(q, rope.cos, rope.sin, positions)
            k = apply_rope(k, rope.cos, rope.sin, positions)
        if cache is not None:
            k, v = cache.append(k, v)
        p_drop = cfg.attn_dropout if self.training else 0.0
        seed, off = rng if rng is not None else (0, 0)
        o = F_.attention(q, k, v, causal=True, window=cfg.window, softcap=cfg.attn_softcap, alibi_slopes=slopes,
                         dropout_p=p_drop, dropout_seed=seed, dropout_offset=off)
        return self.o(o.reshape(B, T, H * D))


class Mlp(nn.Module):
    def __init__(self, cfg: LmConfig):
        super().__init__()
        self.kind = cfg.mlp
        self.F = cfg.d_ff
        mult = 2 if cfg.gated_mlp() else 1
        self.up = Linear(cfg.d_model, mult * cfg.d_ff, cfg.bias)     # gated: rows [W1 | W3]
        self.down = Linear(cfg.d_ff, cfg.d_model, cfg.bias)

    def forward(self, x):
        if self.kind == "gelu":
            return self.down(self.up(x, "gelu"))
        return self.down(F_.gated_activation(self.up(x), "swiglu" if self.kind == "swiglu" else "geglu"))


class Block(nn.Module):
    def __init__(self, cfg: LmConfig, layer: int):
        super().__init__()
        self.cfg, self.layer = cfg, layer
        self.norm1 = Norm(cfg)
        self.attn = Attention(cfg)
        self.norm2 = None if cfg.parallel_block else Norm(cfg)
        self.moe = None
        self.mlp = None
        if cfg.is_moe_layer(layer):
            self.moe = MoEFFN(MoeSpec(cfg.moe_experts, cfg.moe_top_k, cfg.d_model, cfg.expert_ff(),
                                      cfg.moe_capacity_factor, cfg.moe_min_capacity,
                                      "reroute" if cfg.moe_reroute else "drop", cfg.moe_groups, cfg.moe_noisy,
                                      cfg.moe_aux_alpha, cfg.moe_z_alpha), cfg.init_std, cfg.seed + 101 * layer)
            if cfg.moe_shared_expert:
                self.mlp = Mlp(cfg)
        else:
            self.mlp = Mlp(cfg)

    def _ffn(self, h):
        y = 0
        if self.moe is not None:
            y = self.moe(h)
        if self.mlp is not None:
            y = y + self.mlp(h)
        return y

    def _drop(self, x, rng, salt):
        p = self.cfg.resid_dropout
        if not self.training or p <= 0.0:
            return x
        seed, off = rng if rng is not None else (self.cfg.seed, 0)
        return F_.dropout_philox(x, p, seed, off * 4096 + self.layer * 2 + salt)

    def forward(self, x, rope, slopes, positions=None, cache=None, rng=None):
        cfg = self.cfg
        if cfg.prenorm:
            h = self.norm1(x)
            a = self._drop(self.attn(h, rope, slopes, positions, cache, rng), rng, 0)
            if cfg.parallel_block:
                return x + a + self._drop(self._ffn(h), rng, 1)
            x = x + a
            return x + self._drop(self._ffn(self.norm2(x)), rng, 1)
        # post-norm: r1 = x + attn(x); n = norm1(r1); out = norm2(n + ffn(n))
        n = self.norm1(x + self._drop(self.attn(x, rope, slopes, positions, cache, rng), rng, 0))
        return self.norm2(n + self._drop(self._ffn(n), rng, 1))


class KvCache:
    """Contiguous per-layer K/V cache for incremental decode."""

    def __init__(self):
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None

    def append(self, k, v):
        self.k = k if self.k is None else torch.cat([self.k, k], dim=1)
        self.v = v if self.v is None else torch.cat([self.v, v], dim=1)
        return self.k, self.v

    def length(self) -> int:
        return 0 if self.k is None else self.k.shape[1]


class LanguageModel(nn.Module):
    def __init__(self, config: LmConfig):
        super().__init__()
        validate(config)
        self.config = config
        cfg = config
        Vp = cfg.padded_vocab()
        self.wte = nn.Parameter(torch.empty(Vp, cfg.d_model))
        self.wpe = nn.Parameter(torch.empty(cfg.max_position, cfg.d_model)) if cfg.pos == "learned" else None
        self.h = nn.ModuleList([Block(cfg, l) for l in range(cfg.n_layer)])
        self.norm_f = Norm(cfg)
        self.lm_head = None if cfg.tie_embeddings else nn.Parameter(torch.empty(Vp, cfg.d_model))
        self.rope = RopeCache(cfg) if cfg.pos == "rope" else None
        self.register_buffer("slopes", alibi_slopes(cfg.n_head) if cfg.pos == "alibi" else None, persistent=False)
        if cfg.pos == "sinusoidal":
            pe = torch.zeros(cfg.max_position, cfg.d_model)
            pos = torch.arange(cfg.max_position)[:, None].float()
            div = torch.exp(torch.arange(0, cfg.d_model, 2).float() * (-math.log(10000.0) / cfg.d_model))
            pe[:, 0::2] = torch.sin(pos * div)
            pe[:, 1::2] = torch.cos(pos * div)[:, : cfg.d_model // 2]
            self.register_buffer("sin_pe", pe, persistent=False)
        else:
            self.sin_pe = None
        self.rng_state = (cfg.seed, 0)
        self.recompute = cfg.recompute
        self.init_weights()

    # ------------------------------------------------------------------------------------- init
    def init_weights(self) -> None:
        cfg = self.config
        g = torch.Generator().manual_seed(cfg.seed)
        std = cfg.init_std
        m = cfg.d_model / cfg.mup_base_width if cfg.init == "mup" else 1.0
        for name, p in self.named_parameters():
            if p.dim() < 2 or ".moe." in name:
                continue
            s = std
            if cfg.init == "gpt2" and (name.endswith("attn.o.weight") or name.endswith("mlp.down.weight")):
                s = std / math.sqrt(2 * cfg.n_layer)
            if cfg.init == "mup" and name not in ("wte", "wpe"):
                s = std / math.sqrt(m)
            _trunc_normal_(p.data, s, g, cfg.init_truncated)
        with torch.no_grad():
            if cfg.padded_vocab() > cfg.vocab_size:
                self.wte[cfg.vocab_size:].zero_()
                if self.lm_head is not None:
                    self.lm_head[cfg.vocab_size:].zero_()

    def to(self, *args, **kwargs):
        out = super().to(*args, **kwargs)
        if self.rope is not None:
            self.rope.to(self.wte.device)
        return out

    # ---------------------------------------------------------------------------- CPU inference weight modes
    def prepare_cpu_inference(self, mode: str = "f32") -> None:
        """Packs every projection for inference on the CPU: "f32" (contiguous FP32 GEMM), "bf16" (BF16 weight bits,
        FP32 accumulation: half the weight bytes), "int8" (per-output-row symmetric INT8, activations quantised per row,
        integer dot products), "int4" (nibbles with one scale per 32 inputs).  Only no-grad forward passes on CPU
        tensors use the packed form (generation, evaluation); training keeps the FP32 parameters.  Attention on that
        path is the blocked native kernel.  Parity: `LanguageModel::prepare_cpu_inference(CpuWeightMode)` of the
        reference (include/nexus/lm/model.hpp:56-61,151)."""
        mode = mode.lower()
        if mode not in CPU_WEIGHT_MODES:
            raise ValueError(f"cpu weight mode must be one of {CPU_WEIGHT_MODES}")
        total = 0
        for m in self.modules():
            if isinstance(m, Linear):
                total += m.pack_for_cpu(mode)
        self._cpu_mode, self._cpu_bytes = ("f32" if mode == "auto" else mode), total

    def cpu_weight_mode(self) -> str:
        return getattr(self, "_cpu_mode", "auto")

    def cpu_inference_weight_bytes(self) -> int:
        return getattr(self, "_cpu_bytes", 0)

    def set_rng(self, seed: int, offset: int) -> None:
        self.rng_state = (seed, offset)

    # ---------------------------------------------------------------------------------- forward
    def hidden(self, tokens: torch.Tensor, caches: Optional[List[KvCache]] = None, start: int = 0) -> torch.Tensor:
        cfg = self.config
        B, T = tokens.shape
        positions = None
        if start > 0:
            positions = (torch.arange(T, device=tokens.device) + start)[None].expand(B, T)
        if cfg.pos == "learned":
            wpe = self.wpe if start == 0 else None
            x = F_.embedding_pos(tokens, self.wte, wpe)
            if start > 0:
                x = x + self.wpe[positions]
        else:
            x = F_.embedding_pos(tokens, self.wte, None)
            if self.sin_pe is not None:
                x = x + self.sin_pe[start: start + T].to(x.dtype)[None]
        if self.rope is not None and self.rope.cos.device != x.device:
            self.rope.to(x.device)
        if self.training and cfg.resid_dropout > 0:
            x = F_.dropout_philox(x, cfg.resid_dropout, self.rng_state[0], self.rng_state[1] * 4096 + 4095)
        for l, blk in enumerate(self.h):
            cache = caches[l] if caches is not None else None
            use_ckpt = self.training and cache is None and (
                self.recompute == "full" or (self.recompute == "every_k" and l % cfg.recompute_every == 0))
            if use_ckpt:
                from ..autograd.checkpoint import checkpoint
                x = checkpoint(lambda t, b=blk: b(t, self.rope, self.slopes, positions, None, self.rng_state), x)
            else:
                x = blk(x, self.rope, self.slopes, positions, cache, self.rng_state)
        return self.norm_f(x) if cfg.prenorm or True else x

    def logits(self, tokens: torch.Tensor, caches=None, start: int = 0) -> torch.Tensor:
        h = self.hidden(tokens, caches, start)
        w = self.wte if self.lm_head is None else self.lm_head
        out = F_.fused_linear(h, w.to(h.dtype) if w.dtype != h.dtype else w, None)
        m = self.config.mup_base_width / self.config.d_model if self.config.init == "mup" else 1.0
        return out * m if m != 1.0 else out

    def aux_loss(self) -> torch.Tensor:
        tot = 0.0
        for blk in self.h:
            if blk.moe is not None and blk.moe.last_routing is not None:
                tot = tot + blk.moe.losses()
        return tot

    def loss(self, tokens: torch.Tensor, label_smoothing: float = 0.0, z_loss: float = 0.0) -> torch.Tensor:
        lg = self.logits(tokens)
        l = F_.cross_entropy_shifted(lg, tokens, label_smoothing=label_smoothing, z_loss=z_loss,
                                     vocab=self.config.vocab_size)
        if self.config.moe_experts > 0:
            l = l + self.aux_loss()
        return l

    forward = loss

    # ------------------------------------------------------------------------------- generation
    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new: int, greedy: bool = True, temperature: float = 1.0,
                 seed: int = 0) -> torch.Tensor:
        """Incremental decode with a KV cache; prompt [B, T0] -> [B, T0 + max_new]."""
        was = self.training
        self.eval()
        caches = [KvCache() for _ in self.h]
        out = prompt
        lg = self.logits(prompt, caches, 0)[:, -1, : self.config.vocab_size]
        g = torch.Generator(device="cpu").manual_seed(seed)
        for i in range(max_new):
            if greedy:
                nxt = lg.float().argmax(-1, keepdim=True)
            else:
                p = torch.softmax(lg.float().cpu() / max(temperature, 1e-6), -1)
                nxt = torch.multinomial(p, 1, generator=g).to(prompt.device)
            out = torch.cat([out, nxt.to(out.dtype)], dim=1)
            if i + 1 < max_new:
                lg = self.logits(nxt.to(out.dtype), caches, out.shape[1] - 1)[:, -1, : self.config.vocab_size]
        self.train(was)
        return out

    # ------------------------------------------------------------------------------ persistence
    def named_weights(self) -> Dict[str, torch.Tensor]:
        return {n: p.detach() for n, p in self.named_parameters()}

    def save_nxs(self, path: str) -> None:
        from ..nxs import archive
        archive.save_language_model(self, path)

    @staticmethod
    def load_nxs(path: str) -> "LanguageModel":
        from ..nxs import archive
        return archive.load_language_model(path)


def build(config: LmConfig) -> LanguageModel:
    return LanguageModel(config)


class AdamW:
    """`lm::AdamW`: decoupled weight decay on >= 2-D tensors, shared op order with every backend."""

    def __init__(self, model: nn.Module, lr=6e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                 grad_clip: float = 0.0):
        self.params = [p for p in model.parameters() if p.requires_grad]
        self.m = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.v = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.wd = [1.0 if p.dim() >= 2 else 0.0 for p in self.params]
        self.lr, self.b1, self.b2, self.eps, self.weight_decay, self.clip = lr, beta1, beta2, eps, weight_decay, grad_clip
        self.step_count = 0

    def zero_grad(self):
        for p in self.params:
            p.grad = None

    def step(self, lr: Optional[float] = None) -> float:
        self.step_count += 1
        idx = [i for i, p in enumerate(self.params) if p.grad is not None]
        ps = [self.params[i].data for i in idx]
        if all(p.dtype == torch.float32 for p in ps):
            return F_.adamw_multi_tensor(ps, [self.params[i].grad for i in idx], [self.m[i] for i in idx],
                                         [self.v[i] for i in idx], self.step_count, lr or self.lr, self.b1, self.b2,
                                         self.eps, self.weight_decay, self.clip, [self.wd[i] for i in idx])
        # narrow parameters: update an FP32 copy, round once
        f32 = [p.float() for p in ps]
        n = F_.adamw_multi_tensor(f32, [self.params[i].grad.float() for i in idx], [self.m[i] for i in idx],
                                  [self.v[i] for i in idx], self.step_count, lr or self.lr, self.b1, self.b2,
                                  self.eps, self.weight_decay, self.clip, [self.wd[i] for i in idx])
        for p, q in zip(ps, f32):
            p.copy_(q)
        return n
