"""GPT-2 inference engine with a paged KV cache.

* KV pool per layer ``[blocks, block_size, heads, head_dim]`` (BF16, INT8 or FP8-E4M3 with one scale
  per (slot, head)); the native host scheduler (`csrc/host/kv_sched.cpp`: block pool with reference counts,
  per-sequence block and token lists, packing of a step's index rows into the pinned staging buffer) gives
  copy-on-write ``fork_sequence`` and ``truncate``.
* One ``forward`` takes a packed batch of chunks (sequence, new tokens).  Chunks of a sequence whose
  cache is empty run the tcgen05 flash-attention kernel; every other row (decode, speculative
  verification, continuation) runs the paged decode kernel with its own causal limit.
* Linear layers: rows <= 16 use the skinny kernel whose row results do not depend on the batch
  (speculative decoding is token-identical to greedy decoding); larger batches use the tcgen05 GEMM.
* Decode-only batches replay one CUDA graph per bucket (1, 2, 4, ... max_seqs rows) over static inputs.
* Tensor parallelism (heads and MLP columns sharded over a process group) with one all-reduce after the
  attention projection and one after the MLP.
* Weight quantisation: W8A8 (SmoothQuant-style smoothing, activations rounded to the INT8 grid) and
  W4A16 (group-wise, AWQ-style scaling), KV INT8 / FP8.

On a CPU device the same engine runs on plain PyTorch FP32 math (used by the host-logic tests).

Parity: include/nexus/cuda/infer.hpp:41-181, src/cuda/infer.cpp:146-733,758-981,1135-1226 of the reference.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .. import _native

__all__ = ["Gpt2Weights", "QuantOptions", "EngineConfig", "SamplingParams", "Chunk", "StepStats", "Engine",
           "GenerateStats", "SpecStats", "generate", "speculative_generate", "load_gpt2"]

LAYER_KEYS = ("ln1_w", "ln1_b", "attn_w", "attn_b", "proj_w", "proj_b", "ln2_w", "ln2_b", "fc_w", "fc_b", "fc2_w",
              "fc2_b")


# ------------------------------------------------------------------------------------------ weights
@dataclass
class Gpt2Weights:
    """FP32 host weights; linear weights are ``[out, in]``."""
    layers: int = 0
    heads: int = 0
    d: int = 0
    vocab: int = 0
    ctx: int = 0
    wte: Optional[torch.Tensor] = None
    wpe: Optional[torch.Tensor] = None
    ln_f_w: Optional[torch.Tensor] = None
    ln_f_b: Optional[torch.Tensor] = None
    h: List[Dict[str, torch.Tensor]] = field(default_factory=list)

    def parameters(self) -> int:
        n = self.wte.numel() + self.wpe.numel() + self.ln_f_w.numel() + self.ln_f_b.numel()
        return n + sum(t.numel() for layer in self.h for t in layer.values())

    @staticmethod
    def random(layers: int, heads: int, d: int, vocab: int, ctx: int, seed: int = 0) -> "Gpt2Weights":
        g = torch.Generator().manual_seed(seed)

        def n(*shape, std=0.02):
            return torch.randn(*shape, generator=g) * std
        w = Gpt2Weights(layers, heads, d, vocab, ctx, n(vocab, d), n(ctx, d), torch.ones(d), torch.zeros(d))
        ps = 0.02 / math.sqrt(2 * layers)
        for _ in range(layers):
            w.h.append({"ln1_w": torch.ones(d), "ln1_b": torch.zeros(d), "attn_w": n(3 * d, d), "attn_b": n(3 * d),
                        "proj_w": n(d, d, std=ps), "proj_b": n(d), "ln2_w": torch.ones(d), "ln2_b": torch.zeros(d),
                        "fc_w": n(4 * d, d), "fc_b": n(4 * d), "fc2_w": n(d, 4 * d, std=ps), "fc2_b": n(d)})
        return w

    @staticmethod
    def from_gpt_model(model) -> "Gpt2Weights":
        """From the training-side flat-buffer ``GptModel``."""
        sd = {k: v.detach().float().cpu() for k, v in model.state_dict().items()}
        L, d = model.L, model.C
        w = Gpt2Weights(L, model.H, d, model.V, sd["wpe"].shape[0], sd["wte"][: model.V].clone(), sd["wpe"],
                        sd["lnf_w"], sd["lnf_b"])
        for l in range(L):
            w.h.append({"ln1_w": sd["ln1_w"][l], "ln1_b": sd["ln1_b"][l], "attn_w": sd["qkv_w"][l],
                        "attn_b": sd["qkv_b"][l], "proj_w": sd["attproj_w"][l], "proj_b": sd["attproj_b"][l],
                        "ln2_w": sd["ln2_w"][l], "ln2_b": sd["ln2_b"][l], "fc_w": sd["fc_w"][l], "fc_b": sd["fc_b"][l],
                        "fc2_w": sd["fcproj_w"][l], "fc2_b": sd["fcproj_b"][l]})
        return w

    @staticmethod
    def from_language_model(model) -> "Gpt2Weights":
        """From ``lm.LanguageModel`` (GPT-2 family: LayerNorm, GELU, learned positions, biases)."""
        cfg = model.config
        sd = {k: v.detach().float().cpu() for k, v in model.state_dict().items()}
        w = Gpt2Weights(cfg.n_layer, cfg.n_head, cfg.d_model, cfg.vocab_size, cfg.max_position, sd["wte"], sd["wpe"],
                        sd["norm_f.weight"], sd["norm_f.bias"])
        for l in range(cfg.n_layer):
            p = f"h.{l}."
            w.h.append({"ln1_w": sd[p + "norm1.weight"], "ln1_b": sd[p + "norm1.bias"],
                        "attn_w": sd[p + "attn.qkv.weight"], "attn_b": sd[p + "attn.qkv.bias"],
                        "proj_w": sd[p + "attn.o.weight"], "proj_b": sd[p + "attn.o.bias"],
                        "ln2_w": sd[p + "norm2.weight"], "ln2_b": sd[p + "norm2.bias"],
                        "fc_w": sd[p + "mlp.up.weight"], "fc_b": sd[p + "mlp.up.bias"],
                        "fc2_w": sd[p + "mlp.down.weight"], "fc2_b": sd[p + "mlp.down.bias"]})
        return w


def load_gpt2(path: str) -> Gpt2Weights:
    """Loads a GPT-2 checkpoint written by ``GptModel``/``LanguageModel`` archives (``.nxs``) or a torch file."""
    if str(path).endswith((".pt", ".pth")):
        sd = torch.load(path, map_location="cpu")
        w = Gpt2Weights(**{k: sd[k] for k in ("layers", "heads", "d", "vocab", "ctx")})
        w.wte, w.wpe, w.ln_f_w, w.ln_f_b, w.h = sd["wte"], sd["wpe"], sd["ln_f_w"], sd["ln_f_b"], sd["h"]
        return w
    from ..lm.model import LanguageModel
    return Gpt2Weights.from_language_model(LanguageModel.load_nxs(path))


# ------------------------------------------------------------------------------------------ config
@dataclass
class QuantOptions:
    weights: str = "bf16"        # "bf16" | "w8a8" | "w4a16"
    kv: str = "bf16"             # "bf16" | "int8" | "fp8"
    w4_group: int = 128
    smooth_alpha: float = 0.5    # W8A8 smoothing exponent
    calibration: Sequence[int] = ()   # tokens for activation statistics; empty: no smoothing


@dataclass
class EngineConfig:
    precision: str = "bf16"      # "bf16" | "fp32" (fp32: reference math, any device)
    max_seqs: int = 64
    max_tokens: int = 2048       # per step, prefill included
    block_size: int = 16
    kv_bytes: int = 1 << 30
    cuda_graphs: bool = True
    quant: QuantOptions = field(default_factory=QuantOptions)
    device: str = "cuda"
    decode_splits: int = 0       # 0: chosen per step from the batch size and context length
    tp_graphs: bool = False      # decode CUDA graphs of a tensor-parallel engine (its all-reduces are captured too);
                                 # call Engine.release_graphs() before the process group is destroyed
    tp_comm: str = "nccl"        # "nccl" | "fused": the tensor-parallel all-reduces run as the peer-memory kernel
                                 # (symmetric buffers, flag barriers with a device-resident generation: graph safe)


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0   # prompt + output tokens
    frequency_penalty: float = 0.0    # output tokens only
    presence_penalty: float = 0.0
    seed: int = 0


@dataclass
class Chunk:
    seq: int = -1
    tokens: Sequence[int] = ()
    logits: int = 1          # logits of the last `logits` tokens are produced (0: none)
    output: bool = False     # tokens are model output (frequency / presence counters)


@dataclass
class PendingTokens:
    """Tokens of one ``Engine.sample(..., pending=True)`` call on their way to the host."""
    event: object
    pinned: torch.Tensor
    rows: int
    seqs: List[int]


@dataclass
class StepStats:
    tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    graph: bool = False
    ms: float = 0.0


# ------------------------------------------------------------------------------------------ linear layers
class _Linear:
    """One linear layer in the engine's storage format (dense BF16/FP32, INT8 or INT4)."""

    def __init__(self, w: torch.Tensor, b: Optional[torch.Tensor], dev, fast: bool, quant: str = "bf16", group: int = 128,
                 smooth: Optional[torch.Tensor] = None):
        self.n, self.k = w.shape
        self.fast, self.quant, self.group = fast, quant, group
        self.bias = None if b is None else b.to(dev, torch.bfloat16 if fast else torch.float32)
        self.inv_smooth = None
        if quant == "bf16" or not fast and quant == "bf16":
            self.w = w.to(dev, torch.bfloat16 if fast else torch.float32).contiguous()
            self.nbytes = self.w.numel() * self.w.element_size()
            return
        wf = w.float()
        if quant == "fp8":
            if not fast:
                raise ValueError("fp8 weights need the kernel path (CUDA, bf16 precision)")
            # E4M3 codes with one scale per output row; activations are quantised per row at run time
            scale = wf.abs().amax(dim=1).clamp_min(1e-12) / 448.0
            self.wq = (wf / scale[:, None]).to(dev).to(torch.float8_e4m3fn).contiguous()
            self.scales = scale.to(dev, torch.float32).contiguous()
            self.nbytes = self.wq.numel() + self.scales.numel() * 4
            self._dense = None
            return
        if quant == "w8a8":
            if smooth is not None:  # x' = x / s, w' = w * s
                wf = wf * smooth[None, :]
                self.inv_smooth = (1.0 / smooth).to(dev, torch.float32)
            scale = wf.abs().amax(dim=1).clamp_min(1e-8) / 127.0
            q = torch.round(wf / scale[:, None]).clamp_(-127, 127).to(torch.int8)
            self.wq, self.scales = q.to(dev).contiguous(), scale.to(dev, torch.float32)
        elif quant == "w4a16":
            if self.k % group:
                raise ValueError(f"w4a16: in-features {self.k} not divisible by group {group}")
            g = wf.view(self.n, self.k // group, group)
            scale = g.abs().amax(dim=2).clamp_min(1e-8) / 7.0
            q = (torch.round(g / scale[:, :, None]).clamp_(-8, 7) + 8).to(torch.uint8).view(self.n, self.k)
            packed = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
            self.wq, self.scales = packed.to(dev), scale.to(dev, torch.float32).contiguous()
        else:
            raise ValueError(f"unknown weight quantisation {quant!r}")
        self.nbytes = self.wq.numel() + self.scales.numel() * 4
        self._dense = None if fast else self.dense().float()

    def dense(self) -> torch.Tensor:
        """Dequantised weights (BF16 on the kernel path, FP32 otherwise)."""
        if self.quant == "bf16":
            return self.w
        if self.quant == "fp8":
            from ..ops import _lowp as LP
            return LP.fp8_dequantize(self.wq, None).float().mul_(self.scales[:, None]).to(torch.bfloat16)
        if self.fast:
            from ..ops import _infer as I
            return I.wq_dequant(self.wq, self.scales, bits=8 if self.quant == "w8a8" else 4, group=self.group, k=self.k)
        if self.quant == "w8a8":
            return self.wq.float() * self.scales[:, None]
        lo, hi = (self.wq & 15).float() - 8.0, (self.wq >> 4).float() - 8.0
        q = torch.stack([lo, hi], dim=2).view(self.n, self.k)
        return (q.view(self.n, self.k // self.group, self.group) * self.scales[:, :, None]).view(self.n, self.k)


# ------------------------------------------------------------------------------------------ engine
class Engine:
    def __init__(self, weights: Gpt2Weights, config: Optional[EngineConfig] = None, group=None):
        self.cfg = config or EngineConfig()
        cfg = self.cfg
        self.dev = torch.device(cfg.device)
        self.fast = self.dev.type == "cuda" and cfg.precision == "bf16"
        if self.dev.type == "cuda" and cfg.precision == "bf16":
            from ..ops import _cuda as K
            K.lib()  # fails loudly when the kernel library is missing
        self.group = group
        self.tp = group.size() if group is not None else 1
        self.tp_rank = group.rank() if group is not None else 0
        self.L, self.H, self.d, self.V, self.ctx = weights.layers, weights.heads, weights.d, weights.vocab, weights.ctx
        self.D = self.d // self.H
        self.Hp = -(-self.H // self.tp)                    # heads per rank (last rank may hold fewer)
        self.h0 = min(self.H, self.tp_rank * self.Hp)
        self.Hl = max(0, min(self.Hp, self.H - self.h0))  # local heads
        F = 4 * self.d
        self.Fl = F // self.tp
        if F % self.tp:
            raise ValueError("MLP width must divide by the tensor-parallel size")
        if self.fast and self.D not in (64, 128):
            raise ValueError("the kernel path supports head_dim 64 and 128")
        self.Vp = (self.V + 63) // 64 * 64
        self.wdt = torch.bfloat16 if self.fast else torch.float32
        self._load(weights)
        self._alloc_kv()
        # sequences, block lists, reference counts and batch packing live in the native scheduler
        self.sched = _native.KvScheduler(self.n_blocks, cfg.block_size, cfg.max_seqs, self.ctx)
        self.block_table = torch.zeros((cfg.max_seqs, self.max_blocks), dtype=torch.int32, device=self.dev)
        self.counts_all = torch.zeros((cfg.max_seqs, self.V), dtype=torch.int32, device=self.dev)
        self.counts_out = torch.zeros((cfg.max_seqs, self.V), dtype=torch.int32, device=self.dev)
        self._ones = torch.ones(cfg.max_tokens, dtype=torch.int32, device=self.dev)
        # pipelined decode: last sampled token per sequence (device), pinned landing buffers, host positions to complete
        self._last_tok = torch.zeros(cfg.max_seqs, dtype=torch.int32, device=self.dev)
        self._tok_pins = [torch.zeros(cfg.max_seqs, dtype=torch.int32).pin_memory() for _ in range(3)] \
            if self.dev.type == "cuda" else []
        self._tok_pin_next = 0
        self._patch: Dict[int, int] = {}
        self._stage_bufs: Dict[int, torch.Tensor] = {}
        self._stage_evt: dict = {}
        self._sample_cache: dict = {}
        self._logits: Optional[torch.Tensor] = None
        self._logit_seq: List[int] = []
        self._stats = StepStats()
        self._graphs: Dict[int, object] = {}
        self._static: Dict[int, dict] = {}
        self._pin = None
        self._capture = None
        self._fused_ar = None
        if self.tp > 1 and cfg.tp_comm == "fused":
            if not self.fast:
                raise ValueError("tp_comm='fused' needs the kernel path (CUDA, bf16 precision)")
            from ..parallel.symm import SymmetricWorkspace
            ws = SymmetricWorkspace(group)
            n = (cfg.max_tokens * self.d + 7) // 8 * 8
            self._fused_ar = (ws, ws.alloc(n, torch.float32), ws.alloc(n, torch.float32))
        elif cfg.tp_comm not in ("nccl", "fused"):
            raise ValueError("tp_comm must be 'nccl' or 'fused'")

    # ----------------------------------------------------------------------------- weights / KV pool
    def _load(self, w: Gpt2Weights) -> None:
        dev, q = self.dev, self.cfg.quant
        fl = torch.float32
        wte = torch.zeros((self.Vp, self.d))
        wte[: self.V] = w.wte
        self.wte = wte.to(dev, self.wdt)
        self.wpe = w.wpe.to(dev, self.wdt)
        self.lnf_w, self.lnf_b = w.ln_f_w.to(dev, fl), w.ln_f_b.to(dev, fl)
        smooth = self._calibrate(w) if (q.weights == "w8a8" and len(q.calibration)) else None
        D, h0, Hl, d = self.D, self.h0, self.Hl, self.d
        rows = slice(h0 * D, (h0 + Hl) * D)
        f0, f1 = self.tp_rank * self.Fl, (self.tp_rank + 1) * self.Fl
        self.layers: List[dict] = []
        self.weight_nbytes = (self.wte.numel() + self.wpe.numel()) * self.wte.element_size()
        first = self.tp_rank == 0
        for l, lw in enumerate(w.h):
            aw, ab = lw["attn_w"], lw["attn_b"]
            qkv_w = torch.cat([aw[i * d: (i + 1) * d][rows] for i in range(3)], 0)
            qkv_b = torch.cat([ab[i * d: (i + 1) * d][rows] for i in range(3)], 0)
            sm = smooth[l] if smooth is not None else {}
            mk = lambda wt, b, key: _Linear(wt, b, dev, self.fast, q.weights, q.w4_group, sm.get(key))  # noqa: E731
            layer = {
                "ln1_w": lw["ln1_w"].to(dev, fl), "ln1_b": lw["ln1_b"].to(dev, fl),
                "ln2_w": lw["ln2_w"].to(dev, fl), "ln2_b": lw["ln2_b"].to(dev, fl),
                "qkv": mk(qkv_w, qkv_b, "qkv"),
                # row-parallel layers add their bias on the first rank only
                "proj": mk(lw["proj_w"][:, rows].contiguous(), lw["proj_b"] if first else None, "proj"),
                "fc": mk(lw["fc_w"][f0:f1].contiguous(), lw["fc_b"][f0:f1], "fc"),
                "fc2": mk(lw["fc2_w"][:, f0:f1].contiguous(), lw["fc2_b"] if first else None, "fc2"),
            }
            self.weight_nbytes += sum(layer[k].nbytes for k in ("qkv", "proj", "fc", "fc2"))
            self.layers.append(layer)

    def _calibrate(self, w: Gpt2Weights):
        """Per-layer SmoothQuant factors s_j = max|x_j|^a / max|w_j|^(1-a) from a reference FP32 pass."""
        toks = torch.tensor(list(self.cfg.quant.calibration), dtype=torch.long)[: self.ctx]
        a = self.cfg.quant.smooth_alpha
        x = w.wte[toks] + w.wpe[: toks.numel()]
        out = []
        T, H, D = toks.numel(), self.H, self.D
        mask = torch.ones(T, T).tril().bool()
        F = torch.nn.functional

        def s_of(act, weight):
            am, wm = act.abs().amax(0).clamp_min(1e-5), weight.abs().amax(0).clamp_min(1e-5)
            return (am.pow(a) / wm.pow(1 - a)).clamp(1e-2, 1e2)
        for lw in w.h:
            h1 = F.layer_norm(x, (self.d,), lw["ln1_w"], lw["ln1_b"])
            s = {"qkv": s_of(h1, lw["attn_w"])}
            qkv = h1 @ lw["attn_w"].t() + lw["attn_b"]
            q_, k_, v_ = (t.view(T, H, D).transpose(0, 1) for t in qkv.split(self.d, dim=1))
            att = (q_ @ k_.transpose(1, 2)) / math.sqrt(D)
            att = att.masked_fill(~mask, float("-inf")).softmax(-1) @ v_
            att = att.transpose(0, 1).reshape(T, self.d)
            s["proj"] = s_of(att, lw["proj_w"])
            x = x + att @ lw["proj_w"].t() + lw["proj_b"]
            h2 = F.layer_norm(x, (self.d,), lw["ln2_w"], lw["ln2_b"])
            s["fc"] = s_of(h2, lw["fc_w"])
            f = F.gelu(h2 @ lw["fc_w"].t() + lw["fc_b"], approximate="tanh")
            s["fc2"] = s_of(f, lw["fc2_w"])
            x = x + f @ lw["fc2_w"].t() + lw["fc2_b"]
            # the smoothing vectors of the sharded layers follow the local columns
            D_, h0, Hl = self.D, self.h0, self.Hl
            s["proj"] = s["proj"][h0 * D_: (h0 + Hl) * D_]
            s["fc2"] = s["fc2"][self.tp_rank * self.Fl: (self.tp_rank + 1) * self.Fl]
            out.append(s)
        return out

    def _alloc_kv(self) -> None:
        cfg = self.cfg
        kind = cfg.quant.kv
        self.kv_kind = {"bf16": 0, "int8": 1, "fp8": 2}[kind]
        if not self.fast and self.kv_kind == 2:
            raise ValueError("FP8 KV needs the kernel path")
        elem = (2 if self.fast else 4) if self.kv_kind == 0 else 1
        # sized by the heads of the fullest rank, so that every rank of a tensor-parallel group owns the same number of
        # blocks (the scheduler runs replicated) even when the heads do not divide evenly or a rank holds none
        per_tok = self.L * 2 * self.Hp * self.D * elem + (self.L * 2 * self.Hp * 4 if self.kv_kind else 0)
        self._kv_tok_bytes = per_tok
        self.n_blocks = max(2, int(cfg.kv_bytes // max(1, per_tok * cfg.block_size)))
        self.max_blocks = -(-self.ctx // cfg.block_size)
        bs, Hl, D = cfg.block_size, max(self.Hl, 1), self.D
        dt = self.wdt if self.kv_kind == 0 else (torch.int8 if self.kv_kind == 1 else torch.uint8)
        self.k_cache = [torch.zeros((self.n_blocks, bs, Hl, D), dtype=dt, device=self.dev) for _ in range(self.L)]
        self.v_cache = [torch.zeros((self.n_blocks, bs, Hl, D), dtype=dt, device=self.dev) for _ in range(self.L)]
        if self.kv_kind:
            self.k_scale = [torch.ones((self.n_blocks * bs, Hl), dtype=torch.float32, device=self.dev) for _ in range(self.L)]
            self.v_scale = [torch.ones((self.n_blocks * bs, Hl), dtype=torch.float32, device=self.dev) for _ in range(self.L)]
        else:
            self.k_scale = self.v_scale = [None] * self.L

    # ----------------------------------------------------------------------------- sequences / blocks
    def add_sequence(self) -> int:
        sid = self.sched.add()
        self.counts_all[sid].zero_()
        self.counts_out[sid].zero_()
        return sid

    def fork_sequence(self, src: int) -> int:
        """New sequence sharing every block of ``src`` (copy-on-write on the next append)."""
        sid = self.sched.fork(src)
        self.counts_all[sid].copy_(self.counts_all[src])
        self.counts_out[sid].copy_(self.counts_out[src])
        self._write_table(sid)
        return sid

    def free_sequence(self, seq: int) -> None:
        self.sched.free(seq)

    def truncate(self, seq: int, length: int) -> None:
        removed, n_out = self.sched.truncate(seq, length)
        if not removed:
            return
        # counters: remove the dropped tokens (host list -> one small device update)
        t = torch.tensor(removed, dtype=torch.long, device=self.dev)
        ones = torch.ones_like(t, dtype=torch.int32)
        self.counts_all[seq].index_add_(0, t, -ones)
        if n_out > 0:
            t2 = t[len(removed) - n_out:]
            self.counts_out[seq].index_add_(0, t2, -ones[: t2.numel()])
        self._write_table(seq)

    def length(self, seq: int) -> int:
        return self.sched.length(seq)

    def tokens(self, seq: int) -> List[int]:
        return self.sched.tokens(seq)

    def free_blocks(self) -> int:
        return self.sched.free_blocks()

    def total_blocks(self) -> int:
        return self.n_blocks

    def block_size(self) -> int:
        return self.cfg.block_size

    def blocks_needed(self, seq: int, new_tokens: int) -> int:
        """Blocks that appending ``new_tokens`` would take from the free list (copy-on-write included)."""
        return self.sched.blocks_needed(seq, new_tokens)

    def _write_table(self, seq: int) -> None:
        blocks = self.sched.blocks(seq)
        if blocks:
            row = torch.tensor(blocks, dtype=torch.int32)
            self.block_table[seq, : len(blocks)].copy_(row.to(self.dev), non_blocking=True)

    def _copy_block(self, old: int, nb: int) -> None:
        """Copy-on-write of a shared partial block: every layer's K and V page (and scales) from ``old`` to ``nb``."""
        bs = self.cfg.block_size
        for l in range(self.L):
            self.k_cache[l][nb].copy_(self.k_cache[l][old])
            self.v_cache[l][nb].copy_(self.v_cache[l][old])
            if self.kv_kind:
                self.k_scale[l][nb * bs: (nb + 1) * bs].copy_(self.k_scale[l][old * bs: (old + 1) * bs])
                self.v_scale[l][nb * bs: (nb + 1) * bs].copy_(self.v_scale[l][old * bs: (old + 1) * bs])

    # ----------------------------------------------------------------------------- math helpers
    def _linear(self, x, lin: _Linear, *, act=None, residual=None, out_dtype=None):
        """x [n, k] -> act(x W^T + b) (+ residual, FP32)."""
        if not self.fast:
            y = x @ (lin.w if lin.quant == "bf16" else lin._dense).t()
            if lin.inv_smooth is not None:  # W8A8 reference: round the smoothed activations to the INT8 grid
                xs = x * lin.inv_smooth
                sc = xs.abs().amax(1, keepdim=True).clamp_min(1e-12) / 127.0
                y = (torch.round(xs / sc).clamp(-127, 127) * sc) @ lin._dense.t()
            elif lin.quant == "w8a8":
                sc = x.abs().amax(1, keepdim=True).clamp_min(1e-12) / 127.0
                y = (torch.round(x / sc).clamp(-127, 127) * sc) @ lin._dense.t()
            if lin.bias is not None:
                y = y + lin.bias
            if act == "gelu":
                y = torch.nn.functional.gelu(y, approximate="tanh")
            return y + residual if residual is not None else y
        from ..ops import _cuda as K
        from ..ops import _infer as I
        n = x.shape[0]
        od = torch.float32 if residual is not None else (out_dtype or torch.bfloat16)
        if lin.quant == "fp8" and n > self._skinny and lin.k % 16 == 0:
            # FP8 tensor-core GEMM: half the weight bytes of BF16 (decode is bound by reading the weights)
            from ..ops import _lowp as LP
            y = LP.fp8_linear(x.to(torch.bfloat16), lin.wq, lin.scales, bias=lin.bias, act=act,
                              out_dtype=torch.float32 if residual is not None else od)
            return residual.add_(y) if residual is not None else y
        if lin.quant == "w8a8":
            _, x, _ = I.quant_rows(x, lin.inv_smooth, want_codes=False, want_fake=True)
        if lin.quant not in ("bf16", "fp8") and n <= self._skinny:   # weights stay packed: the GEMV dequantises on the fly
            y = I.wq_gemv(x, lin.wq, lin.scales, bits=8 if lin.quant == "w8a8" else 4, group=lin.group, bias=lin.bias)
            if act == "gelu":
                y = torch.nn.functional.gelu(y, approximate="tanh")
            if residual is not None:
                return residual.add_(y)
            return y if od == torch.bfloat16 else y.to(od)
        w = lin.dense()
        if n <= self._skinny:
            return I.skinny_gemm(x, w, lin.bias, act=act, residual=residual, out=residual, out_dtype=od)
        # a few rows give the tensor-core GEMM one row of tiles: slices along K keep every SM busy (fixed summation
        # order, so a row's result does not depend on what else is in the batch)
        few = n < 256
        return K.gemm(x, w, bias=lin.bias, act=act, residual=residual, out=residual, out_dtype=od,
                      split_k=0 if few else 1, block_n=128 if few else 0, deterministic=True)

    def _norm(self, x, w, b):
        if not self.fast:
            return torch.nn.functional.layer_norm(x, (self.d,), w, b)
        from ..ops import _cuda as K
        return K.norm_fwd(x, w, b, out_dtype=torch.bfloat16, want_stats=False)[0]

    def _all_reduce(self, t):
        """Sum of ``t`` [n, d] FP32 over the tensor-parallel group."""
        if self.tp == 1:
            return t
        if self._fused_ar is None:
            self.group.all_reduce_tensor(t, "sum")
            return t
        from ..parallel.symm import fused_all_reduce
        ws, src, dst = self._fused_ar
        count = (t.numel() + 7) // 8 * 8
        src.local[: t.numel()].copy_(t.reshape(-1))
        fused_all_reduce(ws, src, dst, count)
        return dst.local[: t.numel()].view(t.shape)

    # ----------------------------------------------------------------------------- forward
    def forward(self, chunks: Sequence[Chunk], layers: int = -1, device_tokens: bool = False) -> torch.Tensor:
        """Runs the packed batch; returns FP32 logits ``[logit_rows, vocab_padded]`` on the device.

        ``device_tokens`` (one-token chunks): the token of every chunk is the one the last ``sample`` drew
        for its sequence, taken from the device-resident table without the host having read it yet; the chunk's own
        token value is ignored and the host-side token list is completed by ``collect``.  This is what lets a server
        launch decode step n + 1 before it has read the tokens of step n."""
        t0 = time.perf_counter()
        cfg = self.cfg
        nl = self.L if layers < 0 else min(layers, self.L)
        stats = StepStats()
        live = [c for c in chunks if len(c.tokens)]
        flat: List[int] = []
        if not device_tokens:
            for c in live:
                flat.extend(int(t) for t in c.tokens)
        else:
            flat = [0] * len(live)
        plan = self.sched.plan([c.seq for c in live], [len(c.tokens) for c in live], flat, [c.logits for c in live],
                               [int(bool(c.output)) for c in live], device_tokens, cfg.max_tokens)
        for old, nb in plan["cows"]:
            self._copy_block(old, nb)
        for sid in plan["tables"]:
            self._write_table(sid)
        for sid, idx in plan["patches"]:
            self._patch[sid] = idx          # filled in by collect() once the token has been read
        N, R = plan["tokens"], plan["logit_rows"]
        runs, out_rows = plan["runs"], plan["out_rows"]
        self._logit_seq = plan["logit_seq"]
        stats.prefill_tokens, stats.decode_tokens = plan["prefill_tokens"], plan["decode_tokens"]
        stats.tokens = N
        if N == 0:
            self._logits = torch.zeros((0, self.Vp), dtype=torch.float32, device=self.dev)
            self._stats = stats
            return self._logits
        self._skinny = 16
        decode_only = all(k == "paged" for k, *_ in runs) and N == R == stats.decode_tokens
        # tensor-parallel ranks run the same schedule, so with tp_graphs every rank captures and replays the same buckets
        # in the same order, the all-reduces of the layer loop captured with the kernels around them
        use_graph = self.fast and cfg.cuda_graphs and decode_only and nl == self.L and (self.tp == 1 or cfg.tp_graphs)
        bucket = 1 << (N - 1).bit_length() if use_graph else N
        # one staging buffer in pinned memory, reused every step, and ONE host-to-device copy for all index arrays
        ints = self._stage(bucket)
        self.sched.write(ints.data_ptr(), bucket)
        if use_graph:
            logits = self._decode_graph(bucket, ints, N if device_tokens else 0)[:R]
            dv = self._static[bucket]["ints"]
            stats.graph = True
        else:
            dv = ints.to(self.dev, non_blocking=True)
            if device_tokens:
                dv[0, :N] = self._last_tok[dv[3, :N].long()]
            logits = self._body(dv[0], dv[1], dv[2], dv[3], dv[4], dv[5][:R], runs, nl)
        if self.dev.type == "cuda":
            ev = self._stage_evt.get(bucket)
            if ev is None:
                ev = self._stage_evt[bucket] = torch.cuda.Event()
            ev.record()
        # token counters (repetition: every token; frequency / presence: output tokens only), from the index arrays
        # that are on the device already
        flat = dv[3, :N].long() * self.V + dv[0, :N].long()
        ones = self._ones[:N]
        self.counts_all.view(-1).index_add_(0, flat, ones)
        if len(out_rows) == N:
            self.counts_out.view(-1).index_add_(0, flat, ones)
        elif out_rows:
            fo = flat[torch.tensor(out_rows, dtype=torch.long).to(self.dev, non_blocking=True)]
            self.counts_out.view(-1).index_add_(0, fo, self._ones[: len(out_rows)])
        self._logits = logits
        stats.ms = (time.perf_counter() - t0) * 1e3
        self._stats = stats
        return logits

    def _body(self, tok, pos, slot, rseq, ctx_len, logit_rows, runs, nl: int) -> torch.Tensor:
        """Layer loop over device index arrays (also the body of the captured decode graphs)."""
        N = tok.shape[0]
        d, D, Hl = self.d, self.D, self.Hl
        cap = self._capture
        if self.fast:
            from ..ops import _cuda as K
            from ..ops import _infer as I
            x = K.embedding_pos_fwd(tok, self.wte, self.wpe, positions=pos, out_dtype=torch.float32, seq_len=1)
        else:
            x = self.wte[tok.long()] + self.wpe[pos.long()]
        bs = self.cfg.block_size
        dl = Hl * D
        for l in range(nl):
            lw = self.layers[l]
            if Hl == 0:   # more ranks than heads: this rank only takes part in the all-reduce
                x = x + self._all_reduce(torch.zeros_like(x))
                h2 = self._norm(x, lw["ln2_w"], lw["ln2_b"])
                f = self._linear(h2, lw["fc"], act="gelu")
                x = x + self._all_reduce(self._linear(f, lw["fc2"], out_dtype=torch.float32).float())
                continue
            h = self._norm(x, lw["ln1_w"], lw["ln1_b"])
            qkv = self._linear(h, lw["qkv"])                         # [N, 3 * dl]
            q = qkv[:, :dl].view(N, Hl, D)
            k = qkv[:, dl: 2 * dl].view(N, Hl, D)
            v = qkv[:, 2 * dl:].view(N, Hl, D)
            att = torch.empty((N, Hl, D), dtype=qkv.dtype, device=self.dev)
            if self.fast:
                I.kv_append(k, v, slot, self.k_cache[l], self.v_cache[l], k_scale=self.k_scale[l],
                            v_scale=self.v_scale[l], kv_kind=self.kv_kind)
                for kind, r0, r1, _ in runs:
                    if kind == "flash":
                        K.attention_fwd(q[r0:r1].unsqueeze(0), k[r0:r1].unsqueeze(0), v[r0:r1].unsqueeze(0), causal=True,
                                        out=att[r0:r1].unsqueeze(0))
                    else:
                        I.paged_attention(q[r0:r1], self.k_cache[l], self.v_cache[l], self.block_table, rseq[r0:r1],
                                          ctx_len[r0:r1], att[r0:r1], block_size=bs, kv_heads=Hl,
                                          k_scale=self.k_scale[l], v_scale=self.v_scale[l], kv_kind=self.kv_kind,
                                          splits=self._splits(r1 - r0))
            else:
                self._ref_attention(l, q, k, v, slot, rseq, ctx_len, att)
            att2 = att.view(N, dl)
            if self.tp == 1:
                x = self._linear(att2, lw["proj"], residual=x)
            else:
                part = self._linear(att2, lw["proj"], out_dtype=torch.float32)
                x = x + self._all_reduce(part.float())
            h2 = self._norm(x, lw["ln2_w"], lw["ln2_b"])
            f = self._linear(h2, lw["fc"], act="gelu")
            if self.tp == 1:
                x = self._linear(f, lw["fc2"], residual=x)
            else:
                part = self._linear(f, lw["fc2"], out_dtype=torch.float32)
                x = x + self._all_reduce(part.float())
            if cap is not None:
                cap.append(x.detach().float().cpu())
        R = logit_rows.shape[0]
        if R == 0:
            return torch.zeros((0, self.Vp), dtype=torch.float32, device=self.dev)
        xr = x.index_select(0, logit_rows.long()) if not self.fast else x[logit_rows.long()]
        hf = self._norm(xr, self.lnf_w, self.lnf_b)
        if not self.fast:
            return hf @ self.wte.t()
        if R <= self._skinny:
            return I.skinny_gemm(hf, self.wte, out_dtype=torch.float32)
        return K.gemm(hf, self.wte, out_dtype=torch.float32)

    def _splits(self, rows: int) -> int:
        if self.cfg.decode_splits > 0:
            return self.cfg.decode_splits
        ctas = rows * max(self.Hl, 1)
        return 1 if ctas >= 296 else max(1, min(16, 592 // max(ctas, 1)))

    def _ref_attention(self, l, q, k, v, slot, rseq, ctx_len, att) -> None:
        """PyTorch reference of kv_append + paged attention (FP32; optional INT8 KV)."""
        bs, Hl, D = self.cfg.block_size, self.Hl, self.D
        kc, vc = self.k_cache[l].view(-1, Hl, D), self.v_cache[l].view(-1, Hl, D)
        sl = slot.long()
        ok = sl >= 0
        if self.kv_kind == 1:
            for src, cache, scale in ((k, kc, self.k_scale[l]), (v, vc, self.v_scale[l])):
                am = src.abs().amax(-1)
                sc = torch.where(am > 0, am / 127.0, torch.ones_like(am))
                cache[sl[ok]] = torch.round(src / sc[..., None]).clamp(-127, 127).to(torch.int8)[ok]
                scale[sl[ok]] = sc[ok]
        else:
            kc[sl[ok]] = k[ok].to(kc.dtype)
            vc[sl[ok]] = v[ok].to(vc.dtype)
        scale = D ** -0.5
        for r in range(q.shape[0]):
            n = int(ctx_len[r])
            if n == 0:
                att[r] = 0
                continue
            blocks = self.block_table[int(rseq[r]), : -(-n // bs)].long()
            idx = (blocks[:, None] * bs + torch.arange(bs, device=self.dev)[None, :]).reshape(-1)[:n]
            kk, vv = kc[idx].float(), vc[idx].float()
            if self.kv_kind == 1:
                kk, vv = kk * self.k_scale[l][idx][..., None], vv * self.v_scale[l][idx][..., None]
            s = torch.einsum("hd,nhd->hn", q[r].float(), kk) * scale
            att[r] = torch.einsum("hn,nhd->hd", s.softmax(-1), vv).to(att.dtype)

    def _stage(self, width: int) -> torch.Tensor:
        """Host staging tensor [6, width] int32 (pinned on a GPU), one per width, reused by every step."""
        t = self._stage_bufs.get(width)
        ev = self._stage_evt.get(width)
        if ev is not None:
            ev.synchronize()          # the copy that last read this buffer has run
        if t is None:
            t = torch.zeros((6, width), dtype=torch.int32)
            if self.dev.type == "cuda":
                t = t.pin_memory()
            if len(self._stage_bufs) > 64:
                self._stage_bufs.clear()
                self._stage_evt.clear()
            self._stage_bufs[width] = t
        return t

    # ----------------------------------------------------------------------------- decode graphs
    def _decode_graph(self, bucket: int, ints: torch.Tensor, device_rows: int = 0) -> torch.Tensor:
        st = self._static.get(bucket)
        if st is None:
            st = {"ints": torch.zeros((6, bucket), dtype=torch.int32, device=self.dev)}
            st["ints"][2].fill_(-1)
            self._static[bucket] = st
            runs = [("paged", 0, bucket, -1)]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):    # warm-up outside capture: lazy allocations, scratch growth
                st["ints"].copy_(ints, non_blocking=True)
                i = st["ints"]
                self._body(i[0], i[1], i[2], i[3], i[4], i[5], runs, self.L)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                i = st["ints"]
                st["logits"] = self._body(i[0], i[1], i[2], i[3], i[4], i[5], runs, self.L)
            self._graphs[bucket] = g
        st["ints"].copy_(ints, non_blocking=True)
        if device_rows:   # tokens drawn by the previous step, still only on the device
            st["ints"][0, :device_rows] = self._last_tok[st["ints"][3, :device_rows].long()]
        self._graphs[bucket].replay()
        return st["logits"]

    def release_graphs(self) -> None:
        """Drops every captured decode graph and its static buffers.  A tensor-parallel engine must do this before its
        process group is destroyed: tearing the communicator down while graphs that captured its collectives are alive
        did not return."""
        if self.dev.type == "cuda":
            torch.cuda.synchronize()
        self._graphs.clear()
        self._static.clear()
        if self.dev.type == "cuda":
            torch.cuda.synchronize()

    # ----------------------------------------------------------------------------- outputs
    def logit_rows(self) -> int:
        return 0 if self._logits is None else self._logits.shape[0]

    def vocab(self) -> int:
        return self.V

    def vocab_padded(self) -> int:
        return self.Vp

    def logits_host(self, row: int) -> torch.Tensor:
        return self._logits[row, : self.V].float().cpu()

    def sample(self, params: Sequence[SamplingParams], seqs: Optional[Sequence[int]] = None, offsets=0,
               pending: bool = False):
        """One token per logit row.  ``offsets``: Philox counter per row (or one value for all rows);
        using the request's own token index makes a request's draws independent of the batch.

        ``pending``: nothing is read back; the tokens stay in the device table that
        ``forward(device_tokens=True)`` reads, an asynchronous copy into pinned memory is started, and the returned
        ``PendingTokens`` is turned into the list by ``collect`` later."""
        R = self.logit_rows()
        if len(params) != R:
            raise ValueError(f"sample: {len(params)} parameter sets for {R} logit rows")
        seqs = list(seqs) if seqs is not None else list(self._logit_seq)
        offs = [int(offsets)] * R if isinstance(offsets, int) else [int(o) for o in offsets]
        if self.fast:
            from ..ops import _infer as I
            # the packed parameter block of an unchanged set of requests stays on the device
            key = tuple((id(p), p.temperature, p.top_k, p.top_p, p.min_p, p.repetition_penalty, p.frequency_penalty,
                         p.presence_penalty, p.seed) for p in params)
            cached = self._sample_cache.get("params")
            if cached is None or cached[0] != key:
                need = any(p.repetition_penalty != 1.0 or p.frequency_penalty or p.presence_penalty for p in params)
                cached = (key, I.pack_sample_params(params).to(self.dev, non_blocking=True), need)
                self._sample_cache["params"] = cached
            _, pd, need_counts = cached
            # offsets (uint64) and count rows (int32) travel in one pinned staging tensor
            st = self._sample_cache.get(R)
            if st is None:
                st = torch.zeros(3 * R, dtype=torch.int32)
                st = st.pin_memory() if self.dev.type == "cuda" else st
                self._sample_cache[R] = st
            hn = st.numpy()
            hn[: 2 * R].view("int64")[:] = offs
            hn[2 * R:] = seqs
            dvs = st.to(self.dev, non_blocking=True)
            od, rows = dvs[: 2 * R].view(torch.int64), dvs[2 * R:]
            out = I.sample(self._logits, pd, od, vocab=self.V, counts_all=self.counts_all if need_counts else None,
                           counts_out=self.counts_out if need_counts else None, count_row=rows)
            o32 = out.to(torch.int32)
            self._last_tok.index_copy_(0, rows.long(), o32)      # the table forward(device_tokens=True) reads
            if pending:
                pin = self._tok_pins[self._tok_pin_next % len(self._tok_pins)]
                self._tok_pin_next += 1
                pin[:R].copy_(o32, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                return PendingTokens(ev, pin, R, seqs)
            return out.cpu().tolist()
        from .sampling import sample_reference
        toks = [sample_reference(self._logits[r, : self.V].float().cpu(), params[r], self.counts_all[seqs[r]].cpu(),
                                 self.counts_out[seqs[r]].cpu(), offs[r]) for r in range(R)]
        t32 = torch.tensor(toks, dtype=torch.int32, device=self.dev)
        self._last_tok.index_copy_(0, torch.tensor(seqs, dtype=torch.long, device=self.dev), t32)
        if pending:   # reference path: nothing is asynchronous, the handle only defers the hand-over
            return PendingTokens(None, t32.cpu(), R, seqs)
        return toks

    def collect(self, pending: "PendingTokens") -> List[int]:
        """Waits for the tokens of a ``sample(..., pending=True)`` call and completes the host-side token lists of the
        sequences that were fed from the device table since."""
        if pending.event is not None:
            pending.event.synchronize()
        toks = [int(t) for t in pending.pinned[: pending.rows].tolist()]
        for seq, t in zip(pending.seqs, toks):
            idx = self._patch.pop(seq, None)
            if idx is not None:
                self.sched.patch(seq, idx, t)       # no-op when the sequence is gone or the slot was filled already
        return toks

    def nll(self, targets: Sequence[int]) -> List[float]:
        t = torch.tensor(list(targets), dtype=torch.int32, device=self.dev)
        if self.fast:
            from ..ops import _infer as I
            return [float(x) for x in I.nll(self._logits, t, self.V).cpu()]
        lg = self._logits[:, : self.V].float()
        return [float(x) for x in (lg.logsumexp(-1) - lg.gather(1, t.long()[:, None])[:, 0]).cpu()]

    def last_step(self) -> StepStats:
        return self._stats

    def weight_bytes(self) -> int:
        return self.weight_nbytes

    def kv_bytes_per_token(self) -> int:
        return self._kv_tok_bytes

    def layers_count(self) -> int:
        return self.L

    def graphs_captured(self) -> int:
        return len(self._graphs)

    def config(self) -> EngineConfig:
        return self.cfg

    def impl_capture(self, capture: Optional[list]) -> None:
        """Test hook: when set, every layer's residual stream is appended to ``capture``."""
        self._capture = capture


# ------------------------------------------------------------------------------------------ generation
@dataclass
class GenerateStats:
    ttft_ms: float = 0.0
    tpot_ms: float = 0.0
    tokens: int = 0


def _sync(engine: Engine) -> None:
    if engine.dev.type == "cuda":
        torch.cuda.synchronize(engine.dev)


def generate(engine: Engine, prompt: Sequence[int], max_new: int, sp: Optional[SamplingParams] = None,
             stats: Optional[GenerateStats] = None, stop_token: Optional[int] = None) -> List[int]:
    sp = sp or SamplingParams(temperature=0.0)
    seq = engine.add_sequence()
    out: List[int] = []
    try:
        t0 = time.perf_counter()
        engine.forward([Chunk(seq, list(prompt), 1, False)])
        tok = engine.sample([sp], [seq], len(prompt))[0]
        t1 = time.perf_counter()
        out.append(tok)
        while len(out) < max_new and tok != stop_token and engine.length(seq) < engine.ctx:
            engine.forward([Chunk(seq, [tok], 1, True)])
            tok = engine.sample([sp], [seq], len(prompt) + len(out))[0]
            out.append(tok)
        _sync(engine)
        t2 = time.perf_counter()
        if stats is not None:
            stats.ttft_ms = (t1 - t0) * 1e3
            stats.tpot_ms = (t2 - t1) * 1e3 / max(1, len(out) - 1)
            stats.tokens = len(out)
    finally:
        engine.free_sequence(seq)
    return out


@dataclass
class SpecStats:
    steps: int = 0            # target verification passes
    drafted: int = 0
    accepted: int = 0
    tokens_per_step: float = 0.0
    ms: float = 0.0


def speculative_generate(engine: Engine, prompt: Sequence[int], max_new: int, draft_layers: int, gamma: int,
                         stats: Optional[SpecStats] = None) -> List[int]:
    """Greedy speculative decoding; the draft model is the first ``draft_layers`` layers of the target
    (shared KV pages; verification rewrites the drafted positions in every layer).  The output equals
    greedy decoding token for token."""
    greedy = SamplingParams(temperature=0.0)
    seq = engine.add_sequence()
    out: List[int] = []
    st = SpecStats()
    t0 = time.perf_counter()
    try:
        engine.forward([Chunk(seq, list(prompt), 1, False)])
        tok = engine.sample([greedy], [seq], 0)[0]
        out.append(tok)
        while len(out) < max_new:
            base = engine.length(seq)
            g = min(gamma, max_new - len(out), engine.ctx - base - 1)
            if g <= 0:
                engine.forward([Chunk(seq, [out[-1]], 1, True)])
                out.append(engine.sample([greedy], [seq], 0)[0])
                st.steps += 1
                continue
            draft = []
            cur = out[-1]
            for _ in range(g):
                engine.forward([Chunk(seq, [cur], 1, True)], layers=draft_layers)
                cur = engine.sample([greedy], [seq], 0)[0]
                draft.append(cur)
            engine.truncate(seq, base)
            engine.forward([Chunk(seq, [out[-1]] + draft, g + 1, True)])
            target = engine.sample([greedy] * (g + 1), [seq] * (g + 1), 0)
            n_ok = 0
            while n_ok < g and draft[n_ok] == target[n_ok]:
                n_ok += 1
            accepted = draft[:n_ok] + [target[n_ok]]
            engine.truncate(seq, base + 1 + n_ok)
            out.extend(accepted)
            st.steps += 1
            st.drafted += g
            st.accepted += n_ok
        out = out[:max_new]
    finally:
        engine.free_sequence(seq)
    _sync(engine)
    st.ms = (time.perf_counter() - t0) * 1e3
    st.tokens_per_step = len(out) / max(1, st.steps)
    if stats is not None:
        stats.__dict__.update(st.__dict__)
    return out
