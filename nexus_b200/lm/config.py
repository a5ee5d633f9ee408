"""Config-driven decoder language models: :class:`LmConfig`, presets, JSON round-trip and analytic
parameter counts.

Parity: include/nexus/lm/config.hpp:23-131 and src/lm/config.cpp (validate, count_parameters,
preset table, to_json/from_json/apply_overrides) of the reference.  Field names, enum spellings
and the preset table are the same, so configuration files move over unchanged.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field, fields
from typing import Dict, List

NORM_KINDS = ("layernorm", "rmsnorm")
MLP_KINDS = ("gelu", "swiglu", "geglu")
POS_KINDS = ("none", "sinusoidal", "learned", "rope", "alibi")
INIT_KINDS = ("gpt2", "llama", "mup")
ROPE_SCALING_TYPES = ("none", "linear", "ntk", "dynamic", "yarn", "llama3")
RECOMPUTE_KINDS = ("none", "full", "every_k")


class ConfigError(ValueError):
    pass


@dataclass
class RopeScaling:
    type: str = "none"
    factor: float = 1.0
    original_max_position: int = 0  # 0: max_position
    low_freq_factor: float = 1.0    # llama3
    high_freq_factor: float = 4.0   # llama3
    beta_fast: float = 32.0         # yarn
    beta_slow: float = 1.0          # yarn
    attention_factor: float = 0.0   # yarn; 0: 0.1 ln(factor) + 1


@dataclass
class LmConfig:
    name: str = "custom"
    vocab_size: int = 0
    n_layer: int = 0
    d_model: int = 0
    n_head: int = 0
    n_kv_head: int = 0   # 0: n_head (MHA)
    head_dim: int = 0    # 0: d_model / n_head
    d_ff: int = 0
    max_position: int = 2048
    norm: str = "rmsnorm"
    norm_eps: float = 1.0e-5
    prenorm: bool = True
    mlp: str = "swiglu"
    pos: str = "rope"
    rope_theta: float = 10000.0
    rotary_dim: int = 0  # 0: head_dim
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    tie_embeddings: bool = False
    bias: bool = False
    qkv_bias: bool = False
    qk_norm: bool = False
    parallel_block: bool = False
    window: int = 0
    attn_softcap: float = 0.0
    resid_dropout: float = 0.0
    attn_dropout: float = 0.0
    vocab_pad_multiple: int = 1
    init: str = "gpt2"
    init_std: float = 0.02
    init_truncated: bool = False
    mup_base_width: int = 256
    seed: int = 1234
    dtype: str = "float32"
    recompute: str = "none"
    recompute_every: int = 2
    moe_experts: int = 0
    moe_top_k: int = 2
    moe_every: int = 1
    moe_d_ff: int = 0
    moe_capacity_factor: float = 1.25
    moe_min_capacity: int = 4
    moe_reroute: bool = False
    moe_groups: int = 1
    moe_noisy: bool = False
    moe_shared_expert: bool = False
    moe_aux_alpha: float = 0.01
    moe_z_alpha: float = 1.0e-3

    # ---- derived -----------------------------------------------------------------------------
    def kv_heads(self) -> int:
        return self.n_kv_head if self.n_kv_head > 0 else self.n_head

    def hdim(self) -> int:
        if self.head_dim > 0:
            return self.head_dim
        return self.d_model // self.n_head if self.n_head > 0 else 0

    def rot_dim(self) -> int:
        return self.rotary_dim if self.rotary_dim > 0 else self.hdim()

    def padded_vocab(self) -> int:
        m = max(1, self.vocab_pad_multiple)
        return (self.vocab_size + m - 1) // m * m

    def gated_mlp(self) -> bool:
        return self.mlp != "gelu"

    def is_moe_layer(self, layer: int) -> bool:
        return self.moe_experts > 0 and self.moe_every > 0 and layer % self.moe_every == self.moe_every - 1

    def expert_ff(self) -> int:
        return self.moe_d_ff if self.moe_d_ff > 0 else self.d_ff


def validate(c: LmConfig) -> None:
    """Raises :class:`ConfigError` for an invalid field; nothing is silently corrected."""
    if min(c.n_layer, c.d_model, c.n_head, c.d_ff, c.max_position) < 1 or c.vocab_size < 2:
        raise ConfigError("vocab_size, n_layer, d_model, n_head, d_ff, max_position must be positive")
    for val, allowed, what in ((c.norm, NORM_KINDS, "norm"), (c.mlp, MLP_KINDS, "mlp"), (c.pos, POS_KINDS, "pos"),
                               (c.init, INIT_KINDS, "init"), (c.recompute, RECOMPUTE_KINDS, "recompute"),
                               (c.rope_scaling.type, ROPE_SCALING_TYPES, "rope_scaling.type")):
        if val not in allowed:
            raise ConfigError(f"unknown {what}: {val}")
    if c.head_dim == 0 and c.d_model % c.n_head != 0:
        raise ConfigError("head_dim must be given when d_model % n_head != 0")
    if c.n_head % c.kv_heads() != 0:
        raise ConfigError("n_head must be a multiple of n_kv_head (GQA)")
    if c.pos == "rope" and (c.rot_dim() % 2 != 0 or c.rot_dim() > c.hdim()):
        raise ConfigError("rotary_dim must be even and <= head_dim")
    if c.vocab_pad_multiple < 1:
        raise ConfigError("vocab_pad_multiple must be >= 1")
    if not (0.0 <= c.resid_dropout < 1.0 and 0.0 <= c.attn_dropout < 1.0):
        raise ConfigError("dropout must be in [0, 1)")
    if c.init == "mup" and c.mup_base_width < 1:
        raise ConfigError("mup_base_width must be >= 1")
    if c.recompute == "every_k" and c.recompute_every < 1:
        raise ConfigError("recompute_every must be >= 1")
    if c.dtype not in ("float32", "bfloat16", "float16"):
        raise ConfigError("dtype must be float32, bfloat16 or float16")
    if c.moe_experts < 0 or (c.moe_experts > 0 and (
            c.moe_top_k < 1 or c.moe_top_k > c.moe_experts or c.moe_every < 1 or c.moe_capacity_factor <= 0.0
            or c.moe_groups < 1 or c.moe_min_capacity < 0)):
        raise ConfigError("MoE: 1 <= moe_top_k <= moe_experts, moe_every >= 1, capacity_factor > 0, groups >= 1")
    if c.moe_experts > 0 and (c.mlp != "swiglu" or c.bias or c.parallel_block or not c.prenorm):
        raise ConfigError("MoE experts are SwiGLU MLPs; bias, parallel block and post-norm are not supported")
    if c.moe_experts > 0 and c.recompute != "none":
        raise ConfigError("MoE layers cannot be recomputed (routing would be re-run)")


def _mlp_params(c: LmConfig) -> int:
    d, F = c.d_model, c.d_ff
    if c.gated_mlp():
        return d * 2 * F + F * d + (2 * F + d if c.bias else 0)
    return d * F + F * d + (F + d if c.bias else 0)


def count_parameters(c: LmConfig) -> int:
    """Analytic parameter count (padded vocabulary included), no allocation."""
    validate(c)
    d, H, Hk, D, V = c.d_model, c.n_head, c.kv_heads(), c.hdim(), c.padded_vocab()
    norm = d + (d if (c.norm == "layernorm" and c.bias) else 0)
    total = V * d
    if not c.tie_embeddings:
        total += V * d
    if c.pos == "learned":
        total += c.max_position * d
    layer = (1 if c.parallel_block else 2) * norm
    layer += d * (H + 2 * Hk) * D
    if c.bias or c.qkv_bias:
        layer += (H + 2 * Hk) * D
    layer += H * D * d + (d if c.bias else 0)
    if c.qk_norm:
        layer += 2 * D
    layer += _mlp_params(c)
    total += c.n_layer * layer + norm
    Fe = c.expert_ff()
    for l in range(c.n_layer):
        if not c.is_moe_layer(l):
            continue
        if not c.moe_shared_expert:
            total -= _mlp_params(c)
        total += d * c.moe_experts * (2 if c.moe_noisy else 1) + c.moe_experts * 3 * d * Fe
    return total


def count_active_parameters(c: LmConfig) -> int:
    """Parameters touched per token: router + top-k experts (+ shared expert) in MoE layers."""
    total = count_parameters(c)
    for l in range(c.n_layer):
        if c.is_moe_layer(l):
            total -= (c.moe_experts - c.moe_top_k) * 3 * c.d_model * c.expert_ff()
    return total


# ------------------------------------------------------------------------------------------ presets
def _gpt2(name: str, L: int, d: int, H: int) -> LmConfig:
    return LmConfig(name=name, vocab_size=50257, n_layer=L, d_model=d, n_head=H, d_ff=4 * d, max_position=1024,
                    norm="layernorm", norm_eps=1e-5, mlp="gelu", pos="learned", tie_embeddings=True, bias=True,
                    init="gpt2")


def _llama_like(name, vocab, L, d, H, Hkv, ff, max_pos, theta, eps, tie=False) -> LmConfig:
    return LmConfig(name=name, vocab_size=vocab, n_layer=L, d_model=d, n_head=H, n_kv_head=Hkv, d_ff=ff,
                    max_position=max_pos, norm="rmsnorm", norm_eps=eps, mlp="swiglu", pos="rope", rope_theta=theta,
                    tie_embeddings=tie, bias=False, init="llama")


def _presets() -> Dict[str, LmConfig]:
    p: Dict[str, LmConfig] = {}
    for name, L, d, H in (("gpt2-124m", 12, 768, 12), ("gpt2-350m", 24, 1024, 16), ("gpt2-774m", 36, 1280, 20),
                          ("gpt2-1.5b", 48, 1600, 25)):
        p[name] = _gpt2(name, L, d, H)
    p["llama2-7b"] = _llama_like("llama2-7b", 32000, 32, 4096, 32, 32, 11008, 4096, 1e4, 1e-5)
    c = _llama_like("llama3-8b", 128256, 32, 4096, 32, 8, 14336, 8192, 5e5, 1e-5)
    p["llama3-8b"] = c
    c = _llama_like("mistral-7b", 32000, 32, 4096, 32, 8, 14336, 32768, 1e4, 1e-5)
    c.window = 4096
    p["mistral-7b"] = c
    for name, vocab, L, d, H, Hkv, ff, tie in (("qwen2-0.5b", 151936, 24, 896, 14, 2, 4864, True),
                                               ("qwen2-1.5b", 151936, 28, 1536, 12, 2, 8960, True),
                                               ("qwen2-7b", 152064, 28, 3584, 28, 4, 18944, False)):
        c = _llama_like(name, vocab, L, d, H, Hkv, ff, 32768, 1e6, 1e-6, tie)
        c.qkv_bias = True
        p[name] = c
    p["tinyllama-1.1b"] = _llama_like("tinyllama-1.1b", 32000, 22, 2048, 32, 4, 5632, 2048, 1e4, 1e-5)
    c = _llama_like("moe-124m", 8192, 5, 512, 8, 8, 1856, 1024, 1e4, 1e-5, True)
    c.moe_experts, c.moe_top_k = 8, 2
    p["moe-124m"] = c
    # the five benchmark configurations of this framework
    c = _gpt2("nano", 4, 128, 4)
    c.vocab_size, c.d_ff, c.max_position = 256, 512, 128
    p["nano"] = c
    c = _llama_like("moe-16l-64e", 32000, 16, 2048, 16, 16, 1408, 2048, 1e4, 1e-5)
    c.moe_experts, c.moe_top_k, c.moe_d_ff, c.moe_capacity_factor, c.moe_aux_alpha = 64, 2, 1408, 1.25, 0.01
    p["moe-16l-64e"] = c
    return p


def preset(name: str) -> LmConfig:
    table = _presets()
    if name not in table:
        raise ConfigError(f"unknown preset: {name}")
    return table[name]


def preset_names() -> List[str]:
    return list(_presets().keys())


# --------------------------------------------------------------------------------------------- JSON
def to_json(c: LmConfig, indent=None) -> str:
    return json.dumps(asdict(c), indent=indent)


def _apply(c: LmConfig, obj: dict) -> LmConfig:
    known = {f.name for f in fields(LmConfig)}
    for k, v in obj.items():
        if k not in known:
            raise ConfigError(f"unknown config key: {k}")
        if k == "rope_scaling":
            rs_known = {f.name for f in fields(RopeScaling)}
            for rk, rv in v.items():
                if rk not in rs_known:
                    raise ConfigError(f"unknown rope_scaling key: {rk}")
                setattr(c.rope_scaling, rk, rv)
        else:
            setattr(c, k, v)
    return c


def from_json(text: str) -> LmConfig:
    """Unknown keys raise; missing keys keep their defaults."""
    return _apply(LmConfig(), json.loads(text))


def apply_overrides(base: LmConfig, text: str) -> LmConfig:
    import copy

    return _apply(copy.deepcopy(base), json.loads(text))
