"""Rotary position embedding: inverse-frequency tables for six scaling schemes and the rotate-half
application (partial rotary supported).

Parity: include/nexus/lm/rope.hpp:6-21 and src/lm/rope.cpp of the reference (`rope_inv_freq`,
`RopeCache`; formulas identical to HF transformers' ``rope_scaling`` implementations).
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

from .config import LmConfig, RopeScaling


def rope_inv_freq(rot_dim: int, theta: float, scaling: RopeScaling, max_position: int,
                  seq_len: int = 0) -> Tuple[torch.Tensor, float]:
    """Returns (inv_freq [rot_dim/2] float64->float32, attention scaling factor)."""
    half = rot_dim // 2
    idx = torch.arange(0, half, dtype=torch.float64)
    base = float(theta)
    t = scaling.type
    orig = scaling.original_max_position or max_position
    factor = float(scaling.factor)
    attn = 1.0
    if t == "ntk":
        base = base * factor ** (rot_dim / (rot_dim - 2))
    elif t == "dynamic":
        sl = max(seq_len, orig)
        if sl > orig:
            base = base * ((factor * sl / orig) - (factor - 1.0)) ** (rot_dim / (rot_dim - 2))
    inv = 1.0 / (base ** (2.0 * idx / rot_dim))
    if t == "linear":
        inv = inv / factor
    elif t == "yarn":
        def corr_dim(rot):
            return (rot_dim * math.log(orig / (rot * 2 * math.pi))) / (2 * math.log(base))
        low = max(math.floor(corr_dim(scaling.beta_fast)), 0)
        high = min(math.ceil(corr_dim(scaling.beta_slow)), rot_dim - 1)
        if low == high:
            high += 0.001
        ramp = torch.clamp((torch.arange(half, dtype=torch.float64) - low) / (high - low), 0, 1)
        extrap = 1.0 - ramp
        inv = (inv / factor) * (1 - extrap) + inv * extrap
        attn = scaling.attention_factor if scaling.attention_factor > 0 else 0.1 * math.log(factor) + 1.0
    elif t == "llama3":
        low_wl = orig / scaling.low_freq_factor
        high_wl = orig / scaling.high_freq_factor
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > low_wl, inv / factor, inv)
        smooth = (orig / wavelen - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)
        smoothed = (1 - smooth) * inv / factor + smooth * inv
        medium = ~(wavelen < high_wl) & ~(wavelen > low_wl)
        inv = torch.where(medium, smoothed, scaled)
    return inv.to(torch.float32), float(attn)


class RopeCache:
    """cos/sin tables [max_position, rot_dim/2] for a config."""

    def __init__(self, config: LmConfig, device="cpu", seq_len: int = 0):
        self.rot_dim = config.rot_dim()
        inv, self.attention_factor = rope_inv_freq(self.rot_dim, config.rope_theta, config.rope_scaling,
                                                   config.max_position, seq_len)
        n = max(config.max_position, seq_len)
        ang = torch.arange(n, dtype=torch.float32)[:, None] * inv[None]
        self.cos = (ang.cos() * self.attention_factor).to(device)
        self.sin = (ang.sin() * self.attention_factor).to(device)

    def to(self, device):
        self.cos, self.sin = self.cos.to(device), self.sin.to(device)
        return self


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor = None,
               inverse: bool = False) -> torch.Tensor:
    """Rotate-half RoPE on x [B, T, H, D]; cos/sin [P, rot/2]; positions [B, T] or None (0..T-1).
    ``inverse`` applies the transpose rotation (the backward of the forward rotation)."""
    B, T, H, D = x.shape
    half = cos.shape[1]
    rot = 2 * half
    if positions is None:
        c, s = cos[:T][None, :, None, :], sin[:T][None, :, None, :]
    else:
        c, s = cos[positions.long()][:, :, None, :], sin[positions.long()][:, :, None, :]
    if inverse:
        s = -s
    xf = x.float()
    x1, x2 = xf[..., :half], xf[..., half:rot]
    o1 = x1 * c - x2 * s
    o2 = x2 * c + x1 * s
    out = torch.cat([o1, o2, xf[..., rot:]], dim=-1) if rot < D else torch.cat([o1, o2], dim=-1)
    return out.to(x.dtype)


def alibi_slopes(n_head: int) -> torch.Tensor:
    """Per-head ALiBi slopes (geometric sequence; the usual interleave for non powers of two)."""
    def pow2(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(n_head).is_integer():
        return torch.tensor(pow2(n_head), dtype=torch.float32)
    closest = 2 ** math.floor(math.log2(n_head))
    extra = pow2(2 * closest)[0::2][: n_head - closest]
    return torch.tensor(pow2(closest) + extra, dtype=torch.float32)
