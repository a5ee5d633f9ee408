"""Host reference of the single-kernel sampler (same rules, FP64 accumulation): penalties, temperature,
top-k, top-p, min-p, one Philox4x32-10 draw per row; ``temperature <= 0`` is greedy with ties going to
the lowest id.  Parity: src/cuda/infer_kernels.cu:292 (`sample_kernel`) of the reference."""
from __future__ import annotations

import numpy as np
import torch


def philox_uniform_scalar(seed: int, offset: int) -> float:
    """First lane of Philox block ``offset`` under key ``seed``, top 24 bits -> [0, 1)."""
    try:
        from .. import _native
        return float(_native.philox_uniform(1, int(seed), int(offset))[0])
    except ImportError:
        m32 = 0xFFFFFFFF
        c = [offset & m32, (offset >> 32) & m32, 0, 0]
        k0, k1 = seed & m32, (seed >> 32) & m32
        for _ in range(10):
            p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
            c = [((p1 >> 32) ^ c[1] ^ k0) & m32, p1 & m32, ((p0 >> 32) ^ c[3] ^ k1) & m32, p0 & m32]
            k0, k1 = (k0 + 0x9E3779B9) & m32, (k1 + 0xBB67AE85) & m32
        return (c[0] >> 8) / 16777216.0


def apply_penalties(logits: np.ndarray, p, counts_all=None, counts_out=None) -> np.ndarray:
    v = logits.astype(np.float32).copy()
    if counts_all is not None and p.repetition_penalty != 1.0:
        seen = np.asarray(counts_all) > 0
        v[seen] = np.where(v[seen] > 0, v[seen] / np.float32(p.repetition_penalty),
                           v[seen] * np.float32(p.repetition_penalty))
    if counts_out is not None and (p.frequency_penalty or p.presence_penalty):
        n = np.asarray(counts_out)
        hit = n > 0
        v[hit] -= (np.float32(p.frequency_penalty) * n[hit] + np.float32(p.presence_penalty)).astype(np.float32)
    return v


def kept_mass(logits, p, counts_all=None, counts_out=None):
    """Unnormalised probabilities e = exp(v - max) with every filtered-out token set to 0."""
    v = apply_penalties(np.asarray(logits, dtype=np.float32), p, counts_all, counts_out)
    v = v * np.float32(1.0 / p.temperature)
    e = np.exp((v - v.max()).astype(np.float64))
    thr = p.min_p if p.min_p > 0 else 0.0
    if 0 < p.top_k < e.size:
        thr = max(thr, np.sort(e)[-p.top_k])
    if 0.0 < p.top_p < 1.0:
        order = np.sort(e)[::-1]
        cum = np.cumsum(order)
        idx = int(np.searchsorted(cum, p.top_p * cum[-1], side="left"))
        thr = max(thr, order[min(idx, e.size - 1)])
    return np.where(e >= thr, e, 0.0)


def sample_reference(logits, p, counts_all=None, counts_out=None, offset: int = 0) -> int:
    logits = logits.numpy() if isinstance(logits, torch.Tensor) else np.asarray(logits)
    ca = counts_all.numpy() if isinstance(counts_all, torch.Tensor) else counts_all
    co = counts_out.numpy() if isinstance(counts_out, torch.Tensor) else counts_out
    if p.temperature <= 0:
        v = apply_penalties(logits, p, ca, co)
        return int(np.argmax(v))          # numpy returns the first (lowest-id) maximum
    e = kept_mass(logits, p, ca, co)
    u = philox_uniform_scalar(p.seed, offset)
    cum = np.cumsum(e)
    target = u * cum[-1]
    idx = int(np.searchsorted(cum, target, side="right"))
    idx = min(idx, e.size - 1)
    while e[idx] == 0.0 and idx > 0:      # numerical edge: fall back to the last kept token
        idx -= 1
    return idx
