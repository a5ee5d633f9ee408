"""Philox4x32-10 counter-based random numbers on the host, bit-identical to the device kernels.

Element ``i`` of a stream uses counter block ``offset + i // 4`` and lane ``i % 4``; a uniform is the
top 24 bits divided by 2**24; dropout keeps an element iff ``u >= p`` and scales by ``1 / (1 - p)``.
The mask is never stored: forward and backward regenerate it from (seed, offset).

Parity: src/fused/training.cpp:321-379 of the reference (philox4x32_10, philox_uniform,
dropout_philox) and src/cuda/kernels_train.cu:322-365.
"""
from __future__ import annotations

import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    """Vectorised over counter arrays (uint32).  Returns four uint32 arrays."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint32).astype(np.uint64) for c in (c0, c1, c2, c3))
    for _ in range(10):
        p0 = M0 * c0
        p1 = M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & MASK32
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return tuple(c.astype(np.uint32) for c in (c0, c1, c2, c3))


def philox_uniform(n: int, seed: int, offset: int) -> np.ndarray:
    """``n`` float32 uniforms in [0, 1) of stream (seed, offset)."""
    nblk = (n + 3) // 4
    blk = np.arange(nblk, dtype=np.uint64) + np.uint64(offset)
    lanes = philox4x32_10((blk & MASK32).astype(np.uint32), (blk >> np.uint64(32)).astype(np.uint32),
                          np.zeros(nblk, np.uint32), np.zeros(nblk, np.uint32),
                          seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    u = np.stack(lanes, axis=1).reshape(-1)[:n]
    return ((u >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)).astype(np.float32)


def dropout_mask(n: int, p: float, seed: int, offset: int) -> np.ndarray:
    """Boolean keep-mask of the stream."""
    return philox_uniform(n, seed, offset) >= np.float32(p)
