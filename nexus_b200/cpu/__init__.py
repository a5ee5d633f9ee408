"""CPU runtime: feature / topology detection, the persistent thread pool with a deterministic static
partition, FP32 and quantised (INT8, INT4 group-wise) GEMM whose results are bit-identical across thread
counts, the AdamW kernel for optimizer offload (no FMA, same op order as the GPU kernel) and the FP64
attention oracle.
Parity: include/nexus/cpu/{features,threads,gemm,adam}.hpp, include/nexus/attention/*.hpp of the reference."""
from __future__ import annotations

from typing import Optional

import numpy as np

from .. import _native as N

ThreadPool = N.ThreadPool
PackedWeights = N.PackedWeights


def features() -> dict:
    return dict(N.cpu_features())


_pool: Optional[ThreadPool] = None


def pool(workers: int = 0) -> ThreadPool:
    """Process-wide pool, one worker per physical core by default."""
    global _pool
    if _pool is None or (workers and _pool.size != workers):
        _pool = ThreadPool(workers or int(features()["physical_cores"]))
    return _pool


def gemm_nt(x, w, bias=None, threads: int = 0) -> np.ndarray:
    """x [m, k] @ w[n, k]^T (+ bias)."""
    return N.cpu_gemm_nt(pool(threads), np.ascontiguousarray(x, np.float32), np.ascontiguousarray(w, np.float32), bias)


def to_bf16_bits(w) -> np.ndarray:
    """FP32 -> BF16 bit patterns (uint16, round to nearest even)."""
    u = np.ascontiguousarray(w, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def gemm_nt_bf16(x, w_bits, bias=None, threads: int = 0) -> np.ndarray:
    """x [m, k] @ w[n, k]^T (+ bias) with the weights stored as BF16 bit patterns (`to_bf16_bits`)."""
    return N.cpu_gemm_nt_bf16(pool(threads), np.ascontiguousarray(x, np.float32), np.ascontiguousarray(w_bits, np.uint16), bias)


def flash_attention(q, k, v, causal=True, window=0, scale=None, softcap=0.0, alibi=None, threads: int = 0):
    """Blocked attention on the CPU (online softmax over 64-key blocks, no [Tq, Tk] matrix): q [B, Tq, H, D],
    k / v [B, Tk, Hkv, D] FP32; causal with the last query aligned to the last key, sliding window, soft-capping,
    ALiBi slopes, grouped-query heads.  Returns (o [B, Tq, H, D], lse [B, H, Tq]).
    Parity: include/nexus/attention/cpu.hpp:42-47 of the reference (`flash_attention_forward` with `AttentionParams`)."""
    q = np.ascontiguousarray(q, np.float32)
    sc = float(scale) if scale is not None else q.shape[-1] ** -0.5
    al = np.zeros(0, np.float32) if alibi is None else np.ascontiguousarray(alibi, np.float32)
    return N.cpu_flash_attention(pool(threads), q, np.ascontiguousarray(k, np.float32), np.ascontiguousarray(v, np.float32),
                                 bool(causal), int(window), sc, float(softcap), al)


def pack_weights(w, bits: int = 8, group: int = 32) -> PackedWeights:
    return N.pack_weights(np.ascontiguousarray(w, np.float32), bits, group)


def quant_gemm(x, packed: PackedWeights, threads: int = 0) -> np.ndarray:
    return N.cpu_quant_gemm(pool(threads), np.ascontiguousarray(x, np.float32), packed)


def adamw_range(p, g, m, v, lr, wd, beta1, beta2, eps, inv_bias1, inv_bias2, clip=1.0) -> None:
    """In-place AdamW on FP32 arrays (optimizer offload); bit-equal to the GPU kernel for FP32 gradients."""
    N.adamw_range(p, g, m, v, lr, wd, beta1, beta2, eps, inv_bias1, inv_bias2, clip)


def sq_norm(x) -> float:
    return float(N.sq_norm(np.ascontiguousarray(x, np.float32)))


def math_attention(q, k, v, causal=True, window=0, scale=1.0, softcap=0.0):
    """FP64 reference attention ([B, T, H, D] layout)."""
    return N.math_attention(q, k, v, causal=causal, window=window, scale=scale, softcap=softcap)
