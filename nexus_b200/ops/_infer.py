"""ctypes bindings of the inference kernels (``csrc/cuda/infer_kernels.cu``): paged KV cache append,
paged decode attention, skinny GEMM, row gather, sampler, token counts, NLL, RoPE, gated activations and
weight-only quantisation.  Every wrapper launches on the current torch CUDA stream."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _cuda as K

KV_BF16, KV_INT8, KV_FP8 = 0, 1, 2


class PagedArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_row_stride", C.c_int64), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("k_scale", C.c_void_p), ("v_scale", C.c_void_p), ("block_table", C.c_void_p),
                ("row_seq", C.c_void_p), ("ctx_len", C.c_void_p), ("out", C.c_void_p), ("o_row_stride", C.c_int64),
                ("part_o", C.c_void_p), ("part_ml", C.c_void_p), ("scale", C.c_float), ("rows", C.c_int),
                ("heads", C.c_int), ("kv_heads", C.c_int), ("head_dim", C.c_int), ("block_size", C.c_int),
                ("max_blocks", C.c_int), ("splits", C.c_int), ("kv_kind", C.c_int), ("num_blocks", C.c_int),
                ("status", C.c_void_p)]


class SampleParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float),
                ("repetition_penalty", C.c_float), ("frequency_penalty", C.c_float), ("presence_penalty", C.c_float),
                ("top_k", C.c_int), ("pad", C.c_int), ("seed", C.c_uint64)]


def skinny_max_rows() -> int:
    return int(K.lib().nx_skinny_max_rows())


def kv_append(k, v, slots, k_cache, v_cache, *, k_scale=None, v_scale=None, kv_kind=KV_BF16) -> None:
    """k/v: [tokens, kv_heads, D] (row-strided views allowed); slots: int32 [tokens]."""
    tokens, hk, d = k.shape
    K._check(K.lib().nx_kv_append(K._p(k), K._p(v), C.c_int64(k.stride(0)), C.c_int64(v.stride(0)), K._p(slots),
                                  K._p(k_cache), K._p(v_cache), K._p(k_scale), K._p(v_scale), C.c_int(tokens),
                                  C.c_int(hk), C.c_int(d), C.c_int(kv_kind), K._stream()), "nx_kv_append")


def paged_attention(q, k_cache, v_cache, block_table, row_seq, ctx_len, out, *, block_size, kv_heads, scale=None,
                    k_scale=None, v_scale=None, kv_kind=KV_BF16, splits=1) -> torch.Tensor:
    """q/out: [rows, heads, D] (row-strided views allowed).  Row r attends to the first ``ctx_len[r]``
    cached tokens of sequence ``row_seq[r]``."""
    rows, heads, d = q.shape
    a = PagedArgs()
    a.q, a.q_row_stride = q.data_ptr(), q.stride(0)
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.k_scale = k_scale.data_ptr() if k_scale is not None else None
    a.v_scale = v_scale.data_ptr() if v_scale is not None else None
    a.block_table, a.row_seq, a.ctx_len = block_table.data_ptr(), row_seq.data_ptr(), ctx_len.data_ptr()
    a.out, a.o_row_stride = out.data_ptr(), out.stride(0)
    a.scale = scale if scale is not None else d ** -0.5
    a.rows, a.heads, a.kv_heads, a.head_dim = rows, heads, kv_heads, d
    a.block_size, a.max_blocks, a.splits, a.kv_kind = block_size, block_table.shape[1], splits, kv_kind
    a.num_blocks = k_cache.shape[0] if k_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() else 0
    a.status = K.status_word(q.device).data_ptr()
    if splits > 1:
        po = K.scratch(rows * heads * splits * d * 4, "paged_o", q.device)
        pm = K.scratch(rows * heads * splits * 8, "paged_ml", q.device)
        a.part_o, a.part_ml = po.data_ptr(), pm.data_ptr()
    K._check(K.lib().nx_paged_attention_decode(C.byref(a), K._stream()), "nx_paged_attention_decode")
    return out


def skinny_gemm(x, w, bias=None, *, act=None, residual=None, out=None, out_dtype=None) -> torch.Tensor:
    """y = act(x @ w^T + bias) + residual for 1 <= rows <= skinny_max_rows(); w is [n, k]."""
    m, k = x.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or (residual.dtype if residual is not None else x.dtype),
                          device=x.device)
    if residual is not None and residual.dtype != out.dtype:
        raise ValueError("skinny_gemm: residual and output dtypes differ")
    K._check(K.lib().nx_skinny_gemm(K._p(x), C.c_int64(x.stride(0)), K._p(w), C.c_int64(w.stride(0)), K._p(bias),
                                    K._p(residual), C.c_int64(residual.stride(0) if residual is not None else 0),
                                    K._p(out), C.c_int64(out.stride(0)), C.c_int(K._DT[out.dtype]), C.c_int(m),
                                    C.c_int(n), C.c_int(k), C.c_int(K.ACT[act]), K._stream()), "nx_skinny_gemm")
    return out


def gather_rows(x, rows, out=None) -> torch.Tensor:
    n, cols = rows.numel(), x.shape[1]
    out = torch.empty((n, cols), dtype=x.dtype, device=x.device) if out is None else out
    K._check(K.lib().nx_gather_rows(K._p(x), K._p(rows), K._p(out), C.c_int(n), C.c_int(cols), K._stream()),
             "nx_gather_rows")
    return out


def count_tokens(tokens, row_of, counts) -> None:
    K._check(K.lib().nx_count_tokens(K._p(tokens), K._p(row_of), K._p(counts), C.c_int(tokens.numel()),
                                     C.c_int(counts.shape[1]), K._stream()), "nx_count_tokens")


def nll(logits, targets, vocab: Optional[int] = None) -> torch.Tensor:
    rows = logits.shape[0]
    out = torch.empty(rows, dtype=torch.float32, device=logits.device)
    K._check(K.lib().nx_nll(K._p(logits), C.c_int64(logits.stride(0)), K._p(targets), K._p(out), C.c_int(rows),
                            C.c_int(vocab or logits.shape[1]), K._stream()), "nx_nll")
    return out


def pack_sample_params(params) -> torch.Tensor:
    """params: iterable of objects with the SamplingParams fields -> uint8 host tensor (pinned if possible)."""
    arr = (SampleParams * len(params))()
    for i, p in enumerate(params):
        arr[i].temperature, arr[i].top_p, arr[i].min_p = p.temperature, p.top_p, p.min_p
        arr[i].repetition_penalty, arr[i].frequency_penalty = p.repetition_penalty, p.frequency_penalty
        arr[i].presence_penalty, arr[i].top_k, arr[i].seed = p.presence_penalty, p.top_k, p.seed
    return torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)


def sample(logits, params_dev, offsets, *, vocab=None, counts_all=None, counts_out=None, count_row=None,
           out=None) -> torch.Tensor:
    """logits: FP32 [rows, ld]; params_dev: device copy of ``pack_sample_params``; offsets: uint64 [rows]."""
    rows = logits.shape[0]
    v = vocab or logits.shape[1]
    work = K.scratch(rows * v * 4, "sample_work", logits.device)
    out = torch.empty(rows, dtype=torch.int32, device=logits.device) if out is None else out
    K._check(K.lib().nx_sample(K._p(logits), C.c_int64(logits.stride(0)), C.c_int(v), K._p(params_dev),
                               K._p(counts_all), K._p(counts_out), K._p(count_row), K._p(offsets), K._p(work),
                               K._p(out), C.c_int(rows), K._stream()), "nx_sample")
    return out


def rope_(x, positions, cos_t, sin_t, *, rot_dim=None, inverse=False, interleaved=False) -> torch.Tensor:
    """In-place rotary embedding on x [rows, heads, D] (row-strided view allowed)."""
    rows, heads, d = x.shape
    K._check(K.lib().nx_rope(K._p(x), C.c_int64(x.stride(0)), K._p(positions), K._p(cos_t), K._p(sin_t),
                             C.c_int(rows), C.c_int(heads), C.c_int(d), C.c_int(rot_dim or d), C.c_int(int(inverse)),
                             C.c_int(int(interleaved)), K._stream()), "nx_rope")
    return x


def gated_fwd(h, act: str = "silu") -> torch.Tensor:
    n, f2 = h.shape
    y = torch.empty((n, f2 // 2), dtype=h.dtype, device=h.device)
    K._check(K.lib().nx_gated_fwd(K._p(h), K._p(y), C.c_int64(n), C.c_int(f2 // 2), C.c_int(0 if act == "silu" else 1),
                                  K._stream()), "nx_gated_fwd")
    return y


def gated_bwd(h, dy, act: str = "silu") -> torch.Tensor:
    n, f2 = h.shape
    dh = torch.empty_like(h)
    K._check(K.lib().nx_gated_bwd(K._p(h), K._p(dy), K._p(dh), C.c_int64(n), C.c_int(f2 // 2),
                                  C.c_int(0 if act == "silu" else 1), K._stream()), "nx_gated_bwd")
    return dh


def wq_gemv(x, wq, scales, *, bits, group=128, bias=None, out=None) -> torch.Tensor:
    m, k = x.shape
    n = wq.shape[0]
    out = torch.empty((m, n), dtype=x.dtype, device=x.device) if out is None else out
    K._check(K.lib().nx_wq_gemv(K._p(x), C.c_int64(x.stride(0)), K._p(wq), K._p(scales), C.c_int(bits), C.c_int(group),
                                K._p(bias), K._p(out), C.c_int64(out.stride(0)), C.c_int(m), C.c_int(n), C.c_int(k),
                                K._stream()), "nx_wq_gemv")
    return out


def wq_dequant(wq, scales, *, bits, group=128, k=None, out=None) -> torch.Tensor:
    n = wq.shape[0]
    k = k or (wq.shape[1] if bits == 8 else wq.shape[1] * 2)
    out = torch.empty((n, k), dtype=torch.bfloat16, device=wq.device) if out is None else out
    K._check(K.lib().nx_wq_dequant(K._p(wq), K._p(scales), C.c_int(bits), C.c_int(group), K._p(out), C.c_int(n),
                                   C.c_int(k), K._stream()), "nx_wq_dequant")
    return out


def quant_rows(x, inv_smooth=None, *, want_codes=True, want_fake=False):
    """Per-row INT8 quantisation.  Returns (codes int8 | None, fake-quant bf16 | None, row_scale f32)."""
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.int8, device=x.device) if want_codes else None
    fq = torch.empty((rows, cols), dtype=torch.bfloat16, device=x.device) if want_fake else None
    rs = torch.empty(rows, dtype=torch.float32, device=x.device)
    K._check(K.lib().nx_quant_rows(K._p(x), K._p(inv_smooth), K._p(q), K._p(fq), K._p(rs), C.c_int(rows),
                                   C.c_int(cols), K._stream()), "nx_quant_rows")
    return q, fq, rs
