"""Kernel micro-benchmarks with roofline fractions.

Every case is timed with CUDA events on the launching stream after warm-up; between timed launches a
buffer larger than the L2 cache is rewritten so that every launch starts cold.  Throughput is the
algorithmic FLOPs (or bytes) of the case divided by the median time, and is reported as a fraction of
the measured cuBLAS BF16 / device-copy peaks when a peaks file is given.

    python -m nexus_b200.bench.kernels [--only REGEX] [--small] [--iters N] [--peaks FILE] [--json OUT] [--library]

``--library`` adds, after each GEMM case, the same shape and operand layouts through ``torch.matmul`` /
``torch.addmm`` (cuBLASLt; BF16 output, bias in the library epilogue, no activation), so the distance
between this package's tcgen05 kernel and the vendor library is read off per shape.

``--small`` shrinks every case to a few hundred MB (still larger than L2) with one warm-up launch: the
form to run under a profiler.
"""
from __future__ import annotations

import argparse
import json
import re
import statistics
import sys
from typing import Callable, Dict, List, Tuple

import torch


def _time(fn: Callable[[], None], iters: int, warmup: int, flush: torch.Tensor) -> Tuple[float, float]:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times), min(times)


def build_cases(small: bool, library: bool = False) -> Dict[str, Tuple[Callable[[], None], float, float]]:
    """name -> (launch, flops, bytes); exactly one of flops / bytes drives the roofline."""
    from ..ops import _cuda as K
    from ..ops import _infer as I
    dev = "cuda"
    bf = torch.bfloat16
    cases: Dict[str, Tuple[Callable[[], None], float, float]] = {}
    g = torch.Generator(device=dev).manual_seed(0)

    def rn(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(dtype)

    M = 4096 if small else 16384
    C, F, V = 768, 3072, 50304

    def add_gemm(name, m, n, k, **kw):
        a_mn, b_mn = kw.get("a_mn", False), kw.get("b_mn", False)
        a = rn(k, m) if a_mn else rn(m, k)
        b = rn(k, n) if b_mn else rn(n, k)
        extra = {}
        if kw.get("bias"):
            extra["bias"] = rn(n)
        if kw.get("act"):
            extra["act"] = kw["act"]
        out = torch.zeros((m, n), dtype=torch.float32 if kw.get("acc") else bf, device=dev)
        if kw.get("acc"):
            extra.update(accumulate=True, split_k=kw.get("split_k", 1))
        cases[name] = (lambda: K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, **extra), 2.0 * m * n * k, 0.0)
        if library and not kw.get("acc"):
            # the same contraction through torch (cuBLASLt), bias in its epilogue, activation left out
            at, bt = (a.t() if a_mn else a), (b if b_mn else b.t())
            lib_out = torch.empty((m, n), dtype=bf, device=dev)
            bias = extra.get("bias")
            if bias is not None:
                cases[name + "@cublaslt"] = (lambda: torch.addmm(bias, at, bt, out=lib_out), 2.0 * m * n * k, 0.0)
            else:
                cases[name + "@cublaslt"] = (lambda: torch.matmul(at, bt, out=lib_out), 2.0 * m * n * k, 0.0)
        elif library:
            at, bt = (a.t() if a_mn else a), (b if b_mn else b.t())
            lib_acc = torch.zeros((m, n), dtype=bf, device=dev)
            cases[name + "@cublaslt"] = (lambda: torch.addmm(lib_acc, at, bt, out=lib_acc), 2.0 * m * n * k, 0.0)

    add_gemm("gemm_qkv_fwd", M, 3 * C, C, bias=True)
    add_gemm("gemm_fc_fwd_gelu", M, F, C, bias=True, act="gelu")
    add_gemm("gemm_fcproj_fwd", M, C, F, bias=True)
    add_gemm("gemm_head_fwd", M, V, C)
    add_gemm("gemm_dgrad_fc", M, C, F, b_mn=True)
    add_gemm("gemm_wgrad_fc", F, C, M, a_mn=True, b_mn=True, acc=True, split_k=2)
    add_gemm("gemm_wgrad_head", V, C, M, a_mn=True, b_mn=True, acc=True)
    if not small:
        add_gemm("gemm_8192", 8192, 8192, 8192)
    else:
        add_gemm("gemm_4096", 4096, 4096, 4096)

    # block-scaled FP8 (MX) GEMMs: Llama-7B projection shapes at 8192 tokens, and the quantiser that feeds them
    from ..ops import _lowp as L

    def add_mx(name, m, n, k, out_dtype=bf):
        aq, asf = L.mx_quantize(rn(m, k))
        bq, bsf = L.mx_quantize(rn(n, k, scale=0.05))
        cases[name] = (lambda: L.mx_gemm(aq, asf, bq, bsf, out_dtype=out_dtype), 2.0 * m * n * k, 0.0)

    mm = 2048 if small else 8192
    add_mx("mxfp8_gemm_llama_qkv", mm, 3 * 4096, 4096)
    add_mx("mxfp8_gemm_llama_ffn_up", mm, 11008, 4096)
    add_mx("mxfp8_gemm_llama_ffn_down", mm, 4096, 11008)
    add_mx("mxfp8_gemm_8192_fp8_out", mm, 8192, 8192, out_dtype=torch.float8_e4m3fn)
    xq_src = rn(mm, 4096)
    cases["mxfp8_quantize_rows"] = (lambda: L.mx_quantize(xq_src), 0.0, mm * 4096 * 3 + mm * 4096 // 32)
    cases["mxfp8_quantize_transposed"] = (lambda: L.mx_quantize(xq_src, transpose=True), 0.0, mm * 4096 * 3 + mm * 4096 // 32)

    B, H, T, D = (4 if small else 16), 12, 1024, 64
    qkv = rn(B, T, 3, H, D)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    o, lse = K.attention_fwd(q, k, v, causal=True)
    do = rn(B, T, H, D)
    fl = 4.0 * B * H * T * T * D / 2
    cases["attention_fwd_causal"] = (lambda: K.attention_fwd(q, k, v, causal=True, out=o), fl, 0.0)
    cases["attention_bwd_causal"] = (lambda: K.attention_bwd(q, k, v, o, lse, do, causal=True), 2.5 * fl, 0.0)

    # Llama-7B attention shape: head_dim 128, 4096 tokens
    B2, H2, T2, D2 = (1 if small else 2), 32, 4096, 128
    qkv2 = rn(B2, T2, 3, H2, D2)
    q2, k2, v2 = qkv2[:, :, 0], qkv2[:, :, 1], qkv2[:, :, 2]
    o2, lse2 = K.attention_fwd(q2, k2, v2, causal=True)
    do2 = rn(B2, T2, H2, D2)
    fl2 = 4.0 * B2 * H2 * T2 * T2 * D2 / 2
    cases["attention_fwd_causal_d128_t4096"] = (lambda: K.attention_fwd(q2, k2, v2, causal=True, out=o2), fl2, 0.0)
    cases["attention_bwd_causal_d128_t4096"] = (lambda: K.attention_bwd(q2, k2, v2, o2, lse2, do2, causal=True), 2.5 * fl2, 0.0)

    N = M
    x = rn(N, C, dtype=torch.float32)
    gam, bet = torch.ones(C, device=dev), torch.zeros(C, device=dev)
    cases["layernorm_fwd"] = (lambda: K.norm_fwd(x, gam, bet, out_dtype=bf), 0.0, N * C * (4 + 2) + N * 8)
    y, mean, rstd = K.norm_fwd(x, gam, bet, out_dtype=bf)
    dy = rn(N, C)
    dg, db = torch.zeros(C, device=dev), torch.zeros(C, device=dev)
    cases["layernorm_bwd"] = (lambda: K.norm_bwd(dy, x, gam, mean, rstd, dx_dtype=torch.float32, dgamma=dg, dbeta=db),
                              0.0, N * C * (2 + 4 + 4))
    rows = 2048 if small else 16384
    logits = rn(rows, V)
    toks = torch.randint(0, 50257, (rows // 1024, 1024), dtype=torch.int32, device=dev)
    cases["cross_entropy_fused"] = (lambda: K.cross_entropy_shifted(logits, toks, vocab=50257, seq_len=1024), 0.0, rows * V * 2 * 2)
    dyc = rn(N, F)
    outc = torch.zeros(F, device=dev)
    cases["bias_grad_colsum"] = (lambda: K.colsum(dyc, out=outc, accumulate=True), 0.0, N * F * 2)
    P = (16 if small else 124) * 1024 * 1024
    pm, pg = torch.zeros(P, device=dev), rn(P, dtype=torch.float32, scale=1e-3)
    m1, v1, lp = torch.zeros(P, device=dev), torch.zeros(P, device=dev), torch.zeros(P, dtype=bf, device=dev)
    st = K.opt_state_tensor(dev)
    st.copy_(torch.frombuffer(bytearray(K.pack_opt_state(lr=1e-3, weight_decay=0.1, beta1=0.9, beta2=0.95, eps=1e-8,
                                                         max_grad_norm=1.0, loss_scale=1.0)), dtype=torch.uint8))
    chunks = K.make_chunks([(0, P, 1.0, 1.0)], device=dev)
    cases["grad_norm"] = (lambda: K.grad_norm(pg, st), 0.0, P * 4)
    cases["adamw_multi_tensor"] = (lambda: K.adamw(pm, pg, m1, v1, lp, chunks, st), 0.0, P * (4 * 4 + 3 * 4 + 2))

    # inference
    nseq, ctx, bs = (16 if small else 64), 1024, 16
    nb = nseq * ctx // bs
    kc, vc = rn(nb, bs, H, D), rn(nb, bs, H, D)
    table = torch.randperm(nb, device=dev, generator=g).to(torch.int32).view(nseq, ctx // bs)
    qd = rn(nseq, H, D)
    od = torch.empty_like(qd)
    rs = torch.arange(nseq, dtype=torch.int32, device=dev)
    cl = torch.full((nseq,), ctx, dtype=torch.int32, device=dev)
    for sp in (1, 4):
        cases[f"paged_decode_attention_split{sp}"] = (
            lambda sp=sp: I.paged_attention(qd, kc, vc, table, rs, cl, od, block_size=bs, kv_heads=H, splits=sp),
            0.0, 2.0 * nseq * ctx * H * D * 2)
    # the same bytes with one head per cache row, i.e. every 16-token page of a head is one contiguous 2 KiB block
    nb1 = nseq * H * ctx // bs
    kc1, vc1 = rn(nb1, bs, 1, D), rn(nb1, bs, 1, D)
    table1 = torch.randperm(nb1, device=dev, generator=g).to(torch.int32).view(nseq * H, ctx // bs)
    qd1, od1 = rn(nseq * H, 1, D), torch.empty(nseq * H, 1, D, dtype=bf, device=dev)
    rs1 = torch.arange(nseq * H, dtype=torch.int32, device=dev)
    cl1 = torch.full((nseq * H,), ctx, dtype=torch.int32, device=dev)
    cases["paged_decode_attention_contiguous_pages"] = (
        lambda: I.paged_attention(qd1, kc1, vc1, table1, rs1, cl1, od1, block_size=bs, kv_heads=1, splits=1),
        0.0, 2.0 * nseq * ctx * H * D * 2)
    xs, ws, bsk = rn(8, C), rn(F, C, scale=0.05), rn(F)
    cases["skinny_gemm_m8"] = (lambda: I.skinny_gemm(xs, ws, bsk, act="gelu"), 0.0, F * C * 2)
    wh = rn(V, C, scale=0.05)
    cases["skinny_gemm_head_m8"] = (lambda: I.skinny_gemm(xs, wh, out_dtype=torch.float32), 0.0, V * C * 2)
    from ..infer.engine import SamplingParams
    lg = rn(64, V, dtype=torch.float32)
    pd = I.pack_sample_params([SamplingParams(temperature=0.8, top_k=50, top_p=0.9, seed=1)] * 64).to(dev)
    offs = torch.arange(64, dtype=torch.int64, device=dev)
    cases["sampler_topk_topp_64rows"] = (lambda: I.sample(lg, pd, offs, vocab=50257), 0.0, 64 * V * 4)
    return cases


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=".*")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json")
    ap.add_argument("--json", default="")
    ap.add_argument("--library", action="store_true",
                    help="also time every GEMM shape through torch.matmul / addmm (cuBLASLt) as '<case>@cublaslt'")
    args = ap.parse_args(argv)
    peak_tf, peak_gb = None, None
    try:
        with open(args.peaks) as f:
            pk = json.load(f)
        peak_tf, peak_gb = float(pk["bf16_tflops"]), float(pk["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        pass
    pat = re.compile(args.only)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows: List[dict] = []
    for name, (fn, flops, nbytes) in build_cases(args.small, args.library).items():
        if not pat.search(name):
            continue
        med, best = _time(fn, 1 if args.small else args.iters, 1 if args.small else args.warmup, flush)
        row = {"case": name, "ms_median": med, "ms_best": best}
        if flops:
            row["tflops"] = flops / (med * 1e-3) / 1e12
            if peak_tf:
                row["frac_of_measured_bf16_peak"] = row["tflops"] / peak_tf
        else:
            row["gbs"] = nbytes / (med * 1e-3) / 1e9
            if peak_gb:
                row["frac_of_measured_hbm_copy"] = row["gbs"] / peak_gb
        rows.append(row)
        rate = f"{row['tflops']:8.1f} TFLOP/s" if flops else f"{row['gbs']:8.1f} GB/s  "
        frac = row.get("frac_of_measured_bf16_peak", row.get("frac_of_measured_hbm_copy"))
        print(f"{name:34s} {med * 1e3:10.1f} us  {rate}  {'' if frac is None else f'{frac:5.2f} of measured'}", flush=True)
    from ..ops import _cuda as K
    K.check_status()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
