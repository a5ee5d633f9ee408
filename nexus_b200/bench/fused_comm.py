"""Timing and roofline of the fused compute+collective GEMMs on the GPUs of one node, next to the un-fused form
(NCCL collective + the same tcgen05 GEMM) on the same box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m nexus_b200.bench.fused_comm [--tokens 32768] [--d 4096] [--ff 11008] [--iters 10] [--check]

Shapes are one tensor-parallel transformer block of width ``d`` with ``tokens`` rows in total (sequence parallel:
each rank holds tokens / N rows of the activations; weights are split N ways).  Every line is device-timed with CUDA
events (max over ranks, after warm-up, inputs far larger than L2).  The roofline of a fused kernel is the slower of
FLOPs / measured GEMM peak and bytes that must cross NVLink / 770 GB/s (the measured peer-copy rate per direction).

  ag_gemm      Y[M, n_loc]  = all-gather(X)[M, d] @ W[n_loc, d]^T          (column-parallel forward, qkv / up);
               push form: copier CTAs of the GEMM kernel store this rank's rows into the peers' gather buffers
  ag_pull      the same product with each tile TMA-loaded from its owner's memory (every column tile re-reads it)
  gemm_rs      Z[M/N, d]    = reduce-scatter(A[M, k_loc] @ W[d, k_loc]^T)   (row-parallel forward, o / down);
               push form: copier CTAs of the GEMM kernel store finished row blocks into the owners' slots
  dgrad_ag     dA[M, k_loc] = all-gather(dZ)[M, d] @ W[d, k_loc]            (row-parallel backward, MN-major weight)
  wgrad_k      dW[n_loc, d] = dY[M, n_loc]^T @ all-gather(X)[M, d]          (contraction over the sharded rows)
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--ff", type=int, default=11008)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--copiers", type=int, default=8, help="copier CTAs of the all-gather GEMM")
    ap.add_argument("--pull", action="store_true", help="also time the pull forms (remote tiles re-read per column tile)")
    ap.add_argument("--loopback", action="store_true",
                    help="one GPU: run the fused kernels as rank 0 of 2 with the 'peer' buffers in this GPU's own memory and "
                         "the arrival flags pre-set (for profiler captures, which must be single-process: the copier CTAs "
                         "and the flag waits run as they do over NVLink, the pushed bytes land in local HBM)")
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="GEMM peak for the roofline (default: MEASURED_PEAKS.json)")
    args = ap.parse_args(argv)

    from ..ops import _cuda as K
    from ..parallel.process_group import init_process_group
    from ..parallel.symm import GatherSite, SymmetricWorkspace, gemm_ag, gemm_dist, gemm_rs, sum_slots

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if args.loopback:
        return _loopback(args, dev)
    pg = init_process_group("nccl", f"cuda:{local}")
    ws = SymmetricWorkspace(pg)
    n = world
    peak = args.peak_tflops
    if peak <= 0:
        try:
            root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
            peak = float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["bf16_tflops"])
        except Exception:
            peak = 1590.0
    link = 770e9
    M, d = args.tokens, args.d
    Ml = M // n
    ff_loc = (args.ff // n + 127) // 128 * 128
    qkv_loc = (3 * d // n + 127) // 128 * 128
    bf = torch.bfloat16
    gen = torch.Generator(device=dev).manual_seed(7 + rank)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=gen) * scale).to(bf)

    def timed(fn, iters=args.iters):
        for _ in range(3):
            fn()
        pg.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        K.check_status(dev)
        ms = e0.elapsed_time(e1) / iters
        return float(pg.all_reduce_scalar(ms, "max"))

    rows = []

    def report(name, shape, flops, nv_bytes, fused_ms, base_ms, err=None):
        roof_ms = max(flops / (peak * 1e12), nv_bytes / link) * 1e3
        rows.append({"op": name, "shape": shape, "fused_ms": round(fused_ms, 4), "nccl_plus_gemm_ms": round(base_ms, 4),
                     "speedup": round(base_ms / fused_ms, 3), "tflops": round(flops / fused_ms / 1e9, 1),
                     "nvlink_GBps_min": round(nv_bytes / fused_ms / 1e6, 1), "roofline_ms": round(roof_ms, 4),
                     "fraction_of_roofline": round(roof_ms / fused_ms, 3), "max_rel_err": err})

    # ------------------------------------------------------------------ symmetric operands
    x_sym = ws.alloc(Ml * d, bf)
    x_loc = x_sym.local.view(Ml, d)
    x_loc.copy_(rnd(Ml, d))
    x_full = torch.empty(M, d, dtype=bf, device=dev)
    torch.cuda.synchronize(); ws.barrier(); torch.cuda.synchronize()

    def gather_x():
        pg.all_gather_tensor(x_full.view(-1), x_loc.reshape(-1))

    site = GatherSite(ws, Ml)
    xg = ws.alloc(M * d, bf)                       # gather buffer; this rank's block is filled once
    xg.local.view(M, d)[rank * Ml: (rank + 1) * Ml].copy_(x_loc)
    torch.cuda.synchronize(); ws.barrier(); torch.cuda.synchronize()
    for n_loc, tag in ((qkv_loc, "qkv"), (2 * ff_loc, "up")):
        w = rnd(n_loc, d, scale=0.02)
        y = torch.empty(M, n_loc, dtype=bf, device=dev)
        y2 = torch.empty_like(y)

        def fused_ag():
            ws.barrier()          # peers have finished with the previous contents of their gather buffers
            gemm_ag(site, xg, w, y, k=d, copier_ctas=args.copiers)

        fused = timed(fused_ag)
        base = timed(lambda: (gather_x(), K.gemm(x_full, w, out=y2)))
        local = timed(lambda: K.gemm(x_full, w, out=y2))
        err = None
        if args.check:
            gather_x(); K.gemm(x_full, w, out=y2)
            xg.local.view(M, d)[: rank * Ml].zero_(); xg.local.view(M, d)[(rank + 1) * Ml:].zero_()
            torch.cuda.synchronize(); fused_ag(); torch.cuda.synchronize()
            err = float((y.float() - y2.float()).abs().max() / y2.float().abs().max())
            err = max(err, float((xg.local.view(M, d).float() - x_full.float()).abs().max()))
        report(f"ag_gemm[{tag}]", [M, n_loc, d], 2.0 * M * n_loc * d, (n - 1) * Ml * d * 2, fused, base, err)
        rows[-1]["local_gemm_ms"] = round(local, 4)
        if args.pull:
            pull = timed(lambda: gemm_dist(ws, x_loc, w, y, a_peers=x_sym))
            report(f"ag_pull[{tag}]", [M, n_loc, d], 2.0 * M * n_loc * d, (n - 1) * Ml * d * 2, pull, base, None)
        del w, y, y2

    # ------------------------------------------------------------------ GEMM -> reduce-scatter (slot form)
    slots = ws.alloc(n * Ml * d, bf)
    partial = torch.empty(M, d, dtype=bf, device=dev)
    done = torch.zeros(M // 256, dtype=torch.int32, device=dev)
    for k_loc, tag in ((d // n, "o"), (ff_loc, "down")):
        a = rnd(M, k_loc)
        w = rnd(d, k_loc, scale=0.02)
        z = torch.empty(Ml, d, dtype=torch.float32, device=dev)
        full = torch.empty(M, d, dtype=bf, device=dev)
        z2 = torch.empty(Ml, d, dtype=bf, device=dev)

        def fused_rs():
            ws.barrier()       # the owners have consumed the previous contents of their slots
            gemm_rs(ws, a, w, partial, slots, done, copier_ctas=args.copiers)
            ws.barrier()       # every rank's partial blocks have landed
            sum_slots(slots.local, n, Ml, d, z, own=partial[rank * Ml: (rank + 1) * Ml], own_rank=rank)

        def base_rs():
            K.gemm(a, w, out=full)
            pg.reduce_scatter_tensor(z2.view(-1), full.view(-1))

        fused = timed(fused_rs)
        base = timed(base_rs)
        err = None
        if args.check:
            fused_rs(); base_rs(); torch.cuda.synchronize()
            err = float((z - z2.float()).abs().max() / z2.float().abs().max())
        report(f"gemm_rs[{tag}]", [M, d, k_loc], 2.0 * M * d * k_loc, (n - 1) * Ml * d * 2, fused, base, err)
        del a, w, z, full, z2

    # ------------------------------------------------------------------ dgrad with all-gather, MN-major weight
    k_loc = ff_loc
    w = rnd(d, k_loc, scale=0.02)          # row-parallel weight [d, k_loc]; dA = AG(dZ) @ W
    da = torch.empty(M, k_loc, dtype=bf, device=dev)
    da2 = torch.empty_like(da)
    def fused_dgrad():
        ws.barrier()
        gemm_ag(site, xg, w, da, k=d, b_mn=True, copier_ctas=args.copiers)

    fused = timed(fused_dgrad)
    base = timed(lambda: (gather_x(), K.gemm(x_full, w, b_mn=True, out=da2)))
    err = None
    if args.check:
        gather_x(); K.gemm(x_full, w, b_mn=True, out=da2); fused_dgrad(); torch.cuda.synchronize()
        err = float((da.float() - da2.float()).abs().max() / da2.float().abs().max())
    report("dgrad_ag[down]", [M, k_loc, d], 2.0 * M * k_loc * d, (n - 1) * Ml * d * 2, fused, base, err)
    del w, da, da2

    # ------------------------------------------------------------------ all-reduce: in-switch, peer loads, NCCL
    from ..parallel.symm import fused_all_reduce, multimem_all_reduce
    ar_rows = []
    for numel in (256 * 1600, 16 << 20, 64 << 20):                     # FP32: a decode step's activations ... a gradient bucket
        buf = ws.alloc(numel, torch.float32)
        dst = ws.alloc(numel, torch.float32)
        buf.local.normal_()
        ref = buf.local.clone()
        t_mm = timed(lambda: multimem_all_reduce(ws, buf, numel, scale=1.0 / n)) if buf.multicast else None
        t_pl = timed(lambda: fused_all_reduce(ws, buf, dst, numel, scale=1.0 / n, multimem=False))
        t_nc = timed(lambda: pg.all_reduce_tensor(ref, "sum"))
        bus = 2.0 * (n - 1) / n * numel * 4                            # bytes per GPU of a ring all-reduce (bus bandwidth)
        ar_rows.append({"op": "all_reduce[fp32]", "mbytes": round(numel * 4 / 2 ** 20, 1),
                        "multimem_ms": None if t_mm is None else round(t_mm, 4), "peer_load_ms": round(t_pl, 4),
                        "nccl_ms": round(t_nc, 4),
                        "multimem_busbw_GBps": None if t_mm is None else round(bus / t_mm / 1e6, 1),
                        "peer_load_busbw_GBps": round(bus / t_pl / 1e6, 1), "nccl_busbw_GBps": round(bus / t_nc / 1e6, 1)})
    if rank == 0:
        for r in ar_rows:
            print("all_reduce fp32 %7.1f MiB   in-switch %s ms (%s GB/s bus)   peer loads %.4f ms (%.1f)   NCCL %.4f ms (%.1f)"
                  % (r["mbytes"], r["multimem_ms"], r["multimem_busbw_GBps"], r["peer_load_ms"], r["peer_load_busbw_GBps"],
                     r["nccl_ms"], r["nccl_busbw_GBps"]), flush=True)
    rows.extend(ar_rows)

    # ------------------------------------------------------------------ wgrad over the sharded rows (pull form)
    if not args.pull:
        return _finish(rank, n, M, d, peak, link, rows, pg)
    n_loc = qkv_loc
    dy = rnd(M, n_loc)                     # local [M(k), n_loc]: A, MN-major
    dw = torch.zeros(n_loc, d, dtype=torch.float32, device=dev)
    dw2 = torch.zeros_like(dw)
    fused = timed(lambda: gemm_dist(ws, dy, x_loc, dw, b_peers=x_sym, a_mn=True, b_mn=True, b_shard="k"))
    base = timed(lambda: (gather_x(), K.gemm(dy, x_full, a_mn=True, b_mn=True, out=dw2)))
    err = None
    if args.check:
        gather_x(); K.gemm(dy, x_full, a_mn=True, b_mn=True, out=dw2)
        gemm_dist(ws, dy, x_loc, dw, b_peers=x_sym, a_mn=True, b_mn=True, b_shard="k"); torch.cuda.synchronize()
        err = float((dw - dw2).abs().max() / dw2.abs().max())
    report("wgrad_k[qkv]", [n_loc, d, M], 2.0 * M * n_loc * d, (n - 1) * Ml * d * 2, fused, base, err)

    return _finish(rank, n, M, d, peak, link, rows, pg)


def _loopback(args, dev) -> int:
    """Rank 0 of an emulated 2-rank group on ONE GPU (see --loopback)."""
    import types
    from ..ops import _cuda as K
    from ..parallel.symm import SymmetricBuffer, gemm_ag, gemm_rs, sum_slots
    n, M, d = 2, args.tokens, args.d
    Ml = M // n
    bf = torch.bfloat16
    ff_loc = (args.ff // n + 127) // 128 * 128
    ws = types.SimpleNamespace(n=n, rank=0, device=dev)

    def pair(numel, dtype, fill=None):
        a, b = torch.zeros(numel, dtype=dtype, device=dev), torch.zeros(numel, dtype=dtype, device=dev)
        if fill is not None:
            a.fill_(fill)
        return SymmetricBuffer(a, [a.data_ptr(), b.data_ptr()])

    site = types.SimpleNamespace(ws=ws, rows=Ml, flags=pair(n * (Ml // 128), torch.int32, fill=1 << 30),
                                 counter=torch.zeros(1, dtype=torch.int32, device=dev))
    xg = pair(M * d, bf)
    xg.local.copy_(torch.randn(M * d, device=dev).to(bf))
    w = (torch.randn(2 * ff_loc, d, device=dev) * 0.02).to(bf)
    y = torch.empty(M, 2 * ff_loc, dtype=bf, device=dev)
    a = torch.randn(M, ff_loc, device=dev).to(bf)
    wd = (torch.randn(d, ff_loc, device=dev) * 0.02).to(bf)
    slots = pair(n * Ml * d, bf)
    partial = torch.empty(M, d, dtype=bf, device=dev)
    done = torch.zeros(M // 256, dtype=torch.int32, device=dev)
    z = torch.empty(Ml, d, dtype=torch.float32, device=dev)
    out = {}
    for name, fn in (("ag_gemm[up]", lambda: gemm_ag(site, xg, w, y, k=d, copier_ctas=args.copiers)),
                     ("gemm_rs[down]", lambda: (gemm_rs(ws, a, wd, partial, slots, done, copier_ctas=args.copiers),
                                                sum_slots(slots.local, n, Ml, d, z, own=partial[:Ml], own_rank=0)))):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        K.check_status(dev)
        out[name] = round(e0.elapsed_time(e1) / args.iters, 4)
    ref = xg.local.view(M, d)[:512].float() @ w.float().t()
    err = float((y[:512].float() - ref).abs().max() / ref.abs().max())
    print(json.dumps({"bench": "fused_comm loopback (1 GPU as rank 0 of 2; pushed bytes land in local HBM)", "tokens": M,
                      "d": d, "copiers": args.copiers, "ms": out, "ag_gemm_max_rel_err": err}))
    return 0


def _finish(rank, n, M, d, peak, link, rows, pg) -> int:
    if rank == 0:
        print(json.dumps({"bench": "fused_comm", "n_gpus": n, "tokens": M, "d": d, "peak_tflops": peak,
                          "nvlink_GBps": link / 1e9, "rows": rows}))
        for r in rows:
            if "fused_ms" not in r:
                continue
            print("%-16s %-22s fused %8.3f ms  nccl+gemm %8.3f ms  x%.2f  %7.1f TFLOP/s  roofline %.3f ms -> %.2f"
                  % (r["op"], r["shape"], r["fused_ms"], r["nccl_plus_gemm_ms"], r["speedup"], r["tflops"],
                     r["roofline_ms"], r["fraction_of_roofline"]) + (f"  err {r['max_rel_err']:.1e}" if r["max_rel_err"] is not None else "")
                  + (f"  local gemm {r['local_gemm_ms']:.3f} ms" if "local_gemm_ms" in r else ""))
    torch.cuda.synchronize()
    pg.destroy()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
