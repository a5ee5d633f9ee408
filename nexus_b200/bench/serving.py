"""Paged-attention serving throughput: GPT-2 XL (48 layers, d 1600, 25 heads, vocab 50257; random weights), 256
concurrent requests with prompt lengths uniform in [128, 1024] and 256 greedy tokens each, KV pages of 16 tokens,
continuous batching, tensor parallel over the GPUs of one node.

    python -m nexus_b200.bench.serving                                         # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29551 \
        -m nexus_b200.bench.serving                                            # TP = 8

Every rank runs the same scheduler on the same requests (greedy decoding of all-reduced logits is identical on all
ranks), so no token ever has to be broadcast.  Rank 0 prints one JSON line: generated tokens / s over the whole job
(wall clock between barriers around the serving loop, max over ranks), mean TTFT and TPOT.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2-xl", choices=["gpt2-xl", "gpt2-124m", "tiny"])
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--max-new", type=int, default=256)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=1024)
    ap.add_argument("--quant", default="bf16", help="weights: bf16 | fp8 | w8a8 | w4a16")
    ap.add_argument("--tp-comm", default="fused", choices=["fused", "nccl"],
                    help="tensor-parallel all-reduce: the peer-memory kernel (default) or NCCL")
    ap.add_argument("--kv", default="bf16", help="KV cache: bf16 | int8 | fp8")
    ap.add_argument("--batch-tokens", type=int, default=8192)
    ap.add_argument("--kv-gb", type=float, default=0.0, help="KV pool per GPU in GiB (0: sized for the workload)")
    ap.add_argument("--pipeline", type=int, default=1,
                    help="1: launch decode step n + 1 before the tokens of step n are read (device-fed tokens)")
    ap.add_argument("--tp-graphs", type=int, default=0, help="1: capture the decode steps of a tensor-parallel engine too")
    args = ap.parse_args(argv)

    from ..infer import Engine, EngineConfig, Gpt2Weights, QuantOptions, SamplingParams
    from ..serve import Config, Request, Server

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    dev = f"cuda:{local}" if cuda else "cpu"
    group = None
    if cuda:
        torch.cuda.set_device(local)
    if world > 1:
        from ..parallel.process_group import init_process_group
        group = init_process_group(backend="nccl" if cuda else "gloo", device=dev)

    shapes = {"gpt2-xl": (48, 25, 1600, 50257, 2048), "gpt2-124m": (12, 12, 768, 50257, 2048), "tiny": (2, 4, 256, 1000, 2048)}
    L, H, d, V, ctx = shapes[args.model]
    w = Gpt2Weights.random(L, H, d, V, ctx)
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(args.prompt_min, args.prompt_max + 1, (args.requests,), generator=g).tolist()
    prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]
    kv_elem = {"bf16": 2, "int8": 1, "fp8": 1}[args.kv]
    heads_local = -(-H // world)
    tokens_total = sum(lens) + args.requests * args.max_new
    kv_need = tokens_total * L * 2 * heads_local * (d // H) * kv_elem
    kv_bytes = int(args.kv_gb * 2 ** 30) if args.kv_gb > 0 else int(kv_need * 1.15) + (1 << 28)
    eng = Engine(w, EngineConfig(device=dev, precision="bf16" if cuda else "fp32", max_seqs=args.requests,
                                 max_tokens=args.batch_tokens, block_size=16, kv_bytes=kv_bytes,
                                 quant=QuantOptions(weights=args.quant, kv=args.kv), tp_graphs=bool(args.tp_graphs), tp_comm=args.tp_comm),
                 group=group)
    greedy = SamplingParams(temperature=0.0)

    def serve(reqs, new):
        srv = Server(eng, Config(max_batch_tokens=args.batch_tokens, max_running=args.requests,
                                 pipeline_decode=bool(args.pipeline)))
        futs = [srv.submit(Request(p, new, sampling=greedy)) for p in reqs]
        if group is not None:
            group.barrier()
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        srv.run_until_idle()
        if cuda:
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if group is not None:
            dt = float(group.all_reduce_scalar(dt, "max"))
        return srv, futs, dt

    serve(prompts[: min(8, len(prompts))], 8)     # warm-up: scratch buffers, decode graphs of the small buckets
    srv, futs, dt = serve(prompts, args.max_new)
    generated = sum(len(f.result().tokens) for f in futs)
    m = srv.metrics
    if rank == 0:
        print(json.dumps({
            "metric": "paged decode tokens/s (generated tokens, continuous batching, greedy)",
            "value": generated / dt, "unit": "tokens/s", "n_gpus": world, "seconds": dt,
            "prompt_tokens": sum(lens), "generated_tokens": generated, "steps": m.steps,
            "mean_ttft_ms": m.mean_ttft_ms(), "mean_tpot_ms": m.mean_tpot_ms(), "preemptions": m.preemptions,
            "config": {"model": args.model, "tp": world, "requests": args.requests, "prompt_len": [args.prompt_min, args.prompt_max],
                       "max_new": args.max_new, "page_size": 16, "weights": args.quant, "kv": args.kv,
                       "kv_pool_gib": round(kv_bytes / 2 ** 30, 1), "batch_tokens": args.batch_tokens,
                       "tp_graphs": bool(args.tp_graphs), "pipelined_decode_steps": m.pipelined_steps},
            "data": "random prompts from seed 0, random-init weights"}), flush=True)
    if group is not None:
        if args.tp_graphs:
            # graphs that captured collectives go first; the process then leaves without tearing the communicator down
            eng.release_graphs()
            group.barrier()
            torch.cuda.synchronize()
            sys.stdout.flush()
            os._exit(0)
        group.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
