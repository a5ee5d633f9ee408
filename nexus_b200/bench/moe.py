"""Training throughput of the expert-parallel MoE decoder (`models.moe_ep`) on the GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29551 \
        -m nexus_b200.bench.moe [--layers 16 --d-model 2048 --heads 16 --experts 64 --top-k 2 --expert-ff 1408 \
        --vocab 32000 --seq-len 2048 --seqs-per-gpu 8 --micro-batch 1 --capacity-factor 1.25 --aux 0.01 --steps 3 --warmup 2]

One rank per GPU; experts split over the ranks (expert parallel = data parallel group).  Every rank trains on its own
``seqs-per-gpu`` sequences per optimizer step (weak scaling), in micro-batches of ``micro-batch`` sequences.
Device-timed with CUDA events between barriers, max over ranks; rank 0 prints one JSON line (whole-job tokens/s).
Synthetic uniform tokens, random-init weights and router.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--expert-ff", type=int, default=1408)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--seqs-per-gpu", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--capacity-factor", type=float, default=1.25)
    ap.add_argument("--aux", type=float, default=0.01)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="row exchange of the expert-parallel layers: peer-memory dispatch / combine kernels, or NCCL "
                         "variable-split all-to-alls (the same-box comparison)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args(argv)
    os.environ["NEXUS_B200_EP_COMM"] = args.comm

    from ..lm.config import LmConfig
    from ..models.gpt import AdamWConfig
    from ..models.moe_ep import MoeEpDecoder, MoeEpTrainer
    from ..ops import _cuda as K
    from ..parallel.process_group import init_process_group

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    pg = init_process_group("nccl", f"cuda:{local}") if world > 1 else None
    cfg = LmConfig(name="moe-ep", vocab_size=args.vocab, n_layer=args.layers, d_model=args.d_model, n_head=args.heads,
                   d_ff=args.expert_ff, max_position=args.seq_len, norm="rmsnorm", mlp="swiglu", pos="rope",
                   tie_embeddings=False, bias=False, moe_experts=args.experts, moe_top_k=args.top_k,
                   moe_d_ff=args.expert_ff, moe_capacity_factor=args.capacity_factor, moe_aux_alpha=args.aux)
    model = MoeEpDecoder(cfg, pg, dev, micro_batch=args.micro_batch, seq_len=args.seq_len)
    trainer = MoeEpTrainer(model, AdamWConfig(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, grad_clip=1.0))
    n_micro = max(1, args.seqs_per_gpu // args.micro_batch)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    micro = [torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq_len), device=dev, generator=gen)
             for _ in range(n_micro)]

    def barrier():
        if pg is not None:
            pg.barrier()
        torch.cuda.synchronize()

    losses = []

    def step():
        out = trainer.step_accumulate(micro)
        losses.append(out.clone())

    for _ in range(max(1, args.warmup)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = K.launch_count
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    K.check_status(dev)
    ms = e0.elapsed_time(e1) / args.steps
    if pg is not None:
        ms = float(pg.all_reduce_scalar(ms, "max"))
    tokens = args.seqs_per_gpu * args.seq_len * world
    if rank == 0:
        tflops = model.flops_per_token(args.seq_len) * tokens / (ms * 1e-3) / 1e12 / world
        print(json.dumps({
            "metric": "train tokens/s MoE decoder, expert parallel", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "ms_per_step": ms, "steps": args.steps, "warmup": max(1, args.warmup), "scaling": "weak",
            "active_tflops_per_gpu": round(tflops, 1),
            "config": {"layers": args.layers, "d_model": args.d_model, "heads": args.heads, "experts": args.experts,
                       "top_k": args.top_k, "expert_ff": args.expert_ff, "vocab": args.vocab, "seq_len": args.seq_len,
                       "seqs_per_gpu": args.seqs_per_gpu, "micro_batch": args.micro_batch, "ep": world,
                       "capacity_factor": args.capacity_factor, "capacity_rows_per_expert": model.ep.capacity,
                       "aux_alpha": args.aux, "dtype": "bf16", "master": "fp32 AdamW, clip 1.0",
                       "dispatch": ("peer-memory kernels (nx_moe_dispatch / nx_moe_combine)" if args.comm == "fused"
                                    else "NCCL all_to_all_single with per-rank splits")},
            "losses": [[round(float(v), 4) for v in l.cpu()] for l in losses],
            "kernel_launches_per_step": (K.launch_count - launches0) // max(args.steps, 1),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2),
            "data": "synthetic uniform tokens, random-init weights and router"}), flush=True)
    if pg is not None:
        pg.destroy()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
