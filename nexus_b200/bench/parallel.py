"""Training throughput of a tensor-parallel language model (`parallel.ParallelLm`) on the GPUs of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29541 \
        -m nexus_b200.bench.parallel --model llama2-7b --tp 8 --seq-len 4096 --global-batch 8 --micro-batch 1 \
        --precision mxfp8 --steps 3 --warmup 2

One rank per GPU over NCCL.  Every rank builds only its own slices (the full model is never materialised: the
per-rank slices are drawn directly, which is what random-init weights allow), runs `steps` optimizer steps of
`global-batch` sequences (micro-batches accumulate), device-timed with CUDA events between barriers, and rank 0
prints one JSON line with tokens/s (max step time over ranks).  `--check` compares the first loss against the
single-process `LanguageModel` on the same tokens (small configurations only).
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
import types

import torch


class _RandomWeights:
    """Stands in for a full `LanguageModel` in throughput runs: `named_parameters()` yields random-init tensors of
    the full shapes, created on the GPU from the configuration's seed (the same on every rank), so that a model whose
    host copy would take tens of GB per rank is never built on the host.  `ParallelLm` keeps its slices; the rest is
    freed as soon as it has been sliced."""

    def __init__(self, cfg, device):
        self.config = cfg
        self.device = device

    def named_parameters(self):
        cfg = self.config
        g = torch.Generator(device=self.device).manual_seed(cfg.seed)
        for name, shape in build_meta(cfg):
            if len(shape) >= 2:
                yield name, torch.randn(shape, device=self.device, generator=g, dtype=torch.bfloat16) * cfg.init_std
            elif name.endswith(".weight"):
                yield name, torch.ones(shape, device=self.device)
            else:
                yield name, torch.zeros(shape, device=self.device)


def build_meta(cfg):
    """(name, shape) of every parameter of the dense pre-norm model `lm.model.build(cfg)` would create."""
    H, Hk, D, d, Fd = cfg.n_head, cfg.kv_heads(), cfg.hdim(), cfg.d_model, cfg.d_ff
    out = [("wte", (cfg.padded_vocab(), d))]
    if cfg.pos == "learned":
        out.append(("wpe", (cfg.max_position, d)))
    for l in range(cfg.n_layer):
        p = f"h.{l}."
        for nm in ("norm1", "norm2"):
            out.append((p + nm + ".weight", (d,)))
            if cfg.norm == "layernorm":
                out.append((p + nm + ".bias", (d,)))
        out.append((p + "attn.qkv.weight", ((H + 2 * Hk) * D, d)))
        out.append((p + "attn.o.weight", (d, H * D)))
        out.append((p + "mlp.up.weight", ((2 * Fd if cfg.gated_mlp() else Fd), d)))
        out.append((p + "mlp.down.weight", (d, Fd)))
        if cfg.bias:
            out += [(p + "attn.qkv.bias", ((H + 2 * Hk) * D,)), (p + "attn.o.bias", (d,)),
                    (p + "mlp.up.bias", ((2 * Fd if cfg.gated_mlp() else Fd),)), (p + "mlp.down.bias", (d,))]
    out.append(("norm_f.weight", (d,)))
    if cfg.norm == "layernorm":
        out.append(("norm_f.bias", (d,)))
    if not cfg.tie_embeddings:
        out.append(("lm_head", (cfg.padded_vocab(), d)))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama2-7b")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0: the preset's)")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel degree (0: all ranks)")
    ap.add_argument("--cp", type=int, default=1, help="context-parallel degree (the `ParallelLm` path, --comm nccl)")
    ap.add_argument("--cp-algorithm", default="ring", choices=["ring", "ulysses"])
    ap.add_argument("--cp-layout", default="zigzag", choices=["zigzag", "contiguous"])
    ap.add_argument("--cp-comm", default="fused", choices=["fused", "nccl"],
                    help="context-parallel attention over peer memory (fused) or send_recv through NCCL")
    ap.add_argument("--sp", type=int, default=0, help="1: sequence-parallel norm / residual regions")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--global-batch", type=int, default=8, help="sequences per optimizer step (over all dp replicas)")
    ap.add_argument("--micro-batch", type=int, default=1, help="sequences per forward / backward pass")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "mxfp8"])
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="fused: models.llama_tp.LlamaTpModel (all-gather -> GEMM / GEMM -> reduce-scatter inside the "
                         "tcgen05 kernels over peer memory, hand-scheduled backward); nccl: parallel.ParallelLm "
                         "(autograd, NCCL all-reduces at the region boundaries) - the same-box baseline")
    ap.add_argument("--copiers", type=int, default=0,
                    help="copier CTAs of the fused GEMM kernels (0: 8 up to two ranks, 32 beyond, where the link binds)")
    ap.add_argument("--graph", type=int, default=0, help="fused: replay the whole step as one CUDA graph")
    args = ap.parse_args(argv)
    if args.comm == "fused" and args.precision == "bf16" and not args.check and args.cp == 1:
        return run_fused(args)

    from ..fused.ops import linear_precision
    from ..lm.config import preset
    from ..lm.model import build
    from ..ops import _cuda as K
    from ..parallel.parallel_lm import ParallelConfig, ParallelLm
    from ..parallel.process_group import init_process_group

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    pg = init_process_group(backend="nccl", device=f"cuda:{local}")
    tp = args.tp or max(1, world // args.cp)
    dp = world // (tp * args.cp)
    cfg = preset(args.model)
    if args.layers > 0:
        cfg.n_layer = args.layers
    cfg.max_position = max(cfg.max_position, args.seq_len)
    source = build(cfg) if args.check else _RandomWeights(cfg, dev)
    plm = ParallelLm(source, pg, ParallelConfig(dp=dp, tp=tp, cp=args.cp, sp=bool(args.sp), cp_algorithm=args.cp_algorithm,
                                                cp_layout=args.cp_layout, cp_comm=args.cp_comm),
                     device=dev, compute_dtype=torch.bfloat16)
    if not args.check:
        del source
    torch.cuda.empty_cache()
    opt = types.SimpleNamespace(beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    per_replica = args.global_batch // dp
    n_micro = per_replica // args.micro_batch
    gen = torch.Generator(device=dev).manual_seed(1234 + rank // (tp * args.cp))

    def batch():
        return [torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq_len), device=dev, generator=gen)
                for _ in range(n_micro)]

    ctx = linear_precision("mxfp8") if args.precision == "mxfp8" else contextlib.nullcontext()
    losses = []
    with ctx:
        if args.check:
            toks = batch()
            got = plm.forward_backward(toks)
            full = source.to(dev)
            with torch.no_grad():
                want = sum(float(full.loss(t)) for t in toks) / len(toks)
            plm.zero_grad()
            if rank == 0:
                print(json.dumps({"check": "first loss", "parallel": got, "single": want}), flush=True)
            if abs(got - want) > 0.03 * abs(want):
                raise SystemExit(f"loss mismatch: parallel {got} vs single {want}")
        for _ in range(max(1, args.warmup)):
            losses.append(plm.forward_backward(batch()))
            plm.step(opt, 3e-4, clip=1.0)
        pg.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            losses.append(plm.forward_backward(batch()))
            plm.step(opt, 3e-4, clip=1.0)
        e1.record()
        pg.barrier()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    ms = float(pg.all_reduce_scalar(ms, "max"))
    K.check_status()
    tokens = args.global_batch * args.seq_len
    if rank == 0:
        print(json.dumps({
            "metric": f"train tokens/s {args.model} tensor-parallel", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "ms_per_step": ms, "steps": args.steps, "warmup": max(1, args.warmup),
            "config": {"model": args.model, "layers": cfg.n_layer, "tp": tp, "dp": dp, "cp": args.cp,
                       "cp_attention": (f"{args.cp_algorithm}/{args.cp_layout}/" + ("peer memory" if plm._cp_ws is not None else "send_recv")
                                        if args.cp > 1 else None),
                       "sp": bool(args.sp),
                       "seq_len": args.seq_len, "global_batch": args.global_batch, "micro_batch": args.micro_batch,
                       "linear_precision": args.precision, "compute_dtype": "bf16", "master": "fp32 AdamW, clip 1.0"},
            "losses": [round(x, 4) for x in losses],
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2),
            "data": "synthetic uniform tokens, random-init weights"}), flush=True)
    pg.destroy()
    return 0


def run_fused(args) -> int:
    """The tensor + sequence parallel model on the fused kernels: one pass over the whole batch per optimizer step
    (micro-batches accumulate when --micro-batch is smaller than the per-replica batch)."""
    from ..lm.config import preset
    from ..models.gpt import AdamWConfig
    from ..models.llama_tp import LlamaTpModel
    from ..ops import _cuda as K
    from ..parallel.process_group import init_process_group

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    pg = init_process_group(backend="nccl", device=f"cuda:{local}") if world > 1 else None
    cfg = preset(args.model)
    if args.layers > 0:
        cfg.n_layer = args.layers
    cfg.max_position = max(cfg.max_position, args.seq_len)
    model = LlamaTpModel(cfg, pg, device=dev, copier_ctas=args.copiers)
    args.copiers = model.copier_ctas
    model.set_optimizer(AdamWConfig(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, grad_clip=1.0))
    n_micro = max(1, args.global_batch // args.micro_batch)
    gen = torch.Generator(device=dev).manual_seed(1234)
    sets = [[torch.empty((args.micro_batch, args.seq_len), device=dev, dtype=torch.int32) for _ in range(n_micro)]
            for _ in range(2)]

    def refill(tokens):   # fresh uniform tokens for every step, drawn on the device (the same on every rank)
        for t in tokens:
            t.random_(0, cfg.vocab_size, generator=gen)

    loss_log = torch.zeros(args.steps + max(1, args.warmup), dtype=torch.float32, device=dev)
    step_no = [0]

    def step(tokens, fresh=True):
        if fresh:
            refill(tokens)
        for i, t in enumerate(tokens):
            model.forward_backward(t, grad_scale=1.0 / n_micro, accumulate_loss=i > 0, loss_weight=1.0 / n_micro)
        model.optimizer_step()

    def barrier():
        if pg is not None:
            pg.barrier()
        torch.cuda.synchronize()

    for i in range(max(1, args.warmup)):
        step(sets[i % 2])
        loss_log[step_no[0]].copy_(model.loss_buf[0])
        step_no[0] += 1
    graph = None
    if args.graph:
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(sets[0], fresh=False)     # the token buffers are refilled outside the graph, before every replay
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = K.launch_count
    e0.record()
    for i in range(args.steps):
        if graph is not None:
            refill(sets[0])
            graph.replay()
        else:
            step(sets[i % 2])
        loss_log[step_no[0]].copy_(model.loss_buf[0])
        step_no[0] += 1
    e1.record()
    barrier()
    K.check_status(dev)
    ms = e0.elapsed_time(e1) / args.steps
    if pg is not None:
        ms = float(pg.all_reduce_scalar(ms, "max"))
    tokens = args.global_batch * args.seq_len
    if rank == 0:
        try:
            root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
            peak = float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
        except Exception:
            peak = 1400.0
        tflops = model.flops_per_token(args.seq_len) * tokens / (ms * 1e-3) / 1e12 / world
        print(json.dumps({
            "metric": f"train tokens/s {args.model} tensor-parallel", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "ms_per_step": ms, "steps": args.steps, "warmup": max(1, args.warmup),
            "tflops_per_gpu": round(tflops, 1), "fraction_of_sustained_bf16": round(tflops / peak, 3),
            "config": {"model": args.model, "layers": cfg.n_layer, "tp": world, "sp": True, "comm": "fused",
                       "seq_len": args.seq_len, "global_batch": args.global_batch, "micro_batch": args.micro_batch,
                       "linear_precision": "bf16", "compute_dtype": "bf16", "master": "fp32 AdamW, clip 1.0",
                       "copier_ctas": args.copiers, "cuda_graph": bool(args.graph)},
            "losses": [round(float(x), 4) for x in loss_log[: step_no[0]].cpu()],
            "kernel_launches_per_step": (K.launch_count - launches0) // max(args.steps, 1),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2),
            "data": "synthetic uniform tokens, random-init weights"}), flush=True)
    if pg is not None:
        pg.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
