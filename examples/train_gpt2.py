"""Train GPT-2 124M (or any preset) on synthetic tokens with the fused sm_100a backend.

    python examples/train_gpt2.py --steps 50                                   # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_gpt2.py --fsdp
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nexus_b200.lm.config import preset  # noqa: E402
from nexus_b200.train.lm_trainer import AdamW, LanguageTrainerBuilder, SyntheticTokens  # noqa: E402
from nexus_b200.train.schedule import LrSchedule  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2-124m")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--fsdp", action="store_true")
    ap.add_argument("--graph", action="store_true", help="capture the whole step in a CUDA graph")
    a = ap.parse_args()
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    dev = f"cuda:{local}" if torch.cuda.is_available() else "cpu"
    if dev != "cpu":
        torch.cuda.set_device(local)
    cfg = preset(a.model)
    b = (LanguageTrainerBuilder(cfg).data(SyntheticTokens(cfg.vocab_size, seed=1, rank=rank, world=world))
         .optimizer(AdamW(lr=6e-4, beta2=0.95, weight_decay=0.1)).micro_batch(a.micro_batch).seq_len(a.seq_len)
         .global_batch_tokens(a.micro_batch * a.seq_len * world).grad_clip(1.0)
         .precision("bf16" if dev != "cpu" else "fp32", "fp32").execution_policy(dev).log_every(10).compile(a.graph))
    if world > 1:
        from nexus_b200.parallel.process_group import init_process_group
        pg = init_process_group(device=dev)
        b = b.fsdp(pg, None) if a.fsdp else b.process_group(pg)
    trainer = b.build()
    s = trainer.train(a.steps)
    if rank == 0:
        print(f"{s.steps} steps, final loss {s.final_loss:.4f}, {s.tokens / s.seconds:,.0f} tokens/s")


if __name__ == "__main__":
    main()
