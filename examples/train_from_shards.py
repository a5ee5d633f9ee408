"""From raw text to a resumed training run, on CPU or GPU.

    python examples/train_from_shards.py [--workdir DIR] [--steps N] [--device cpu|cuda]

1. trains a byte-level BPE tokenizer on a small generated corpus and writes it as JSON;
2. encodes the corpus into two token shards (`NXTK` files);
3. trains a small decoder LM from the shards through the memory-mapped native reader (`train.ShardTokens`:
   windows numbered across shards, shuffled by a keyed permutation per epoch, read ahead by a worker thread),
   checkpointing as it goes;
4. builds a second trainer, resumes from the newest checkpoint and checks that it continues on the same rows with
   the same loss as an uninterrupted run.
"""
import argparse
import os
import sys
import tempfile

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nexus_b200.ckpt.checkpoint import CheckpointOptions  # noqa: E402
from nexus_b200.lm import LanguageModel, preset  # noqa: E402
from nexus_b200.tools.tokenize import ByteBpe, write_shard  # noqa: E402
from nexus_b200.train import AdamW, LanguageTrainerBuilder, ShardTokens  # noqa: E402


def corpus(seed: int, sentences: int) -> bytes:
    rng = np.random.default_rng(seed)
    subj = ["the kernel", "a tensor", "the scheduler", "every rank", "the optimizer", "a page", "the router"]
    verb = ["loads", "reduces", "scatters", "gathers", "updates", "copies", "routes"]
    obj = ["a tile", "the gradients", "two shards", "the cache", "its tokens", "a block", "the weights"]
    out = []
    for _ in range(sentences):
        out.append(f"{rng.choice(subj)} {rng.choice(verb)} {rng.choice(obj)}.")
    return (" ".join(out)).encode()


def build(cfg, paths, seq, device, ckdir, seed=0):
    torch.manual_seed(seed)
    source = ShardTokens(paths, seq, seed=3, shuffle=True, prefetch=2)
    trainer = (LanguageTrainerBuilder(LanguageModel(cfg)).data(source).optimizer(AdamW(lr=2e-3)).micro_batch(4).seq_len(seq)
               .global_batch_tokens(4 * seq).precision("f32").execution_policy(device).log_every(0)
               .checkpointing(CheckpointOptions(directory=ckdir, every=0, keep=2)).build())
    return trainer, source


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workdir")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    work = a.workdir or tempfile.mkdtemp(prefix="nexus_shards_")
    os.makedirs(work, exist_ok=True)
    text = [corpus(1, 900), corpus(2, 700)]
    tok = ByteBpe.train(text[0] + text[1], 320)
    tok.save(os.path.join(work, "tok.json"))
    paths = []
    for i, t in enumerate(text):
        ids = tok.encode(t)
        paths.append(os.path.join(work, f"train-{i:03d}.bin"))
        write_shard(paths[-1], ids, tok.vocab_size)
        print(f"shard {i}: {len(t)} bytes -> {len(ids)} tokens")
    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab_size, cfg.max_position = 2, 64, 4, 256, tok.vocab_size, 32
    seq, half = 32, a.steps // 2
    # uninterrupted run
    full, src = build(cfg, paths, seq, a.device, os.path.join(work, "ck_full"))
    full.train(a.steps)
    want = [r.loss for r in full.history]
    print(f"{src.windows()} windows in {len(paths)} shards; loss {want[0]:.4f} -> {want[-1]:.4f}")
    # interrupted after half the steps, then resumed by a new trainer
    first, _ = build(cfg, paths, seq, a.device, os.path.join(work, "ck"))
    first.train(half)
    first.save_checkpoint()
    second, src2 = build(cfg, paths, seq, a.device, os.path.join(work, "ck"), seed=99)     # different init: must be overwritten
    assert second.resume_latest(), "no checkpoint found"
    second.train(a.steps - half)
    got = [r.loss for r in first.history] + [r.loss for r in second.history]
    worst = max(abs(x - y) for x, y in zip(got, want))
    print(f"resumed at step {half}: largest loss difference to the uninterrupted run {worst:.2e}")
    ok = worst < 1e-5 and want[-1] < want[0]
    print("OK" if ok else "MISMATCH")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
