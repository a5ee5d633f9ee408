"""Training worker for the launcher tests: FSDP over gloo ranks with periodic checkpoints.  On the
first attempt the rank named by FAIL_RANK exits with code 9 at step FAIL_STEP (between steps, on the host);
after a restart every rank resumes from the newest complete checkpoint (resharding when the world
size changed) and trains to TOTAL_STEPS.  Rank 0 writes `result.json` into the checkpoint directory."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from nexus_b200.ckpt.checkpoint import CheckpointOptions  # noqa: E402
from nexus_b200.lm.config import preset  # noqa: E402
from nexus_b200.parallel.fsdp import FsdpOptions  # noqa: E402
from nexus_b200.parallel.process_group import GroupOptions, init_process_group  # noqa: E402
from nexus_b200.train.lm_trainer import AdamW, LanguageTrainerBuilder, SyntheticTokens  # noqa: E402


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    attempt = int(os.environ.get("NEXUS_RESTART_COUNT", "0"))
    out = os.environ["CKPT_DIR"]
    total = int(os.environ.get("TOTAL_STEPS", "8"))
    fail_rank, fail_step = int(os.environ.get("FAIL_RANK", "-1")), int(os.environ.get("FAIL_STEP", "5"))
    torch.set_num_threads(1)
    pg = init_process_group("gloo", "cpu", GroupOptions(timeout_s=20.0))
    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab_size, cfg.max_position = 2, 32, 2, 64, 64, 16
    trainer = (LanguageTrainerBuilder(cfg).data(SyntheticTokens(cfg.vocab_size, seed=7, rank=rank, world=world))
               .optimizer(AdamW(lr=1e-2)).micro_batch(2).seq_len(16).global_batch_tokens(2 * 16 * world)
               .precision("fp32", "fp32").execution_policy("cpu").log_every(0)
               .fsdp(pg, FsdpOptions(stage=2)).checkpointing(CheckpointOptions(out, every=2, keep=3)).build())
    resumed = trainer.resume_latest()
    start = trainer.step
    losses = []
    while trainer.step < total:
        if attempt == 0 and rank == fail_rank and trainer.step == fail_step:
            os._exit(9)           # between steps: nothing of this rank is in flight
        losses.append(float(trainer.train(1).final_loss))
    if rank == 0:
        with open(os.path.join(out, "result.json"), "w") as f:
            json.dump({"world": world, "attempt": attempt, "resumed": bool(resumed), "start_step": start,
                       "final_step": trainer.step, "losses": losses}, f)
    pg.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
