"""2+ GPU worker (one rank per GPU, launched by torch.distributed.run): the tensor + sequence parallel Llama model
(`models.llama_tp.LlamaTpModel`, fused all-gather -> GEMM / GEMM -> reduce-scatter kernels over peer memory) against
the same model on one rank with the full weights.  Prints 'WORKER_OK' on rank 0."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from nexus_b200.lm.config import LmConfig  # noqa: E402
from nexus_b200.models.gpt import AdamWConfig  # noqa: E402
from nexus_b200.models.llama_tp import LlamaTpModel  # noqa: E402
from nexus_b200.ops import _cuda as K  # noqa: E402
from nexus_b200.parallel.process_group import init_process_group  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    pg = init_process_group("nccl", dev)
    ok = True

    def check(name, cond):
        nonlocal ok
        ok &= bool(cond)
        if rank == 0:
            print(("OK  " if cond else "BAD ") + name, flush=True)

    cfg = LmConfig(name="tiny-llama", vocab_size=1024, n_layer=2, d_model=512, n_head=8, n_kv_head=4, d_ff=1024,
                   max_position=256, norm="rmsnorm", mlp="swiglu", pos="rope", tie_embeddings=False, bias=False)
    full = LlamaTpModel.random_full_weights(cfg, seed=3)
    B, T = world, 256
    tokens = torch.randint(0, cfg.vocab_size, (B, T), dtype=torch.int32, generator=torch.Generator().manual_seed(1)).to(dev)
    single = LlamaTpModel(cfg, device=dev, full_weights=full)
    single.set_optimizer(AdamWConfig(lr=1e-3, grad_clip=1.0))
    tp = LlamaTpModel(cfg, pg, device=dev, full_weights=full, copier_ctas=4)
    tp.set_optimizer(AdamWConfig(lr=1e-3, grad_clip=1.0))

    l1 = float(single.forward_backward(tokens).item())
    l2 = float(tp.forward_backward(tokens).item())
    torch.cuda.synchronize(); K.check_status()
    check(f"first loss: tp {l2:.5f} vs single {l1:.5f}", abs(l1 - l2) < 2e-3)
    g1, g2 = single.gather_full("grads"), tp.gather_full("grads")
    worst = ("", 0.0)
    for name in g1:
        a, b = g2[name], g1[name]
        if name.startswith("norm"):          # replicated: each rank holds the sum over its own rows until the step
            a = a.clone()
            torch.distributed.all_reduce(a)
        rel = (a - b).norm().item() / max(b.norm().item(), 1e-12)
        if rel > worst[1]:
            worst = (name, rel)
    check(f"gradients: worst relative L2 difference {worst[1]:.2e} ({worst[0]})", worst[1] < 3e-2)
    losses = [[], []]
    for step in range(3):
        single.optimizer_step()
        tp.optimizer_step()
        losses[0].append(float(single.forward_backward(tokens).item()))
        losses[1].append(float(tp.forward_backward(tokens).item()))
    torch.cuda.synchronize(); K.check_status()
    s1, s2 = single.read_opt_state(), tp.read_opt_state()
    check(f"grad norm {s2.grad_norm:.5f} vs {s1.grad_norm:.5f}", abs(s1.grad_norm - s2.grad_norm) < 2e-2 * s1.grad_norm)
    check(f"losses after steps: tp {losses[1]} vs single {losses[0]}",
          all(abs(a - b) < 3e-2 for a, b in zip(*losses)) and losses[1][-1] < l2)
    p1, p2 = single.gather_full("params"), tp.gather_full("params")
    upd = max((p1[k] - full[k].to(dev)).norm().item() for k in ("q_w", "down_w"))
    worst = max((p2[k] - p1[k]).norm().item() / max((p1[k] - full[k].to(dev)).norm().item(), 1e-12) for k in ("q_w", "down_w"))
    check(f"parameters after 3 steps: difference relative to the update {worst:.2e} (update {upd:.2e})", worst < 0.25)

    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    pg.all_reduce_tensor(flag, "min")
    if rank == 0:
        print("WORKER_OK" if flag.item() == 1.0 else "WORKER_FAILED", flush=True)
    pg.destroy()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
