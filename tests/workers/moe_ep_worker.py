"""2+ GPU worker (one rank per GPU, launched by torch.distributed.run): the expert-parallel MoE decoder
(`models.moe_ep`, dispatch / combine over peer memory, fused all-reduce of the replicated gradients) against the same
model on one rank that holds every expert and every sequence.  Prints 'WORKER_OK' on rank 0."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from nexus_b200.lm.config import LmConfig  # noqa: E402
from nexus_b200.models.gpt import AdamWConfig  # noqa: E402
from nexus_b200.models.moe_ep import MoeEpDecoder, MoeEpTrainer  # noqa: E402
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

    # capacity factor large enough that nothing is dropped: the two layouts then compute the same function
    cfg = LmConfig(name="tiny-moe", vocab_size=512, n_layer=2, d_model=256, n_head=4, d_ff=256, max_position=256,
                   norm="rmsnorm", mlp="swiglu", pos="rope", tie_embeddings=False, bias=False, moe_experts=4 * world,
                   moe_top_k=2, moe_d_ff=256, moe_capacity_factor=float(2 * world), moe_aux_alpha=0.01, seed=7)
    T = 256
    tokens = torch.randint(0, cfg.vocab_size, (world, T), generator=torch.Generator().manual_seed(1)).to(dev)
    opt = AdamWConfig(lr=1e-3, grad_clip=1.0)
    single = MoeEpTrainer(MoeEpDecoder(cfg, None, dev, micro_batch=world, seq_len=T), opt)
    ep = MoeEpTrainer(MoeEpDecoder(cfg, pg, dev, micro_batch=1, seq_len=T), opt)
    le = cfg.moe_experts // world

    # ---- one forward/backward without the update: losses and gradients
    ce1, aux1 = single.model.loss(tokens)
    (ce1 + aux1).backward()
    ce2, aux2 = ep.model.loss(tokens[rank: rank + 1])
    ((ce2 + aux2) / world).backward()
    torch.cuda.synchronize(); K.check_status()
    both = torch.stack([ce2.detach(), aux2.detach()])
    pg.all_reduce_tensor(both)
    both /= world
    check(f"cross-entropy: mean over ranks {both[0].item():.5f} vs single {ce1.item():.5f}", abs(both[0].item() - ce1.item()) < 3e-3)
    check(f"auxiliary loss: {both[1].item():.6f} vs {aux1.item():.6f}", abs(both[1].item() - aux1.item()) < 2e-4)
    rep = ep.rep_grad_lp.float().clone()
    pg.all_reduce_tensor(rep)
    want = single.rep_grad_lp.float()
    rel = (rep - want).norm().item() / want.norm().item()
    check(f"replicated gradients (summed over ranks) rel-L2 {rel:.2e}", rel < 3e-2)
    worst = 0.0
    for l, (b1, b2) in enumerate(zip(single.model.blocks, ep.model.blocks)):
        for name in ("up", "down"):
            a = getattr(b2.moe, name).grad.float()
            b = getattr(b1.moe, name).grad.float()[rank * le: (rank + 1) * le]
            worst = max(worst, (a - b).norm().item() / max(b.norm().item(), 1e-12))
    check(f"expert gradients of the local experts: worst rel-L2 {worst:.2e}", worst < 3e-2)
    for tr in (single, ep):
        tr.rep_grad_lp.zero_(); tr.exp_grad.zero_()

    # ---- optimizer steps
    l1, l2 = [], []
    for _ in range(4):
        l1.append(single.step(tokens).clone())
        l2.append(ep.step(tokens[rank: rank + 1]).clone())
    torch.cuda.synchronize(); K.check_status()
    l2 = torch.stack(l2)
    pg.all_reduce_tensor(l2)
    l2 /= world
    l1 = torch.stack(l1)
    check(f"losses over 4 steps: ep {[round(v, 4) for v in l2[:, 0].tolist()]} vs single {[round(v, 4) for v in l1[:, 0].tolist()]}",
          (l1[:, 0] - l2[:, 0]).abs().max().item() < 3e-2 and l2[-1, 0].item() < l2[0, 0].item())
    s1, s2 = single.read_opt_state(), ep.read_opt_state()
    check(f"gradient norm {s2.grad_norm:.5f} vs {s1.grad_norm:.5f}; steps {s2.step}",
          abs(s1.grad_norm - s2.grad_norm) < 3e-2 * s1.grad_norm and s2.step == 4)

    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    pg.all_reduce_tensor(flag, "min")
    if rank == 0:
        print("WORKER_OK" if flag.item() == 1.0 else "WORKER_FAILED", flush=True)
    pg.destroy()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
