"""FullShard FSDP on GPUs (one rank per GPU): the unit engine of `parallel/fsdp.py` with its two communication forms.

* equivalence: stage 3 with shards gathered by peer loads and gradients reduce-scattered by owner pull over symmetric
  memory ("fused") trains to the parameters of the NCCL form and of a single process, FP32 and BF16 wire formats;
  per-rank persistent parameter + optimizer bytes are 1 / ranks of the model's.
* ``--bench``: milliseconds per optimizer step of both forms on a GPT-2 124M shaped `LanguageModel`.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port P \
        tests/workers/fsdp_gpu_worker.py [--bench]
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main() -> int:
    from nexus_b200.lm.config import preset
    from nexus_b200.lm.model import LanguageModel
    from nexus_b200.train.lm_trainer import AdamW
    from nexus_b200.ops import _cuda as K
    from nexus_b200.parallel import FsdpEngine, FsdpOptions
    from nexus_b200.parallel.process_group import init_process_group
    from nexus_b200.fused.ops import adamw_multi_tensor

    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    pg = init_process_group("nccl", f"cuda:{local}")
    ok = True

    def check(name, cond):
        nonlocal ok
        ok &= bool(cond)
        if rank == 0:
            print(("OK  " if cond else "BAD ") + name, flush=True)

    if "--bench" in sys.argv:
        cfg = preset("gpt2-124m")
        cfg.max_position = 1024
        torch.manual_seed(0)
        rows = []
        for comm in ("nccl", "fused"):
            m = LanguageModel(cfg).to(dev)
            eng = FsdpEngine(m, pg, FsdpOptions(stage=3, mixed_precision=True, comm=comm))
            gen = torch.Generator(device=dev).manual_seed(1 + rank)
            opt = AdamW()

            def step():
                toks = torch.randint(0, cfg.vocab_size, (8, 1024), device=dev, generator=gen)
                eng.forward_backward(lambda: m.loss(toks), 1.0)
                eng.step(opt, 3e-4, 1.0)
            for _ in range(2):
                step()
            pg.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(4):
                step()
            e1.record()
            torch.cuda.synchronize()
            ms = float(pg.all_reduce_scalar(e0.elapsed_time(e1) / 4, "max"))
            rows.append({"comm": eng.comm(), "ms_per_step": round(ms, 2),
                         "tokens_per_s": round(world * 8 * 1024 / (ms * 1e-3))})
            del eng, m
            torch.cuda.empty_cache()
        if rank == 0:
            print(json.dumps({"bench": "FullShard FSDP, LanguageModel gpt2-124m, 8 x 1024 tokens per GPU, BF16 gather / reduce",
                              "n_gpus": world, "rows": rows}), flush=True)
        K.check_status(dev)
        pg.destroy()
        return 0

    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.max_position, cfg.vocab_size = 4, 128, 2, 256, 64, 512
    torch.manual_seed(0)
    data = torch.randint(0, cfg.vocab_size, (4 * world, 64), device=dev)
    pg.broadcast_tensor(data, 0)

    def train(comm, mixed, stage=3):
        torch.manual_seed(0)
        m = LanguageModel(cfg).to(dev)
        wd = [1.0 if p.dim() >= 2 else 0.0 for p in m.parameters()]
        eng = FsdpEngine(m, pg, FsdpOptions(stage=stage, mixed_precision=mixed, comm=comm))
        for s in range(2):
            for i in range(2):
                idx = rank * 2 + i
                eng.forward_backward(lambda: m.loss(data[idx * 2:(idx + 1) * 2]), 1.0 / (2 * world), sync=i == 1)
            eng.step(AdamW(), 1e-3, 1.0, wd, None)
        torch.cuda.synchronize()
        K.check_status(dev)
        persistent = sum(u.master.numel() * 4 * 3 for u in eng.units)          # master + m + v shards
        return eng.full_parameters(), eng.comm(), eng.trace(), persistent, sum(u.N for u in eng.units)

    # single process on the same data
    torch.manual_seed(0)
    ref_m = LanguageModel(cfg).to(dev)
    ps = list(ref_m.parameters())
    mm, vv = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
    wd = [1.0 if p.dim() >= 2 else 0.0 for p in ps]
    for s in range(2):
        for i in range(2 * world):
            (ref_m.loss(data[i * 2:(i + 1) * 2]) / (2 * world)).backward()
        adamw_multi_tensor([p.data for p in ps], [p.grad for p in ps], mm, vv, s + 1, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1.0, wd)
        for p in ps:
            p.grad = None
    ref = [p.detach().clone() for p in ps]

    key = lambda t: (t.numel(), round(float(t.double().abs().sum()), 3))
    for mixed in (False, True):
        pn, cn, _, _, _ = train("nccl", mixed)
        pf, cf, tr, persistent, total = train("fused", mixed)
        check(f"forms in use: {cn} / {cf}", cn == "nccl" and cf == "fused")
        d_forms = max(float((a - b).abs().max()) for a, b in zip(pf, pn))
        tol_forms = 1e-6 if not mixed else 2e-3
        check(f"stage 3, {'bf16' if mixed else 'fp32'} wire: fused vs NCCL max diff {d_forms:.2e}", d_forms <= tol_forms)
        d_ref = max(float((a - b).abs().max()) for a, b in zip(sorted(pf, key=key), sorted(ref, key=key)))
        check(f"stage 3, {'bf16' if mixed else 'fp32'} wire: fused vs single process max diff {d_ref:.2e}",
              d_ref <= (2e-4 if not mixed else 5e-3))
        check("gathers are prefetched and the reduce-scatters run in backward order",
              any(e.startswith("gather:h1") for e in tr) and tr.index("reduce:h3") < tr.index("reduce:h0"))
        check(f"persistent master + moment bytes per rank {persistent} ~ 12 x parameters / ranks ({12 * total // world})",
              12 * total // world <= persistent <= 12 * total // world + 12 * 64)
    pg.barrier()
    if rank == 0:
        print("WORKER_OK" if ok else "WORKER_FAILED", flush=True)
    pg.destroy()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
