"""2+ GPU worker (one rank per GPU, launched by torch.distributed.run): checks the fused
peer-memory paths against single-GPU / PyTorch references.  Prints 'WORKER_OK' on rank 0."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from nexus_b200.lm.config import preset  # noqa: E402
from nexus_b200.models.gpt import AdamWConfig, GptModel  # noqa: E402
from nexus_b200.ops import _cuda as K  # noqa: E402
from nexus_b200.parallel.process_group import init_process_group  # noqa: E402
from nexus_b200.parallel.symm import (FusedShardedOptimizer, RingAttention, SymmetricWorkspace,  # noqa: E402
                                      fused_all_reduce, gemm_dist, moe_combine, moe_dispatch, ulysses_attention,
                                      vocab_parallel_cross_entropy)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    pg = init_process_group("nccl", dev)
    ws = SymmetricWorkspace(pg)
    ok = True

    def check(name, cond):
        nonlocal ok
        ok &= bool(cond)
        if rank == 0:
            print(("OK  " if cond else "BAD ") + name, flush=True)

    # ---- barrier
    for _ in range(3):
        ws.barrier()
    torch.cuda.synchronize()
    K.check_status()
    check("barrier", True)

    # ---- fused sharded optimizer vs single-GPU run of the same global batch
    cfg = preset("gpt2-124m")
    cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab_size, cfg.max_position = 2, 128, 2, 512, 500, 128
    g = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, cfg.vocab_size, (world, 2, 128), generator=g, dtype=torch.int32).to(dev)
    ref = GptModel(cfg, device=dev, seed=11)
    ref.set_optimizer(AdamWConfig(lr=1e-3))
    init = ref.params.clone()
    model = GptModel(cfg, device=dev, seed=11)
    model.set_optimizer(AdamWConfig(lr=1e-3))
    opt = FusedShardedOptimizer(model, ws)
    for step in range(3):
        for r in range(world):
            ref.forward_backward(tokens[r], grad_scale=1.0 / world, accumulate_loss=r > 0, loss_weight=1.0 / world)
        ref.optimizer_step()
        model.forward_backward(tokens[rank], grad_scale=1.0 / world, loss_weight=1.0 / world)
        opt.step()
    torch.cuda.synchronize()
    K.check_status()
    full = opt.gather_master()
    # Adam's first updates are +-lr whatever the gradient's size, so an element whose tiny gradient
    # rounds differently (atomic split-K order) moves by 2*lr: compare in L2 relative to the update
    upd = (ref.params - init).norm().item()
    err = (full - ref.params).norm().item() / upd
    err_lp = (model.params_lp.float() - ref.params_lp.float()).norm().item() / upd
    frac = ((full - ref.params).abs() > 2e-4).float().mean().item()
    s1, s2 = model.read_opt_state(), ref.read_opt_state()
    check(f"sharded optimizer rel-L2 master {err:.2e} shadow {err_lp:.2e} outliers {frac:.2e}",
          err < 0.05 and err_lp < 0.08 and frac < 0.01)
    check(f"grad norm {s1.grad_norm:.5f} vs {s2.grad_norm:.5f}", abs(s1.grad_norm - s2.grad_norm) < 1e-3 * s2.grad_norm)

    # ---- the same three steps with the reduce-scatter and the all-gather going through NVSwitch (opt-in form)
    if opt.grads.multicast and opt.shadow.multicast and opt.tail.multicast:
        os.environ["NEXUS_B200_SHARDED_MULTIMEM"] = "1"
        model_mc = GptModel(cfg, device=dev, seed=11)
        model_mc.set_optimizer(AdamWConfig(lr=1e-3))
        opt_mc = FusedShardedOptimizer(model_mc, ws)
        for step in range(3):
            model_mc.forward_backward(tokens[rank], grad_scale=1.0 / world, loss_weight=1.0 / world)
            opt_mc.step()
        torch.cuda.synchronize()
        K.check_status()
        os.environ["NEXUS_B200_SHARDED_MULTIMEM"] = "0"
        err_mc = (opt_mc.gather_master() - ref.params).norm().item() / upd
        err_mc_lp = (model_mc.params_lp.float() - ref.params_lp.float()).norm().item() / upd
        check(f"sharded optimizer through NVSwitch rel-L2 master {err_mc:.2e} shadow {err_mc_lp:.2e}",
              err_mc < 0.05 and err_mc_lp < 0.08)
    elif rank == 0:
        print("--  sharded optimizer through NVSwitch: no multicast address on this fabric", flush=True)

    # ---- checkpoint of the sharded state: save -> train -> load -> the same step again gives the same result,
    # ---- and every rank's shard together loads into an unsharded backend (2 -> 1 reshard)
    import torch.distributed as dist
    from nexus_b200.train.gpt_backend import GptLmBackend
    bk = GptLmBackend(cfg, 2, 128, device=dev, seed=11)
    bk.attach_fsdp(pg)
    for step in range(2):
        bk.device_step(tokens[rank], lr=1e-3)
    blob = bk.save_state()
    saved_master = bk._sharded.gather_master().clone()
    bk.device_step(tokens[rank], lr=1e-3)
    torch.cuda.synchronize()
    after_master = bk._sharded.gather_master().clone()
    after_loss = bk.model.loss_buf.clone()
    check("sharded state moved between save and the next step", (after_master - saved_master).abs().max().item() > 0)
    bk.load_state(blob)
    torch.cuda.synchronize()
    check("sharded load_state restores the master shard", torch.equal(bk._sharded.gather_master(), saved_master))
    check("sharded load_state rebuilds the BF16 weights",
          torch.equal(bk.model.params_lp[: bk.model.num_params], saved_master.bfloat16()))
    bk.device_step(tokens[rank], lr=1e-3)
    torch.cuda.synchronize(); K.check_status()
    again = bk._sharded.gather_master()
    d_resume = (again - after_master).norm().item() / max((after_master - saved_master).norm().item(), 1e-12)
    check(f"resume reproduces the next step (rel diff of the update {d_resume:.2e}, loss {bk.model.loss_buf.item():.5f} vs "
          f"{after_loss.item():.5f})", d_resume < 5e-2 and abs(bk.model.loss_buf.item() - after_loss.item()) < 1e-4)
    blobs = [None] * world
    dist.all_gather_object(blobs, blob)
    single = GptLmBackend(cfg, 2, 128, device=dev, seed=99)        # different init: everything must come from the blobs
    single.load_resharded_state(blobs)
    torch.cuda.synchronize()
    check("2 -> 1 reshard: full master from the shards", torch.equal(single.model.params, saved_master))
    st_a, st_b = single.model.read_opt_state(), bk.model.read_opt_state()
    check("2 -> 1 reshard: optimizer step counter", st_a.step == 2 and st_b.step == 3)
    del single

    # ---- the whole sharded step captured in a CUDA graph: replays must still wait at the cross-GPU barriers
    from nexus_b200.train.lm_trainer import AdamW, LanguageTrainerBuilder, SyntheticTokens
    hist = {}
    for graph in (False, True):
        tr = (LanguageTrainerBuilder(cfg).data(SyntheticTokens(cfg.vocab_size, seed=5, rank=rank, world=world))
              .optimizer(AdamW(lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1))
              .micro_batch(2).seq_len(128).global_batch_tokens(2 * 128 * world).grad_clip(1.0)
              .precision("bf16", "fp32").execution_policy(dev).log_every(0).seed(21).compile(graph).fsdp(pg, None).build())
        tr.train(6)
        torch.cuda.synchronize(); K.check_status()
        hist[graph] = ([h.loss for h in tr.history], tr.backend._sharded.gather_master().clone())
    dl = max(abs(a - b) for a, b in zip(*[hist[g][0] for g in (False, True)]))
    dm = (hist[True][1] - hist[False][1]).norm().item() / hist[False][1].norm().item()
    check(f"graph-captured sharded step == eager sharded step (max loss diff {dl:.2e}, master rel diff {dm:.2e})",
          dl < 5e-3 and dm < 1e-3)

    # ---- data parallel: buckets reduced by the peer-memory kernel during the backward pass == one NCCL all-reduce
    import types
    finals = {}
    for bucketed in (False, True):
        b = GptLmBackend(cfg, 2, 128, device=dev, seed=11)
        b.attach_process_group(pg, types.SimpleNamespace(bucketed=bucketed, bucket_layers=1))
        for step in range(3):
            b.device_step(tokens[rank], lr=1e-3)
        torch.cuda.synchronize(); K.check_status()
        finals[bucketed] = (b.model.params.clone(), b.model.read_opt_state().grad_norm,
                            0 if b._ddp is None else b._ddp["buckets"])
    upd = (finals[False][0] - init).norm().item()
    dd = (finals[True][0] - finals[False][0]).norm().item() / upd
    check(f"bucketed overlapped DDP == flat all-reduce (rel diff of the update {dd:.2e}, grad norm "
          f"{finals[True][1]:.5f} vs {finals[False][1]:.5f}, {finals[True][2]} buckets)",
          dd < 5e-2 and abs(finals[True][1] - finals[False][1]) < 1e-3 * finals[False][1] and finals[True][2] == 3 * 4)

    # ---- all-reduce with the cast fused in (BF16 in -> FP32 out), two-shot and one-shot
    for count, one_shot in ((1 << 20, False), (4096, True), (1000 * 8, False)):
        src = ws.alloc(count, torch.bfloat16)
        dst = ws.alloc(count, torch.float32)
        gen = torch.Generator(device=dev).manual_seed(100 + rank)
        src.local.copy_(torch.randn(count, device=dev, generator=gen).bfloat16())
        want = src.local.float().clone()
        pg.all_reduce_tensor(want)
        fused_all_reduce(ws, src, dst, count, scale=0.5, one_shot=one_shot)
        torch.cuda.synchronize()
        check(f"fused all-reduce bf16->fp32 n={count} one_shot={one_shot}",
              (dst.local - 0.5 * want).abs().max().item() < 1e-5)

    # ---- the same sum formed inside NVSwitch (multimem), in place, FP32 and BF16; skipped where the allocation has no
    # multicast address
    from nexus_b200.parallel.symm import multimem_all_reduce
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        count = (1 << 20) + 64
        buf = ws.alloc(count, dt)
        gen = torch.Generator(device=dev).manual_seed(200 + rank)
        buf.local.copy_(torch.randn(count, device=dev, generator=gen).to(dt))
        want = buf.local.float().clone()
        pg.all_reduce_tensor(want)
        head = buf.local[:64].clone()
        done = multimem_all_reduce(ws, buf, count - 64, offset=64, scale=0.5)
        torch.cuda.synchronize()
        K.check_status(dev)
        if done:
            check(f"in-switch all-reduce {str(dt)[6:]} n={count - 64}",
                  (buf.local[64:].float() - 0.5 * want[64:]).abs().max().item() < tol * max(1.0, want.abs().max().item())
                  and torch.equal(buf.local[:64], head))
        elif rank == 0:
            print("--  in-switch all-reduce: no multicast address on this fabric, peer-load kernel stays", flush=True)

    # ---- context parallelism: ring attention (contiguous + zigzag) and Ulysses vs full attention
    Bc, Tl, Hc, Dc = 2, 256, 4, 64
    Tfull = Tl * world
    gen = torch.Generator(device=dev).manual_seed(77)
    qf, kf, vf = (torch.randn(Bc, Tfull, Hc, Dc, device=dev, generator=gen).bfloat16() for _ in range(3))
    for t in (qf, kf, vf):
        pg.broadcast_tensor(t, 0)
    ref_o, _ = K.attention_fwd(qf, kf, vf, causal=True)
    sl = slice(rank * Tl, (rank + 1) * Tl)
    ring = RingAttention(ws, Bc, Tl, Hc, Dc, "contiguous")
    o, _ = ring.forward(qf[:, sl].contiguous(), kf[:, sl].contiguous(), vf[:, sl].contiguous(), causal=True)
    torch.cuda.synchronize()
    check("ring attention (contiguous)", (o.float() - ref_o[:, sl].float()).abs().max().item() < 3e-2)
    half = Tl // 2
    idx = torch.cat([torch.arange(rank * half, (rank + 1) * half),
                     torch.arange((2 * world - 1 - rank) * half, (2 * world - rank) * half)]).to(dev)
    zz = RingAttention(ws, Bc, Tl, Hc, Dc, "zigzag")
    o, _ = zz.forward(qf[:, idx].contiguous(), kf[:, idx].contiguous(), vf[:, idx].contiguous(), causal=True)
    torch.cuda.synchronize()
    check("ring attention (zigzag)", (o.float() - ref_o[:, idx].float()).abs().max().item() < 3e-2)
    # ring backward: gradients of the local tokens against the backward of full attention over all tokens
    dof = torch.randn(Bc, Tl * world, Hc, Dc, device=dev).bfloat16()
    pg.broadcast_tensor(dof, 0)
    ref_o2, ref_lse = K.attention_fwd(qf, kf, vf, causal=True)
    rdq, rdk, rdv = K.attention_bwd(qf, kf, vf, ref_o2, ref_lse, dof, causal=True)
    for name, ra, tok in (("contiguous", ring, sl), ("zigzag", zz, idx)):
        ql, kl, vl, dl = (t[:, tok].contiguous() for t in (qf, kf, vf, dof))
        ol, lsel = ra.forward(ql, kl, vl, causal=True)
        dq, dk, dv = ra.backward(ql, kl, vl, ol, lsel, dl, causal=True)
        torch.cuda.synchronize()
        good = True
        for got, want in ((dq, rdq[:, tok]), (dk, rdk[:, tok]), (dv, rdv[:, tok])):
            good &= (got.float() - want.float()).abs().max().item() <= 4e-2 * want.float().abs().max().item()
        check(f"ring attention backward ({name})", good)
    o = ulysses_attention(ws, qf[:, sl].contiguous(), kf[:, sl].contiguous(), vf[:, sl].contiguous(), causal=True)
    torch.cuda.synchronize()
    check("ulysses attention", (o.float() - ref_o[:, sl].float()).abs().max().item() < 3e-2)
    K.check_status()

    # ---- vocabulary-parallel cross-entropy: loss and logit gradients vs the full-vocabulary loss
    rows_ce, V = 512, 1024 * world
    gen = torch.Generator(device=dev).manual_seed(91)
    full = torch.randn(rows_ce, V, device=dev, generator=gen) * 3
    tg = torch.randint(0, V, (rows_ce,), device=dev, generator=gen)
    pg.broadcast_tensor(full, 0)
    pg.broadcast_tensor(tg, 0)
    tg[::7] = -100
    ref_full = full.clone().requires_grad_(True)
    ref_loss = torch.nn.functional.cross_entropy(ref_full, tg, ignore_index=-100)
    ref_loss.backward()
    vs = rank * (V // world)
    mine = full[:, vs: vs + V // world].clone().requires_grad_(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(4):
        if it == 3:
            e0.record()
        loss = vocab_parallel_cross_entropy(ws, mine, tg, vs)
        if it == 3:
            e1.record()
    loss.backward()
    torch.cuda.synchronize(); K.check_status()
    check("vocab-parallel CE loss", abs(loss.item() - ref_loss.item()) < 1e-4)
    check("vocab-parallel CE gradient",
          (mine.grad - ref_full.grad[:, vs: vs + V // world]).abs().max().item() < 1e-6)
    if rank == 0:
        print(f"INFO vocab-parallel CE forward incl. exchange: {e0.elapsed_time(e1) * 1e3:.1f} us "
              f"({rows_ce} rows x {V // world} local columns)", flush=True)

    # ---- distributed GEMM: all-gather fused into the GEMM (A sharded / B sharded) and GEMM -> reduce-scatter
    torch.manual_seed(5)
    M, N, Kd = 256 * world, 256 * world, 320
    A = torch.randn(M, Kd, device=dev).bfloat16()
    B = torch.randn(N, Kd, device=dev).bfloat16()
    pg.broadcast_tensor(A, 0)
    pg.broadcast_tensor(B, 0)
    ref_out = A.float() @ B.float().t()
    a_sym = ws.alloc(M // world * Kd, torch.bfloat16)
    a_loc = a_sym.local.view(M // world, Kd)
    a_loc.copy_(A[rank * (M // world): (rank + 1) * (M // world)])
    b_sym = ws.alloc(N // world * Kd, torch.bfloat16)
    b_loc = b_sym.local.view(N // world, Kd)
    b_loc.copy_(B[rank * (N // world): (rank + 1) * (N // world)])
    torch.cuda.synchronize()
    ws.barrier()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    gemm_dist(ws, a_loc, B, out, a_peers=a_sym)
    torch.cuda.synchronize(); K.check_status()
    check("AG(A)->GEMM", (out.float() - ref_out).abs().max() <= 1.5e-2 * ref_out.abs().max())
    gemm_dist(ws, A, b_loc, out, b_peers=b_sym)
    torch.cuda.synchronize(); K.check_status()
    check("AG(B)->GEMM", (out.float() - ref_out).abs().max() <= 1.5e-2 * ref_out.abs().max())
    # row-parallel: each rank holds a K slice; out rows reduce-scattered
    Ks = Kd // world // 8 * 8
    Ak = A[:, rank * Ks: (rank + 1) * Ks].contiguous()
    Bk = B[:, rank * Ks: (rank + 1) * Ks].contiguous()
    o_sym = ws.alloc(M // world * N, torch.float32)
    o_sym.local.zero_()
    torch.cuda.synchronize()
    ws.barrier()
    gemm_dist(ws, Ak, Bk, o_sym.local.view(M // world, N), out_peers=o_sym, m=M, n=N)
    ws.barrier()
    torch.cuda.synchronize(); K.check_status()
    ref_rs = A[:, : Ks * world].float() @ B[:, : Ks * world].float().t()
    mine = ref_rs[rank * (M // world): (rank + 1) * (M // world)]
    check("GEMM->RS", (o_sym.local.view(M // world, N) - mine).abs().max() <= 1e-2 * ref_rs.abs().max())

    # ---- GEMM -> reduce-scatter, slot form (BF16 on the wire, owner sums the slots in rank order): deterministic
    from nexus_b200.parallel.symm import sum_slots
    slots = ws.alloc(world * (M // world) * N, torch.bfloat16)
    res = torch.randn(M // world, N, device=dev)
    outs = []
    for rep in range(2):
        ws.barrier()
        gemm_dist(ws, Ak, Bk, slots.local.view(M, N), out_peers=slots, scatter="slots", m=M, n=N)
        ws.barrier()
        z = torch.empty(M // world, N, device=dev)
        z_lp = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
        sum_slots(slots.local, world, M // world, N, z, residual=res, out_lp=z_lp)
        torch.cuda.synchronize(); K.check_status()
        outs.append(z.clone())
    check("GEMM->RS (slots) + residual", (outs[0] - res - mine).abs().max() <= 1.5e-2 * ref_rs.abs().max())
    check("GEMM->RS (slots) is bit-reproducible", torch.equal(outs[0], outs[1]) and torch.equal(z_lp, z.bfloat16()))

    # ---- all-gather fused into the CTA-pair GEMM (push form): result, gathered copy, repeated calls
    from nexus_b200.parallel.symm import GatherSite, gemm_ag
    Mg_l, Kg, Ng = 512, 320, 384
    site = GatherSite(ws, Mg_l)
    Xg_full = torch.randn(Mg_l * world, Kg, device=dev).bfloat16()
    Wg = torch.randn(Ng, Kg, device=dev).bfloat16()
    pg.broadcast_tensor(Xg_full, 0)
    pg.broadcast_tensor(Wg, 0)
    xg = ws.alloc(Mg_l * world * Kg, torch.bfloat16)
    good = True
    for rep in range(3):
        xv = xg.local.view(Mg_l * world, Kg)
        xv.zero_()
        xv[rank * Mg_l: (rank + 1) * Mg_l].copy_(Xg_full[rank * Mg_l: (rank + 1) * Mg_l] * (rep + 1))
        ws.barrier()
        yg = torch.empty(Mg_l * world, Ng, device=dev, dtype=torch.bfloat16)
        gemm_ag(site, xg, Wg, yg, k=Kg, copier_ctas=4)
        torch.cuda.synchronize(); K.check_status()
        ref_g = (Xg_full.float() * (rep + 1)) @ Wg.float().t()
        good &= bool((yg.float() - ref_g).abs().max() <= 1.5e-2 * ref_g.abs().max())
        good &= torch.equal(xv, (Xg_full * (rep + 1)))
        ws.barrier()
    check("AG->GEMM, push form on the CTA-pair kernel (3 calls, gathered copy complete)", good)

    # ---- GEMM -> reduce-scatter in one kernel (push form on the CTA-pair kernel), three calls, vs FP32 reference
    from nexus_b200.parallel.symm import gemm_rs
    Mr, Nr, Kr = 512 * world, 384, 192
    Ar = torch.randn(Mr, Kr, device=dev).bfloat16()              # this rank's K slice of A and B (different per rank)
    Br = torch.randn(Nr, Kr, device=dev).bfloat16()
    prod = Ar.float() @ Br.float().t()
    want = prod.clone()
    pg.all_reduce_tensor(want)
    slots_r = ws.alloc(world * (Mr // world) * Nr, torch.bfloat16)
    partial_r = torch.empty(Mr, Nr, device=dev, dtype=torch.bfloat16)
    done_r = torch.zeros(Mr // 256, dtype=torch.int32, device=dev)
    good = True
    for rep in range(3):
        ws.barrier()
        own_rows = partial_r[rank * (Mr // world): (rank + 1) * (Mr // world)]
        gemm_rs(ws, Ar, Br, partial_r, slots_r, done_r, copier_ctas=4, copy_own=(rep == 2))
        ws.barrier()
        zr = torch.empty(Mr // world, Nr, device=dev)
        sum_slots(slots_r.local, world, Mr // world, Nr, zr, own=None if rep == 2 else own_rows, own_rank=rank)
        torch.cuda.synchronize(); K.check_status()
        mine_r = want[rank * (Mr // world): (rank + 1) * (Mr // world)]
        good &= bool((zr - mine_r).abs().max() <= 2e-2 * want.abs().max())
        slots_r.local.zero_()
        torch.cuda.synchronize()
    check("GEMM->RS, push form on the CTA-pair kernel (3 calls)", good)

    # ---- MN-major operands in the distributed GEMM: dgrad with all-gathered rows, wgrad over K-sharded rows
    W_mn = torch.randn(Kd, 384, device=dev).bfloat16()          # B stored [K][N]
    pg.broadcast_tensor(W_mn, 0)
    out_d = torch.empty(M, 384, device=dev, dtype=torch.bfloat16)
    gemm_dist(ws, a_loc, W_mn, out_d, a_peers=a_sym, b_mn=True)
    torch.cuda.synchronize(); K.check_status()
    ref_d = A.float() @ W_mn.float()
    check("AG(A)->GEMM with MN-major B (dgrad form)", (out_d.float() - ref_d).abs().max() <= 1.5e-2 * ref_d.abs().max())
    Mk = 128 * world                                            # contraction length, 128 rows per rank
    Xs = ws.alloc(128 * 384, torch.bfloat16)                     # this rank's rows of X [Mk, 384]
    Xfull = torch.randn(Mk, 384, device=dev).bfloat16()
    dYfull = torch.randn(Mk, 256, device=dev).bfloat16()
    pg.broadcast_tensor(Xfull, 0)
    pg.broadcast_tensor(dYfull, 0)
    Xs.local.view(128, 384).copy_(Xfull[rank * 128: (rank + 1) * 128])
    torch.cuda.synchronize(); ws.barrier()
    dW = torch.ones(256, 384, device=dev)
    gemm_dist(ws, dYfull, Xs.local.view(128, 384), dW, b_peers=Xs, a_mn=True, b_mn=True, b_shard="k", accumulate=True)
    torch.cuda.synchronize(); K.check_status()
    ref_w = 1.0 + dYfull.float().t() @ Xfull.float()
    check("wgrad with K-sharded B (beta = 1)", (dW - ref_w).abs().max() <= 1.5e-2 * ref_w.abs().max())
    dYs = ws.alloc(128 * 256, torch.bfloat16)
    dYs.local.view(128, 256).copy_(dYfull[rank * 128: (rank + 1) * 128])
    torch.cuda.synchronize(); ws.barrier()
    dW2 = torch.zeros(256, 384, device=dev)
    gemm_dist(ws, dYs.local.view(128, 256), Xfull, dW2, a_peers=dYs, a_mn=True, b_mn=True, a_shard="k")
    torch.cuda.synchronize(); K.check_status()
    check("wgrad with K-sharded A", (dW2 - (ref_w - 1.0)).abs().max() <= 1.5e-2 * ref_w.abs().max())
    ws.barrier()

    # ---- MoE dispatch / combine over peer memory (identity experts)
    E, k, d, T, cap = 2 * world, 2, 64, 32, 64
    le = E // world
    x = torch.randn(T, d, device=dev).bfloat16()
    expert = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).to(torch.int32)
    gate = torch.softmax(torch.randn(T, k, device=dev), -1)
    # global slot of an assignment inside its expert: rank-major, then token order (counts exchanged through NCCL)
    onehot = torch.nn.functional.one_hot(expert.long().reshape(-1), E)
    counts = onehot.sum(0)
    allc = torch.empty(world * E, dtype=counts.dtype, device=dev)
    pg.all_gather_tensor(allc, counts)
    base = allc.view(world, E)[:rank].sum(0)
    within = (onehot.cumsum(0) - 1).gather(1, expert.long().reshape(-1, 1))[:, 0]
    slot = (base[expert.long().reshape(-1)] + within).to(torch.int32)
    bufs = ws.alloc(le * cap * d, torch.bfloat16)
    bufs.local.zero_()
    torch.cuda.synchronize()
    ws.barrier()
    token_of = (torch.arange(T * k, device=dev) // k).to(torch.int32)
    moe_dispatch(ws, x, token_of, expert.reshape(-1).contiguous(), slot, bufs, le, cap)
    ws.barrier()
    y = torch.empty(T, d, device=dev, dtype=torch.bfloat16)
    moe_combine(ws, bufs, expert.contiguous(), slot.view(T, k).contiguous(), gate.contiguous(), y, le, cap)
    ws.barrier()
    torch.cuda.synchronize(); K.check_status()
    check("MoE dispatch+combine", (y.float() - x.float() * gate.sum(-1, keepdim=True)).abs().max() < 3e-2)

    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    pg.all_reduce_tensor(flag, "min")
    if rank == 0:
        print("WORKER_OK" if flag.item() == 1.0 else "WORKER_FAILED", flush=True)
    pg.destroy()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
