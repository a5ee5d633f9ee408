"""Distributed engines without a cluster: N ranks as N threads (ThreadWorld) and real gloo processes."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest
import torch

from nexus_b200.lm import LanguageModel, preset
from nexus_b200.parallel import (DdpEngine, DdpOptions, DistError, DistTimeout, FsdpEngine, FsdpOptions, GroupOptions,
                                 LocalBoard, Watchdog, WatchdogOptions, plan_buckets, run_threads, scaled_lr)
from nexus_b200.parallel.context_parallel import ring_attention, shard_sequence, ulysses_attention, unshard_sequence
from nexus_b200.parallel.dtensor import DeviceMesh, DTensor, Partial, Replicate, Shard, dt_matmul
from nexus_b200.parallel.moe_ep import MoeExpertParallel
from nexus_b200.parallel.parallel_lm import ParallelConfig, ParallelLm
from nexus_b200.parallel.pipeline import balance_partition, make_schedule, simulate_bubble, theoretical_bubble
from nexus_b200.train.lm_trainer import AdamW

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tiny_cfg(kind="gpt"):
    if kind == "gpt":
        c = preset("nano")
        c.n_layer, c.d_model, c.n_head, c.d_ff, c.max_position, c.vocab_size = 4, 32, 4, 64, 32, 67
    else:
        c = preset("tinyllama-1.1b")
        c.n_layer, c.d_model, c.n_head, c.n_kv_head, c.d_ff, c.max_position, c.vocab_size = 4, 32, 4, 2, 48, 32, 67
    return c


# ------------------------------------------------------------------------------------- collectives
def test_collectives_on_thread_world():
    def f(pg):
        r, n = pg.rank(), pg.size()
        t = torch.full((4,), float(r + 1))
        pg.all_reduce_tensor(t, "sum")
        mx = torch.tensor([float(r)])
        pg.all_reduce_tensor(mx, "max")
        rs = torch.empty(2)
        pg.reduce_scatter_tensor(rs, torch.arange(8.0) + r, "sum")
        ag = torch.empty(8)
        pg.all_gather_tensor(ag, torch.full((2,), float(r)))
        b = torch.tensor([float(r)])
        pg.broadcast_tensor(b, 2)
        a2a = pg.all_to_all_v([torch.full((d + 1,), float(r)) for d in range(n)])
        sub = pg.new_group([0, 1])
        sub2 = pg.new_group([2, 3])
        s = torch.ones(1)
        (sub or sub2).all_reduce_tensor(s)
        h = torch.ones(8) * (r + 1)
        pg.all_reduce_hierarchical(h, 2)
        rv = torch.empty(1)
        pg.send_recv(torch.tensor([float(r)]), (r + 1) % n, rv, (r - 1) % n)
        half = torch.ones(2, dtype=torch.bfloat16) * (r + 1)
        pg.all_reduce_tensor(half, "avg")
        pg.barrier()
        return (t[0].item(), mx.item(), rs.tolist(), ag.tolist(), b.item(), [x.numel() for x in a2a], s.item(), h[0].item(),
                rv.item(), half[0].item(), pg.all_reduce_scalar(3, "sum"))
    res = run_threads(4, f)
    for r, out in enumerate(res):
        assert out[0] == 10.0 and out[1] == 3.0 and out[2] == [6.0 + 8 * r, 10.0 + 8 * r]
        assert out[3] == [0, 0, 1, 1, 2, 2, 3, 3] and out[4] == 2.0 and out[5] == [r + 1] * 4
        assert out[6] == 2.0 and out[7] == 10.0 and out[8] == (r - 1) % 4 and out[9] == 2.5 and out[10] == 12


def test_validate_mode_turns_a_mismatch_into_a_named_error():
    def bad(pg):
        t = torch.ones(2)
        if pg.rank() == 0:
            pg.all_reduce_tensor(t)
        else:
            pg.broadcast_tensor(t, 0)
    with pytest.raises(DistError, match="mismatched collective"):
        run_threads(2, bad, GroupOptions(timeout_s=5, validate=True))


def test_missing_rank_times_out_and_poisons_the_group():
    seen = {}

    def f(pg):
        if pg.rank() == 1:
            return "absent"                   # never joins the collective
        t = torch.ones(1)
        t0 = time.monotonic()
        try:
            pg.all_reduce_tensor(t)
        except DistTimeout:
            seen["dt"] = time.monotonic() - t0
            with pytest.raises(DistError):
                pg.barrier()                  # the group is broken from now on
            return "timeout"
    res = run_threads(2, f, GroupOptions(timeout_s=0.5))
    assert res == ["timeout", "absent"] and 0.4 < seen["dt"] < 3.0


def test_rank_raising_an_exception_surfaces_it():
    def f(pg):
        if pg.rank() == 1:
            raise KeyError("rank 1 failed on the host")
        pg.barrier()
    with pytest.raises(KeyError):
        run_threads(2, f, GroupOptions(timeout_s=2))


# ---------------------------------------------------------------------------------------- DDP/FSDP
def single_rank_reference(cfg, data, steps=2, micro=4):
    from nexus_b200.fused.ops import adamw_multi_tensor
    m = LanguageModel(cfg)
    ps = list(m.parameters())
    mm, vv = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
    wd = [1.0 if p.dim() >= 2 else 0.0 for p in ps]
    for s in range(steps):
        for i in range(micro):
            (m.loss(data[i * 2:(i + 1) * 2]) / micro).backward()
        adamw_multi_tensor([p.data for p in ps], [p.grad for p in ps], mm, vv, s + 1, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1.0, wd)
        for p in ps:
            p.grad = None
    return [p.detach().clone() for p in ps]


def test_ddp_matches_single_rank_and_overlaps():
    assert plan_buckets([10, 10, 10, 10], [3, 2, 1, 0], 20) == [[3, 2], [1, 0]]
    assert scaled_lr(1.0, 4, "sqrt") == 2.0 and scaled_lr(1.0, 4, "linear") == 4.0
    cfg = tiny_cfg()
    torch.manual_seed(0)
    data = torch.randint(0, 67, (8, 32))
    ref = single_rank_reference(cfg, data)

    def f(pg):
        from nexus_b200.fused.ops import adamw_multi_tensor
        m = LanguageModel(cfg)
        ps = list(m.parameters())
        eng = DdpEngine(ps, pg, DdpOptions(bucket_bytes=20000))
        mm, vv = [torch.zeros_like(p) for p in ps], [torch.zeros_like(p) for p in ps]
        wd = [1.0 if p.dim() >= 2 else 0.0 for p in ps]
        for s in range(2):
            for i in range(2):                     # 2 micro-steps per rank, no_sync on the first
                idx = pg.rank() * 2 + i
                with eng.backward_context(sync=i == 1):
                    (m.loss(data[idx * 2:(idx + 1) * 2]) / 4).backward()
            eng.finish()
            adamw_multi_tensor([p.data for p in ps], [p.grad for p in ps], mm, vv, s + 1, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1.0, wd)
            for p in ps:
                p.grad = None
        return [p.detach().clone() for p in ps], eng.stats, len(eng.buckets)
    res = run_threads(2, f)
    for a, b in zip(res[0][0], ref):
        assert torch.allclose(a, b, atol=2e-6)
    st = res[0][1]
    assert res[0][2] > 1 and st.first_comm_start_ms < st.backward_ms      # communication started during backward


@pytest.mark.parametrize("stage", (0, 1, 2, 3))
def test_fsdp_stages_agree_with_single_rank(stage):
    cfg = tiny_cfg()
    torch.manual_seed(0)
    data = torch.randint(0, 67, (8, 32))
    ref = single_rank_reference(cfg, data)

    def f(pg):
        m = LanguageModel(cfg)
        wd = [1.0 if p.dim() >= 2 else 0.0 for p in m.parameters()]
        eng = FsdpEngine(m, pg, FsdpOptions(stage=stage))
        for s in range(2):
            for i in range(2):
                idx = pg.rank() * 2 + i
                eng.forward_backward(lambda: m.loss(data[idx * 2:(idx + 1) * 2]), 0.25, sync=i == 1)
            eng.step(AdamW(), 1e-3, 1.0, wd, None)
        return eng.full_parameters(), eng.trace(), eng.save_state()
    res = run_threads(2, f)
    key = lambda t: (t.numel(), round(float(t.double().sum()), 6))
    for a, b in zip(sorted(res[0][0], key=key), sorted(ref, key=key)):
        assert torch.allclose(a, b, atol=3e-6)
    tr = res[0][1]
    if stage == 3:
        assert any(e.startswith("gather:h1:prefetch") or e.startswith("gather:h1:fwd") for e in tr)
        assert tr.index("reduce:h3") < tr.index("reduce:h0")          # reduce-scatter in backward order
    test_fsdp_stages_agree_with_single_rank.blobs = [r[2] for r in res]


def test_fsdp_reshard_2_to_4_ranks():
    test_fsdp_stages_agree_with_single_rank(3)
    blobs = test_fsdp_stages_agree_with_single_rank.blobs
    cfg = tiny_cfg()

    def f(pg):
        m = LanguageModel(cfg)
        eng = FsdpEngine(m, pg, FsdpOptions(stage=3))
        eng.load_resharded(blobs)
        return eng.full_parameters(), eng.steps

    def g(pg):
        m = LanguageModel(cfg)
        eng = FsdpEngine(m, pg, FsdpOptions(stage=3))
        eng.load_state(blobs[pg.rank()])
        return eng.full_parameters()
    four, two = run_threads(4, f), run_threads(2, g)
    assert four[0][1] == 2
    for a, b in zip(four[0][0], two[0]):
        assert torch.equal(a, b)


# ----------------------------------------------------------------------------- TP / SP / PP / CP
PAR_CASES = [ParallelConfig(tp=2), ParallelConfig(tp=2, sp=True, async_tp=True), ParallelConfig(pp=2, pp_schedule="gpipe"),
             ParallelConfig(pp=2, pp_schedule="zb_h1"), ParallelConfig(pp=2, pp_schedule="interleaved_1f1b", virtual_stages=2),
             ParallelConfig(cp=2), ParallelConfig(cp=2, cp_algorithm="ulysses"), ParallelConfig(dp=2, zero=1),
             ParallelConfig(dp=2, pp=2, cp=2, tp=2, sp=True)]


@pytest.mark.parametrize("kind", ("gpt", "llama"))
@pytest.mark.parametrize("pc", PAR_CASES, ids=lambda p: f"dp{p.dp}pp{p.pp}cp{p.cp}tp{p.tp}{'sp' if p.sp else ''}{p.pp_schedule if p.pp > 1 else ''}{p.cp_algorithm if p.cp > 1 else ''}")
def test_parallel_lm_matches_single_rank(kind, pc):
    cfg = tiny_cfg(kind)
    torch.manual_seed(0)
    data = torch.randint(0, 67, (8, 32))
    m0 = LanguageModel(cfg)
    loss0 = 0.0
    for i in range(4):
        l = m0.loss(data[i * 2:(i + 1) * 2]) * 0.25
        l.backward()
        loss0 += float(l.detach())
    ref = {n: p.grad.clone() for n, p in m0.named_parameters()}

    def f(pg):
        pl = ParallelLm(LanguageModel(cfg), pg, pc)
        per = 4 // pc.dp
        micro = [data[(pl.dp_r * per + i) * 2:(pl.dp_r * per + i + 1) * 2] for i in range(per)]
        loss = pl.forward_backward(micro, [0.25] * per)
        grads = pl.assemble_full("grad")
        return loss, grads, pl.step(AdamW(), 1e-3, 1.0)
    res = run_threads(pc.world(), f)
    assert abs(res[0][0] - loss0) < 5e-6
    norm0 = torch.sqrt(sum(g.double().pow(2).sum() for g in ref.values())).item()
    for r in res:
        assert abs(r[2] - norm0) < 1e-5 * norm0
        for n, g in r[1].items():
            want = ref[n]
            if g.shape[0] != want.shape[0]:
                want = torch.nn.functional.pad(want, (0, 0, 0, g.shape[0] - want.shape[0]))
            assert (g - want).abs().max() < 5e-7, n


def test_pipeline_schedules_and_bubbles():
    assert [str(a) for a in make_schedule("1f1b", 4, 1, 6)][:5] == ["F0.1", "F1.1", "F2.1", "B0.1", "F3.1"]
    for s, v in (("gpipe", 1), ("1f1b", 1), ("interleaved_1f1b", 2)):
        assert simulate_bubble(s, 4, 8, v) == pytest.approx(theoretical_bubble(s, 4, 8, v), abs=1e-9)
    assert theoretical_bubble("zb_h1", 4, 8) < simulate_bubble("zb_h1", 4, 8) < theoretical_bubble("1f1b", 4, 8)
    for s in ("gpipe", "1f1b", "zb_h1"):        # every (mb, chunk) appears once as F and once as B, B in mb order
        for r in range(4):
            acts = make_schedule(s, 4, r, 8)
            assert sorted(a.mb for a in acts if a.kind == "F") == list(range(8))
            assert [a.mb for a in acts if a.kind == "B"] == list(range(8))
    with pytest.raises(ValueError):
        make_schedule("interleaved_1f1b", 4, 0, 6, 2)
    assert balance_partition([1, 2, 3, 4, 5, 6], 3) == [(0, 3), (3, 5), (5, 6)]


def test_context_parallel_matches_full_attention():
    from nexus_b200.fused.ops import attention_reference
    torch.manual_seed(0)
    B, T, H, Hkv, D = 2, 32, 4, 2, 8
    q, k, v, do = (torch.randn(B, T, h, D) for h in (H, Hkv, Hkv, H))
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    oref = attention_reference(qr, kr, vr)
    oref.backward(do)
    for layout, fn, cp in (("zigzag", "ring", 4), ("contiguous", "ring", 2), ("contiguous", "ulysses", 2)):
        def f(pg):
            ql, kl, vl = (shard_sequence(t, cp, pg.rank(), layout).requires_grad_(True) for t in (q, k, v))
            o = ring_attention(ql, kl, vl, pg, layout) if fn == "ring" else ulysses_attention(ql, kl, vl, pg)
            o.backward(shard_sequence(do, cp, pg.rank(), layout))
            return o.detach(), ql.grad, kl.grad, vl.grad
        res = run_threads(cp, f)
        full = [unshard_sequence([r[i] for r in res], cp, layout) for i in range(4)]
        for a, b in zip(full, (oref.detach(), qr.grad, kr.grad, vr.grad)):
            assert (a - b).abs().max() < 5e-6


def test_expert_parallel_matches_single_rank():
    from nexus_b200.moe import Spec
    spec = Spec(experts=8, top_k=2, d_model=16, d_ff=8, capacity_factor=2.0)
    g = torch.Generator().manual_seed(5)
    router, up, down = torch.randn(16, 8, generator=g) * 0.5, torch.randn(8, 16, 16, generator=g) * 0.1, torch.randn(8, 16, 8, generator=g) * 0.1
    X = torch.randn(4, 12, 16, generator=g)
    ref = []
    for r in range(4):
        m = MoeExpertParallel(spec, None, full_up=up, full_down=down, router=router.clone())
        x = X[r].clone().requires_grad_(True)
        y = m(x)
        y.sum().backward()
        ref.append((y.detach(), x.grad, m.up.grad.clone()))

    def f(pg):
        m = MoeExpertParallel(spec, pg, full_up=up, full_down=down, router=router.clone())
        x = X[pg.rank()].clone().requires_grad_(True)
        y = m(x)
        y.sum().backward()
        return y.detach(), x.grad, m.up.grad.clone(), m.stats.rows_sent
    res = run_threads(4, f)
    for a, b in zip(res, ref):
        assert (a[0] - b[0]).abs().max() < 1e-6 and (a[1] - b[1]).abs().max() < 1e-6
    assert (torch.cat([r[2] for r in res]) - sum(r[2] for r in ref)).abs().max() < 1e-6
    assert all(r[3] == 24 for r in res)


def test_dtensor_redistribute_and_matmul():
    def f(pg):
        mesh = DeviceMesh(pg, (2, 2), ("dp", "tp"))
        A, B = torch.arange(32.0).view(4, 8), torch.arange(48.0).view(8, 6) / 10
        a = DTensor.from_full(A, mesh, [Shard(0), Shard(1)])
        b = DTensor.from_full(B, mesh, [Replicate(), Shard(0)])
        c = dt_matmul(a, b)
        ok = [type(p) for p in c.placements] == [Shard, Partial] and torch.allclose(c.full_tensor(), A @ B, atol=1e-4)
        ok &= a.redistribute([Replicate(), Shard(0)]).full_tensor().equal(A)
        ok &= c.redistribute([Shard(0), Shard(1)]).full_tensor().allclose(A @ B, atol=1e-4)
        ok &= mesh.flatten(["dp", "tp"]).size() == 4 and mesh.index("tp") == pg.rank() % 2
        return ok
    assert all(run_threads(4, f))


def test_watchdog_flags_stalled_rank_and_straggler():
    board = LocalBoard()
    events = []
    wd = Watchdog(board, 0, 3, WatchdogOptions(stall_timeout_s=0.2, poll_s=0.02, min_lag_s=0.03), on_event=events.append)
    others = [Watchdog(board, r, 3, monitor=False) for r in (1, 2)]
    for step in range(3):
        wd.beat(step, 10.0)
        others[0].beat(step, 10.0)
        if step < 1:
            others[1].beat(step, 10.0)            # rank 2 stops beating after step 0
        time.sleep(0.02)
    time.sleep(0.5)
    wd.stop()
    assert any(e.kind == "stalled" and e.rank == 2 for e in events)
    board2, ev2 = LocalBoard(), []
    w = Watchdog(board2, 0, 2, WatchdogOptions(min_lag_s=0.03), on_event=ev2.append, monitor=False)
    w2 = Watchdog(board2, 1, 2, monitor=False)
    w.beat(5, 20.0)
    time.sleep(0.06)
    w2.beat(5, 20.0)                             # 60 ms late
    w.check_once()
    assert [e.kind for e in ev2] == ["straggler"] and ev2[0].rank == 1


# --------------------------------------------------------------------------------- real processes
WORKER = r"""
import os, sys, torch
sys.path.insert(0, %r)
from nexus_b200.parallel.process_group import init_process_group, GroupOptions, DistError
pg = init_process_group("gloo", options=GroupOptions(timeout_s=4.0))
t = torch.ones(4) * (pg.rank() + 1)
pg.all_reduce_tensor(t)
assert t[0].item() == sum(range(1, pg.size() + 1))
pg.barrier()
if os.environ.get("FAIL_RANK") == str(pg.rank()):
    os._exit(3)                                   # dies between steps, nothing in flight
if os.environ.get("FAIL_RANK") is not None:
    try:
        pg.all_reduce_tensor(t)
        pg.all_reduce_tensor(t)
    except DistError:
        os._exit(4)                               # survivors see a named error, not a hang
    os._exit(5)
print("ok", pg.rank())
"""


def _launch(n, port, extra_env=None):
    procs = []
    for r in range(n):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(n), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), **(extra_env or {}))
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER % ROOT], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE))
    return [p.wait(timeout=120) for p in procs]


def test_gloo_processes_all_reduce():
    assert _launch(2, 29731) == [0, 0]


def test_rank_failure_is_a_clean_error_for_the_others():
    codes = _launch(3, 29741, {"FAIL_RANK": "1"})
    assert codes[1] == 3 and codes[0] == 4 and codes[2] == 4


def test_tcp_store_set_get_add_wait_barrier():
    import threading
    from nexus_b200.parallel.store import TcpStore
    server = TcpStore(port=0, is_server=True, world_size=3, timeout_s=5.0)
    clients = [server] + [TcpStore(port=server.port, world_size=3, timeout_s=5.0) for _ in range(2)]
    clients[1].set("a", b"hello")
    assert clients[2].get("a") == b"hello" and clients[0].check(["a"]) and not clients[0].check(["a", "zz"])
    assert [c.add("n", 2) for c in clients] == [2, 4, 6]
    got = []
    t = threading.Thread(target=lambda: got.append(clients[2].get("late", 5.0)))
    t.start()
    clients[0].set("late", b"x")
    t.join(5)
    assert got == [b"x"]
    with pytest.raises(TimeoutError):
        clients[1].get("never", 0.1)
    order = []
    ts = [threading.Thread(target=lambda i=i: (clients[i].barrier(), order.append(i))) for i in range(3)]
    for x in ts[:2]:
        x.start()
    import time
    time.sleep(0.1)
    assert order == []             # nobody passes before the third arrives
    ts[2].start()
    for x in ts:
        x.join(5)
    assert sorted(order) == [0, 1, 2]
    for c in clients[1:]:
        c.close()
    server.close()


def test_check_call_names_a_mismatched_fused_launch_on_thread_ranks():
    """The host-side guard that the symmetric-memory ops run before their kernels: ranks that are about to launch the
    same thing pass, a rank with a different size raises a named error on every rank, and the guard costs nothing when
    validate mode is off."""
    from nexus_b200.parallel.process_group import DistError, GroupOptions, run_threads

    def agree(pg):
        pg.check_call("gemm_ag", 4096, 1024, (2048, 1024), False)
        pg.check_call("fused_all_reduce", 1 << 20, "bf16", "f32")
        return "ok"
    assert run_threads(3, agree, GroupOptions(validate=True)) == ["ok"] * 3

    def differ(pg):
        try:
            pg.check_call("fused_all_reduce", 1024 if pg.rank() != 1 else 2048, "bf16")
        except DistError as e:
            return "mismatch" if "fused_all_reduce:1024" in str(e) and "fused_all_reduce:2048" in str(e) else str(e)
        return "passed"
    assert run_threads(2, differ, GroupOptions(validate=True)) == ["mismatch"] * 2

    def off(pg):
        pg.check_call("anything", pg.rank())          # validate off: no exchange, no error
        return pg._seq
    assert run_threads(2, off, GroupOptions(validate=False)) == [0, 0]
