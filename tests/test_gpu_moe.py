import pytest
import torch

pytestmark = pytest.mark.gpu


def test_moe_gpu_forward_backward_matches_reference():
    from nexus_b200.moe import gpu as G
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(0)
    N, d, F, E, k = 300, 128, 256, 8, 2
    cap = 64            # 600 assignments over 8 experts: some overflow and are dropped
    x = (torch.randn(N, d, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    router = (torch.randn(E, d, device="cuda") * 0.2).requires_grad_(True)
    up = (torch.randn(E, 2 * F, d, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    down = (torch.randn(E, d, F, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y, counts, dropped = G.moe_ffn(x, router, up, down, k, cap)
    dy = torch.randn_like(y)
    y.backward(dy)
    got = [t.grad.float().clone() for t in (x, router, up, down)]
    xr, rr, ur, dr = (t.detach().float().requires_grad_(True) for t in (x, router, up, down))
    yr, idx, gate, keep = G.reference(xr, rr, ur, dr, k, cap)
    yr.backward(dy.float())
    assert int(dropped) == int((~keep).sum()) and int(dropped) > 0
    assert int(counts.sum()) == int(keep.sum())
    assert (y.float() - yr).norm() / yr.norm() < 2e-2
    for g, r, name in zip(got, (xr, rr, ur, dr), ("dx", "drouter", "dup", "ddown")):
        rel = (g - r.grad).norm() / r.grad.norm()
        assert rel < 4e-2, (name, float(rel))
    K.check_status()


def test_moe_routing_kernels_priority_and_ties():
    from nexus_b200.moe import gpu as G
    logits = torch.zeros(10, 4, device="cuda")
    logits[:, 2] = 1.0          # everyone's first choice is expert 2; ties for the second go to expert 0
    expert, gate, slot, counts, dropped = G.route(logits, 2, 8)
    assert expert[:, 0].tolist() == [2] * 10 and expert[:, 1].tolist() == [0] * 10
    assert slot[:, 0].tolist() == [0, 1, 2, 3, 4, 5, 6, 7, -1, -1]
    assert counts.tolist() == [8, 0, 8, 0] and int(dropped) == 4
    assert torch.allclose(gate.sum(-1), torch.ones(10, device="cuda"))


@pytest.mark.parametrize("groups,overflow,noisy", [(2, "drop", False), (1, "reroute", False), (4, "reroute", True)])
def test_moe_gpu_groups_reroute_and_noisy_router_match_the_cpu_core(groups, overflow, noisy):
    """Capacity per token group, the Reroute overflow policy and the noisy top-k router on the GPU (one warp per group
    walks the assignments in (choice, token) order) against the FP32 CPU core `moe.moe_forward` on the same inputs:
    output rows, numbers of dropped and rerouted assignments, and the gradients of the inputs, the router and the noise
    projection."""
    from nexus_b200.moe import gpu as G
    from nexus_b200.moe import moe as M
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(3)
    N, d, E, k, Fd = 128 * max(groups, 2), 64, 8, 2, 64
    spec = M.Spec(experts=E, top_k=k, d_model=d, d_ff=Fd, capacity_factor=0.75, groups=groups, overflow=overflow,
                  noisy=noisy, min_capacity=8)
    cap = M.capacity_of(spec, N // groups)
    assert cap % 8 == 0
    # skewed router: a few experts overflow, so the policy matters
    x = torch.randn(N, d)
    router = torch.randn(E, d) * 0.5
    router[0] *= 3.0
    noise_w = torch.randn(E, d) * 0.3 if noisy else None
    up, down = torch.randn(E, 2 * Fd, d) * 0.1, torch.randn(E, d, Fd) * 0.1
    xb, ub, db = x.bfloat16(), up.bfloat16(), down.bfloat16()
    # CPU core in FP32 on the BF16-rounded operands
    xc = xb.float().requires_grad_(True)
    rc = router.t().contiguous().requires_grad_(True)
    nc = noise_w.t().contiguous().requires_grad_(True) if noisy else None
    yc, r = M.moe_forward(xc, rc, nc, ub.float(), db.float(), spec, training=True, seed=11)
    go = torch.randn(N, d)
    yc.backward(go)
    # GPU
    xg = xb.cuda().requires_grad_(True)
    rg = router.cuda().requires_grad_(True)
    ng = noise_w.cuda().requires_grad_(True) if noisy else None
    out = G.moe_ffn(xg, rg, ub.cuda(), db.cuda(), k, cap, groups=groups, overflow=overflow, noise_w=ng, noise_seed=11,
                    training=True)
    yg, counts, dropped = out[0], out[1], out[2]
    yg.backward(go.cuda().bfloat16())
    torch.cuda.synchronize()
    K.check_status()
    assert int(dropped) == r.dropped
    if len(out) > 3:
        assert int(out[3]) == r.rerouted
        assert int(counts.sum()) == N * k - r.dropped
    if overflow == "reroute":
        assert r.rerouted > 0
    assert (yg.float().cpu() - yc.detach()).abs().max() < 3e-2 * max(1.0, float(yc.detach().abs().max()))
    rel = lambda a, b: float((a - b).norm() / b.norm().clamp_min(1e-6))
    assert rel(xg.grad.float().cpu(), xc.grad) < 4e-2
    assert rel(rg.grad.float().cpu(), rc.grad.t()) < 4e-2
    if noisy:
        assert rel(ng.grad.float().cpu(), nc.grad.t()) < 6e-2
