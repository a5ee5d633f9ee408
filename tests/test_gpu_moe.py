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
