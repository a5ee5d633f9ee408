import pytest
import torch

from nexus_b200.moe import MoEFFN, Spec, reference, route
from nexus_b200.moe.moe import capacity_of, dequantize_experts, quantize_experts


def test_matches_fp64_oracle_and_has_router_gradients():
    torch.manual_seed(0)
    s = Spec(experts=4, top_k=2, d_model=16, d_ff=8, capacity_factor=1.0, min_capacity=1)
    m = MoEFFN(s)
    x = torch.randn(32, 16)
    y = m(x)
    yr, aux, z = reference(x, m.router.detach(), m.up.detach(), m.down.detach(), s)
    assert (y.double() - yr).abs().max() < 1e-6
    assert float(m.last_routing.aux) == pytest.approx(aux, rel=1e-6) and float(m.last_routing.z) == pytest.approx(z, rel=1e-6)
    (y.sum() + m.losses()).backward()
    assert m.router.grad.abs().sum() > 0 and m.up.grad.abs().sum() > 0


def test_capacity_priority_drop_and_reroute():
    assert capacity_of(Spec(experts=8, top_k=2, d_model=1, d_ff=1, capacity_factor=1.25, min_capacity=4), 64) == 20
    torch.manual_seed(1)
    x = torch.randn(16, 8)
    w = torch.zeros(8, 4)
    w[:, 0] = 5.0                     # every token prefers expert 0
    s = Spec(experts=4, top_k=1, d_model=8, d_ff=4, capacity_factor=1.0, min_capacity=1)
    r = route(x.abs(), w, None, s)
    assert r.capacity == 4 and r.dropped == 12
    assert (r.row[:4, 0] >= 0).all() and (r.row[4:, 0] < 0).all()     # earliest tokens win
    s2 = Spec(experts=4, top_k=1, d_model=8, d_ff=4, capacity_factor=1.0, min_capacity=1, overflow="reroute")
    r2 = route(x.abs(), w, None, s2)
    assert r2.dropped == 0 and r2.rerouted == 12
    counts = (r2.offsets[1:] - r2.offsets[:-1]).tolist()
    assert counts == [4, 4, 4, 4]
    with pytest.raises(ValueError):
        route(x[:15], w, None, Spec(experts=4, top_k=1, d_model=8, d_ff=4, groups=2))


def test_groups_and_gate_normalisation():
    torch.manual_seed(2)
    s = Spec(experts=4, top_k=2, d_model=8, d_ff=4, groups=2, capacity_factor=2.0)
    r = route(torch.randn(16, 8), torch.randn(8, 4), None, s)
    assert torch.allclose(r.gate.sum(-1), torch.ones(16))
    assert int(r.offsets[-1]) == int((r.row >= 0).sum())


def test_expert_quantisation():
    w = torch.randn(4, 8, 16)
    q, sc = quantize_experts(w, "fp8")
    assert (dequantize_experts(q, sc) - w).abs().max() < 0.07 * w.abs().max()
    q, sc = quantize_experts(w, "bf16")
    assert sc is None and (q.float() - w).abs().max() < 0.01 * w.abs().max()


def test_block_scaled_expert_storage_round_trip():
    """'mxfp8' expert storage: E4M3 codes with a power-of-two scale per 32 elements of each row; a column range that a
    per-expert scale would flush to zero survives."""
    from nexus_b200.moe.moe import dequantize_experts, quantize_experts
    torch.manual_seed(0)
    w = torch.randn(3, 40, 64) * 0.02
    w[:, :, :32] *= 1e-6                                   # tiny columns next to ordinary ones
    q, s = quantize_experts(w, "mxfp8")
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.uint8 and s.shape[0] == 3
    back = dequantize_experts(q, s)
    small = (back[:, :, :32] - w[:, :, :32]).norm() / w[:, :, :32].norm()
    assert small < 0.05
    q1, s1 = quantize_experts(w, "fp8")
    coarse = (dequantize_experts(q1, s1)[:, :, :32] - w[:, :, :32]).norm() / w[:, :, :32].norm()
    assert coarse > 0.5                                    # per-expert scaling loses those columns


@pytest.mark.parametrize("groups,overflow", [(1, "drop"), (2, "drop"), (1, "reroute"), (4, "reroute")])
def test_tensor_core_agrees_with_the_native_fp64_oracle_under_every_policy(groups, overflow):
    """The native FP64 oracle (its own router, top-k, capacity walk and expert MLPs) against the tensor implementation
    under tight capacities: outputs, losses, dropped and rerouted counts, with token groups and both overflow policies."""
    from nexus_b200.moe.moe import moe_forward, reference_full
    torch.manual_seed(5)
    s = Spec(experts=8, top_k=2, d_model=16, d_ff=8, capacity_factor=0.6, min_capacity=1, groups=groups, overflow=overflow)
    x = torch.randn(64, 16)
    router = torch.randn(16, 8)
    router[:, 1] *= 3.0
    up, down = torch.randn(8, 16, 16) * 0.3, torch.randn(8, 16, 8) * 0.3
    y, r = moe_forward(x, router, None, up, down, s)
    yr, aux, z, dropped, rerouted = reference_full(x, router, up, down, s)
    assert dropped == r.dropped and rerouted == r.rerouted and dropped + (rerouted if overflow == "reroute" else 0) > 0
    assert (y.double() - yr).abs().max() < 1e-5
    assert float(r.aux) == pytest.approx(aux, rel=1e-6) and float(r.z) == pytest.approx(z, rel=1e-6)


def _assign_oracle(expert, order, E, groups, C, reroute):
    """Plain-Python statement of the assignment rules, kept here as the oracle for the native walk."""
    N, k = len(expert), len(expert[0])
    Ng = N // groups
    ex = [list(r) for r in expert]
    lists = [[[] for _ in range(groups)] for _ in range(E)]
    dropped = rerouted = 0
    for g in range(groups):
        fill = [0] * E
        for j in range(k):
            for t in range(g * Ng, (g + 1) * Ng):
                e = ex[t][j]
                if fill[e] >= C:
                    alt = -1
                    if reroute:
                        for e2 in order[t]:
                            if e2 not in ex[t] and fill[e2] < C:
                                alt = e2
                                break
                    if alt < 0:
                        dropped += 1
                        continue
                    rerouted += 1
                    ex[t][j] = e = alt
                fill[e] += 1
                lists[e][g].append(t * k + j)
    row, offs, perm = [-1] * (N * k), [0], []
    for e in range(E):
        for l in lists[e]:
            for slot in l:
                row[slot] = len(perm)
                perm.append(slot // k)
        offs.append(len(perm))
    return ex, row, offs, perm, dropped, rerouted


@pytest.mark.parametrize("reroute", [False, True])
def test_native_capacity_assignment_matches_the_rules(reroute):
    import numpy as np
    from nexus_b200 import _native
    rng = np.random.default_rng(5)
    for N, E, k, groups, C in [(32, 4, 2, 1, 6), (48, 8, 2, 4, 2), (40, 5, 3, 2, 9), (16, 4, 1, 2, 1), (24, 6, 2, 3, 0), (8, 3, 3, 1, 50)]:
        scores = rng.standard_normal((N, E)) + np.linspace(0, 1.5, E)        # skewed, so that experts overflow
        order = np.argsort(-scores, axis=1, kind="stable")
        expert = order[:, :k].copy()
        got = _native.moe_assign(expert, order if reroute else np.zeros((0, 0), dtype=np.int64), E, groups, C, reroute)
        want = _assign_oracle(expert.tolist(), order.tolist(), E, groups, C, reroute)
        assert got[0].tolist() == want[0] and got[1].reshape(-1).tolist() == want[1]
        assert got[2].tolist() == want[2] and got[3].tolist() == want[3] and (got[4], got[5]) == (want[4], want[5])
        assert got[4] + int((got[1] >= 0).sum()) == N * k
        if C * groups * E < N * k:
            assert got[4] > 0
    with pytest.raises(ValueError):
        _native.moe_assign(np.zeros((10, 2), dtype=np.int64), np.zeros((0, 0), dtype=np.int64), 4, 3, 2, False)
    with pytest.raises(IndexError):
        _native.moe_assign(np.full((4, 1), 9, dtype=np.int64), np.zeros((0, 0), dtype=np.int64), 4, 1, 2, False)
    with pytest.raises(ValueError):
        _native.moe_assign(np.zeros((4, 1), dtype=np.int64), np.zeros((4, 3), dtype=np.int64), 4, 1, 2, True)
