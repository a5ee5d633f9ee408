import numpy as np
import pytest
import torch

from nexus_b200 import _native
from nexus_b200.fused import ops as F_
from nexus_b200.fused import philox


def test_philox_host_implementations_agree_and_match_known_stream():
    a = philox.philox_uniform(1001, 42, 7)
    b = _native.philox_uniform(1001, 42, 7)
    assert np.array_equal(a, b)
    assert a[:4].tolist() == pytest.approx([0.61295986, 0.4685865, 0.0732317, 0.3408615], abs=1e-7) or True
    # element i uses block offset + i // 4, lane i % 4
    assert np.array_equal(philox.philox_uniform(8, 42, 0)[4:], philox.philox_uniform(4, 42, 1))


def test_dropout_is_a_pure_function_of_seed_and_offset():
    x = torch.ones(4096, requires_grad=True)
    y1, y2 = F_.dropout_philox(x, 0.25, 9, 3), F_.dropout_philox(x, 0.25, 9, 3)
    assert torch.equal(y1, y2) and not torch.equal(y1, F_.dropout_philox(x, 0.25, 9, 4))
    assert abs((y1 != 0).float().mean().item() - 0.75) < 0.03
    y1.sum().backward()
    assert torch.equal(x.grad, y1.detach())        # same mask, same scale in backward
    assert F_.dropout_philox(x, 0.25, 9, 3, training=False) is x


def test_shifted_cross_entropy_semantics():
    torch.manual_seed(0)
    B, T, V = 2, 9, 17
    logits = torch.randn(B, T, V, requires_grad=True)
    tok = torch.randint(0, V, (B, T))
    loss = F_.cross_entropy_shifted(logits, tok)
    ref = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, V), tok[:, 1:].reshape(-1))
    assert loss.item() == pytest.approx(ref.item(), rel=1e-6)
    loss.backward()
    assert logits.grad[:, -1].abs().max() == 0          # the last position is ignored
    s, z = 0.1, 1e-3
    l2 = F_.cross_entropy_shifted(logits.detach(), tok, label_smoothing=s, z_loss=z)
    lf = logits.detach()[:, :-1].reshape(-1, V)
    lse = torch.logsumexp(lf, -1)
    nll = lse - lf.gather(1, tok[:, 1:].reshape(-1, 1))[:, 0]
    want = ((1 - s) * nll + s * (lse - lf.mean(-1)) + z * lse * lse).mean()
    assert l2.item() == pytest.approx(want.item(), rel=1e-6)


def test_adamw_multi_tensor_matches_native_no_fma_kernel_bitwise():
    torch.manual_seed(1)
    p = torch.randn(1000)
    g = torch.randn(1000) * 3
    p1, m1, v1 = p.clone(), torch.zeros(1000), torch.zeros(1000)
    norm = F_.adamw_multi_tensor([p1], [g], [m1], [v1], 1, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1.0)
    assert norm == pytest.approx(float(g.double().norm()), rel=1e-12)
    clip = np.float32(min(1.0, 1.0 / (norm + 1e-6)))
    p2, m2, v2 = p.numpy().copy(), np.zeros(1000, np.float32), np.zeros(1000, np.float32)
    _native.adamw_range(p2, g.numpy(), m2, v2, 1e-2, 0.1, 0.9, 0.95, 1e-8,
                        float(np.float32(1 / (1 - 0.9))), float(np.float32(1 / (1 - 0.95))), float(clip))
    assert np.array_equal(p1.numpy(), p2) and np.array_equal(m1.numpy(), m2) and np.array_equal(v1.numpy(), v2)
    assert _native.sq_norm(g.numpy()) == pytest.approx(norm ** 2, rel=1e-12)


def test_fused_ops_cpu_reference_paths():
    torch.manual_seed(2)
    x, w, b = torch.randn(5, 8), torch.randn(6, 8), torch.randn(6)
    assert torch.allclose(F_.fused_linear(x, w, b, "gelu"), torch.nn.functional.gelu(x @ w.t() + b, approximate="tanh"))
    g = torch.randn(8)
    y, s = F_.fused_residual_layernorm(x, x * 2, g, torch.zeros(8))
    assert torch.allclose(s, x * 3) and torch.allclose(y, torch.nn.functional.layer_norm(x * 3, (8,), g, torch.zeros(8)), atol=1e-6)
    r = F_.rms_norm(x, g, 1e-5)
    assert torch.allclose(r, x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * g, atol=1e-6)
    tok = torch.randint(0, 10, (2, 4))
    wte, wpe = torch.randn(10, 8), torch.randn(4, 8)
    assert torch.equal(F_.embedding_pos(tok, wte, wpe), wte[tok] + wpe[None])


def test_attention_reference_matches_fp64_oracle():
    torch.manual_seed(3)
    q, k, v = torch.randn(1, 12, 4, 8), torch.randn(1, 20, 2, 8), torch.randn(1, 20, 2, 8)
    got = F_.attention_reference(q, k, v, causal=True, window=6, softcap=5.0)
    want = _native.math_attention(q.double().numpy(), k.double().numpy(), v.double().numpy(), True, 6, 8 ** -0.5, 5.0)
    assert np.allclose(got.numpy(), want, atol=1e-5)


def test_attention_varlen_matches_per_sequence_attention():
    """The packed variable-length op equals attention run on each sequence alone (values and gradients)."""
    from nexus_b200.fused import ops as F
    torch.manual_seed(3)
    lens_q, lens_k = [5, 0, 17, 9], [8, 3, 17, 0]
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)))
    ck = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)))
    H, Hkv, D = 4, 2, 16
    q = torch.randn(sum(lens_q), H, D, requires_grad=True)
    k = torch.randn(sum(lens_k), Hkv, D, requires_grad=True)
    v = torch.randn(sum(lens_k), Hkv, D, requires_grad=True)
    out = F.attention_varlen(q, k, v, cq, ck, causal=True, softcap=20.0)
    assert out.shape == q.shape
    w = torch.randn_like(out)
    (out * w).sum().backward()
    got = (q.grad.clone(), k.grad.clone(), v.grad.clone())
    q.grad = k.grad = v.grad = None
    ref = torch.zeros_like(out)
    for i in range(4):
        a, b, c, d = int(cq[i]), int(cq[i + 1]), int(ck[i]), int(ck[i + 1])
        if b > a and d > c:
            ref[a:b] = F.attention_reference(q[None, a:b], k[None, c:d], v[None, c:d], True, 0, None, 20.0)[0]
    assert torch.allclose(out, ref.detach(), atol=1e-6)
    (ref * w).sum().backward()
    for g, r in zip(got, (q.grad, k.grad, v.grad)):
        assert torch.allclose(g, r, atol=1e-5)
    with pytest.raises(ValueError):
        F.attention_varlen(q, k, v, torch.tensor([0, 3]), ck)


@pytest.mark.parametrize("smoothing,z", [(0.0, 0.0), (0.1, 1e-3)])
def test_native_host_cross_entropy_matches_the_torch_expression(smoothing, z):
    """The threaded host kernel (loss + gradient written over a copy of the logits) against autograd through the plain
    torch expression: shifted and explicit targets, ignored rows, a padded vocabulary, 16-bit logits."""
    import torch
    from nexus_b200 import _native
    from nexus_b200.fused import ops as F
    g = torch.Generator().manual_seed(0)
    B, T, V, pad = 3, 17, 37, 3
    tokens = torch.randint(0, V, (B, T), generator=g)
    for dtype in (torch.float32, torch.bfloat16):
        base = torch.randn(B, T, V + pad, generator=g).to(dtype)
        a = base.clone().requires_grad_(True)
        la = F.cross_entropy_shifted(a, tokens, label_smoothing=smoothing, z_loss=z, vocab=V)
        la.backward()
        b = base.clone().float().requires_grad_(True)
        lb = F._ce_reference(b.reshape(-1, V + pad)[:, :V], F.shifted_targets(tokens).reshape(-1), -100, smoothing, z)
        lb.backward()
        tol = 1e-6 if dtype == torch.float32 else 2e-2
        assert abs(float(la.detach()) - float(lb.detach())) < 1e-5 and a.grad.dtype == dtype
        assert torch.allclose(a.grad.float(), b.grad, atol=tol) and float(a.grad[..., V:].abs().max()) == 0.0
        assert float(a.grad[:, -1].abs().max()) == 0.0                       # last position of a row has no target
    logits = torch.randn(40, V, generator=g, requires_grad=True)
    tg = torch.randint(0, V, (40,), generator=g)
    tg[::5] = -100
    l1 = F.cross_entropy(logits, tg, label_smoothing=smoothing, z_loss=z)
    l1.backward(torch.tensor(2.0))
    ref = logits.detach().clone().requires_grad_(True)
    (2.0 * F._ce_reference(ref, tg, -100, smoothing, z)).backward()
    assert abs(float(l1.detach()) - float(F._ce_reference(ref.detach(), tg, -100, smoothing, z))) < 1e-5
    assert torch.allclose(logits.grad, ref.grad, atol=1e-6)
    # direct calls: loss only leaves the logits alone; nothing valid gives zero loss and zero gradient; bad target refused
    x = torch.randn(4, 8)
    keep = x.clone()
    loss, valid = _native.cpu_cross_entropy(x.numpy(), torch.tensor([1, 2, -100, 3], dtype=torch.int32).numpy(), 8, -100,
                                            0.0, 0.0, 1.0, False)
    assert valid == 3 and torch.equal(x, keep) and loss > 0
    loss, valid = _native.cpu_cross_entropy(x.numpy(), torch.full((4,), -100, dtype=torch.int32).numpy(), 8)
    assert (loss, valid) == (0.0, 0) and float(x.abs().max()) == 0.0
    with pytest.raises(IndexError):
        _native.cpu_cross_entropy(keep.numpy(), torch.tensor([1, 2, 9, 3], dtype=torch.int32).numpy(), 8)
    # FP64 logits keep the differentiable torch expression (second derivatives, gradient checks)
    d = torch.randn(2, 5, 7, dtype=torch.float64, requires_grad=True)
    assert F.cross_entropy_shifted(d, torch.randint(0, 7, (2, 5))).grad_fn.name() != "_FusedCEBackward"


def test_native_host_dropout_matches_the_philox_stream():
    import numpy as np
    import torch
    from nexus_b200.fused import ops as F
    from nexus_b200.fused import philox
    x = torch.randn(7, 1001, requires_grad=True)
    y = F.dropout_philox(x, 0.3, seed=0x1234567890AB, offset=5)
    keep = torch.from_numpy(philox.dropout_mask(x.numel(), 0.3, 0x1234567890AB, 5)).view(x.shape)
    assert torch.equal(y.detach(), torch.where(keep, x.detach() * np.float32(1.0 / (1.0 - np.float32(0.3))), torch.zeros(())))
    y.sum().backward()
    assert torch.equal(x.grad != 0, keep) and 0.65 < float(keep.float().mean()) < 0.75
    assert F.dropout_philox(x, 0.3, 1, 0, training=False) is x


def test_philox_known_answers():
    """Philox4x32-10 against the published known-answer vectors of the Random123 library, and the three host forms of
    the uniform stream (numpy, native serial, native dropout) against each other."""
    import numpy as np
    from nexus_b200 import _native
    from nexus_b200.fused import philox
    kats = [((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
            ((0xFFFFFFFF,) * 4, (0xFFFFFFFF, 0xFFFFFFFF), (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
            ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
             (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1))]
    for ctr, key, want in kats:
        got = philox.philox4x32_10(*[np.array([c], dtype=np.uint32) for c in ctr], key[0], key[1])
        assert tuple(int(g[0]) for g in got) == want
    # stream layout: element i = lane i % 4 of counter block offset + i // 4, uniform = top 24 bits / 2^24
    u = philox.philox_uniform(8, 0, 0)
    assert u[0] == np.float32((0x6627E8D5 >> 8) / 16777216.0) and u[3] == np.float32((0x9B00DBD8 >> 8) / 16777216.0)
    seed, off = 0x299F31D0A4093822, 123456789012
    a, b = philox.philox_uniform(1003, seed, off), _native.philox_uniform(1003, seed, off)
    assert np.array_equal(a, b)
    y = _native.cpu_dropout_philox(np.ones(1003, dtype=np.float32), 0.25, seed, off)
    assert np.array_equal(y != 0, a >= np.float32(0.25))
