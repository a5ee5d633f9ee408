"""Memory-bound sm_100a kernels vs FP32 PyTorch references: norms, embedding, shifted CE,
Philox dropout, gradient norm + AdamW, column sums."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(a, b, tol):
    return (a.float() - b.float()).abs().max().item() <= tol * max(b.float().abs().max().item(), 1e-6) + 1e-6


@pytest.mark.parametrize("rows,cols", [(64, 128), (1000, 768), (4096, 1600)])
def test_layernorm_fwd_bwd(rows, cols):
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(0)
    x, res = torch.randn(rows, cols, device=DEV), torch.randn(rows, cols, device=DEV)
    g, b = torch.randn(cols, device=DEV), torch.randn(cols, device=DEV)
    s_out = torch.empty_like(x)
    y, mean, rstd = K.norm_fwd(x, g, b, residual=res, sum_out=s_out, out_dtype=torch.bfloat16)
    xs = x + res
    assert close(y, torch.nn.functional.layer_norm(xs, (cols,), g, b, 1e-5), 1e-2)
    assert close(s_out, xs, 1e-6)
    dy, add = torch.randn(rows, cols, device=DEV).bfloat16(), torch.randn(rows, cols, device=DEV)
    dg, db = torch.zeros(cols, device=DEV), torch.zeros(cols, device=DEV)
    lp = torch.empty(rows, cols, device=DEV, dtype=torch.bfloat16)
    dx = K.norm_bwd(dy, xs, g, mean, rstd, add=add, dx_dtype=torch.float32, dgamma=dg, dbeta=db, dx_lp=lp)
    xs2, g2, b2 = xs.clone().requires_grad_(True), g.clone().requires_grad_(True), b.clone().requires_grad_(True)
    torch.nn.functional.layer_norm(xs2, (cols,), g2, b2, 1e-5).backward(dy.float())
    assert close(dx, xs2.grad + add, 1e-4)
    assert close(lp, xs2.grad + add, 1e-2)
    assert close(dg, g2.grad, 1e-3) and close(db, b2.grad, 1e-3)
    # the same pass can also return the column sums of the BF16 dx (a bias gradient), accumulated like dgamma
    dg2, db2 = torch.zeros(cols, device=DEV), torch.zeros(cols, device=DEV)
    cs = torch.ones(cols, device=DEV)
    lp2 = torch.empty_like(lp)
    dx2 = K.norm_bwd(dy, xs, g, mean, rstd, add=add, dx_dtype=torch.float32, dgamma=dg2, dbeta=db2, dx_lp=lp2,
                     dx_colsum=cs, accumulate_params=True)
    assert torch.equal(dx2, dx) and torch.equal(lp2, lp) and close(dg2, dg, 1e-6)
    assert close(cs, 1.0 + lp.float().sum(0), 1e-4)


@pytest.mark.parametrize("rows,cols", [(1000, 768), (512, 4096)])
def test_rmsnorm_fwd_bwd(rows, cols):
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(0)
    x, g = torch.randn(rows, cols, device=DEV), torch.randn(cols, device=DEV)
    y, _, rstd = K.norm_fwd(x, g, None, rms=True, eps=1e-5, out_dtype=torch.float32)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * g
    assert close(y, ref, 1e-5)
    dy, dg = torch.randn(rows, cols, device=DEV), torch.zeros(cols, device=DEV)
    dx = K.norm_bwd(dy, x, g, None, rstd, rms=True, dx_dtype=torch.float32, dgamma=dg)
    x2, g2 = x.clone().requires_grad_(True), g.clone().requires_grad_(True)
    (x2 * torch.rsqrt(x2.pow(2).mean(-1, keepdim=True) + 1e-5) * g2).backward(dy)
    assert close(dx, x2.grad, 1e-4) and close(dg, g2.grad, 1e-3)


@pytest.mark.parametrize("deterministic", (True, False))
def test_embedding(deterministic):
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(0)
    B, T, C, V = 4, 64, 128, 1000
    tok = torch.randint(0, V, (B, T), device=DEV, dtype=torch.int32)
    wte, wpe = torch.randn(V, C, device=DEV), torch.randn(T, C, device=DEV)
    assert close(K.embedding_pos_fwd(tok, wte, wpe), wte[tok.long()] + wpe[None], 1e-6)
    dx = torch.randn(B, T, C, device=DEV)
    dwte, dwpe = torch.zeros_like(wte), torch.zeros_like(wpe)
    K.embedding_bwd(tok, dx, dwte, dwpe, B, T, deterministic=deterministic)
    ref = torch.zeros_like(wte)
    ref.index_add_(0, tok.reshape(-1).long(), dx.reshape(-1, C))
    assert close(dwte, ref, 1e-5) and close(dwpe, dx.sum(0), 1e-5)


@pytest.mark.parametrize("dtype,ld", [(torch.float32, 1024), (torch.bfloat16, 1024), (torch.float32, 1001)])
def test_cross_entropy_shifted(dtype, ld):
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(0)
    B, T, V = 3, 33, 1000
    tok = torch.randint(0, V, (B, T), device=DEV, dtype=torch.int32)
    logits = torch.zeros(B * T, ld, device=DEV, dtype=dtype)
    logits[:, :V] = (torch.randn(B * T, V, device=DEV) * 3).to(dtype)
    ref_in = logits[:, :V].float().clone().requires_grad_(True)
    tg = torch.full((B, T), -100, device=DEV, dtype=torch.long)
    tg[:, :-1] = tok[:, 1:].long()
    sm, z = 0.1, 1e-3
    lse = torch.logsumexp(ref_in, -1)
    valid = tg.reshape(-1) != -100
    nll = lse - ref_in.gather(1, tg.reshape(-1).clamp(min=0)[:, None])[:, 0]
    lossr = ((1 - sm) * nll + sm * (lse - ref_in.mean(-1)) + z * lse * lse)[valid].sum() / valid.sum()
    (lossr * 0.5).backward()
    loss = K.cross_entropy_shifted(logits, tok, vocab=V, smoothing=sm, z_loss=z, grad_scale=0.5)
    bf = dtype == torch.bfloat16
    assert close(loss, lossr.detach().reshape(1), 1e-3 if bf else 1e-5)
    assert close(logits[:, :V], ref_in.grad, 2e-2 if bf else 1e-4)
    assert float(logits[:, V:].float().abs().max()) == 0.0 if ld > V else True


def test_dropout_philox():
    from nexus_b200.ops import _cuda as K
    from nexus_b200.fused.philox import philox_uniform as cpu_uniform
    x = torch.ones(1 << 20, device=DEV)
    y1, y2 = K.dropout(x, 0.25, 1234, 7), K.dropout(x, 0.25, 1234, 7)
    assert torch.equal(y1, y2)
    assert abs((y1 != 0).float().mean().item() - 0.75) < 5e-3
    u = K.philox_uniform(64, 42, 3).cpu()
    assert torch.equal(u, torch.from_numpy(cpu_uniform(64, 42, 3)))


def test_adamw_and_grad_norm():
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(0)
    n = 200000
    master, grad = torch.randn(n, device=DEV), torch.randn(n, device=DEV) * 3
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    shadow = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    st = K.opt_state_tensor(DEV)
    st.copy_(torch.frombuffer(bytearray(K.pack_opt_state(lr=1e-2, weight_decay=0.1, beta1=0.9, beta2=0.95, eps=1e-8,
                                                         max_grad_norm=1.0, loss_scale=1.0)), dtype=torch.uint8))
    chunks = K.make_chunks([(0, 100000, 1.0, 1.0), (100000, 100000, 0.0, 1.0)], device=DEV)
    p0 = master.clone()
    K.grad_norm(grad, st)
    K.adamw(master, grad, m, v, shadow, chunks, st)
    s = K.unpack_opt_state(bytes(st.cpu().numpy().tobytes()))
    gn = grad.double().norm().item()
    assert abs(s.grad_norm - gn) / gn < 1e-5 and s.step == 1 and s.found_inf == 0
    g = grad * s.clip_coef
    pr = p0.clone()
    pr[:100000] -= 1e-2 * 0.1 * pr[:100000]
    mr, vr = 0.1 * g, 0.05 * g * g
    pr -= 1e-2 * (mr / (1 - 0.9)) / ((vr / (1 - 0.95)).sqrt() + 1e-8)
    assert close(master, pr, 1e-5) and close(shadow, pr, 1e-2)
    # non-finite gradients skip the update
    grad[5] = float("nan")
    before = master.clone()
    K.grad_norm(grad, st)
    K.adamw(master, grad, m, v, shadow, chunks, st)
    s = K.unpack_opt_state(bytes(st.cpu().numpy().tobytes()))
    assert s.found_inf == 1 and s.step == 1 and torch.equal(before, master)


def test_colsum_and_nonfinite():
    from nexus_b200.ops import _cuda as K
    dy = torch.randn(1000, 304, device=DEV).bfloat16()
    assert close(K.colsum(dy), dy.float().sum(0), 1e-4)
    dy = torch.randn(777, 300, device=DEV)
    assert close(K.colsum(dy), dy.sum(0), 1e-5)
    assert K.count_nonfinite(torch.tensor([1.0, float("nan"), float("inf")], device=DEV)).item() == 2


@pytest.mark.parametrize("kind", ["swiglu", "geglu"])
def test_gated_activation_autograd_matches_fp32_formula(kind):
    from nexus_b200.fused import ops as F_
    torch.manual_seed(11)
    h = torch.randn(3, 70, 2 * 96, device="cuda").bfloat16().requires_grad_()
    t = torch.randn(3, 70, 96, device="cuda")
    y = F_.gated_activation(h, kind)
    (y.float() * t).sum().backward()
    h2 = h.detach().float().requires_grad_()
    a, b = h2[..., :96], h2[..., 96:]
    ref = (torch.nn.functional.silu(a) if kind == "swiglu" else torch.nn.functional.gelu(a, approximate="tanh")) * b
    (ref * t).sum().backward()
    assert (y.float() - ref).abs().max() < 2e-2 * ref.abs().max()
    assert (h.grad.float() - h2.grad).abs().max() < 2e-2 * h2.grad.abs().max()


def test_dlpack_exchange_on_the_device_and_pinned_host():
    """The native DLPack producer / consumer on CUDA memory and pinned host memory: zero copy in both directions."""
    from nexus_b200.interop import dlpack
    t = torch.arange(24, dtype=torch.float32, device="cuda").reshape(4, 6)
    assert dlpack.device_type(t) == dlpack.K_CUDA
    u = torch.from_dlpack(dlpack.to_dlpack(t))
    assert u.is_cuda and u.data_ptr() == t.data_ptr()
    v = dlpack.from_dlpack(torch.utils.dlpack.to_dlpack(t))
    v[0, 0] = 5.0
    assert v.is_cuda and v.device == t.device and float(t[0, 0]) == 5.0
    w = dlpack.from_dlpack(dlpack.to_dlpack(t.t()))
    assert tuple(w.shape) == (6, 4) and torch.equal(w, t.t())
    h = torch.ones(8, dtype=torch.float32).pin_memory()
    assert dlpack.device_type(h) == dlpack.K_CUDA_HOST
    g = dlpack.from_dlpack(dlpack.to_dlpack(h))
    g[3] = 2.0
    assert float(h[3]) == 2.0 and not g.is_cuda
