import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fp8_quantize_dequantize_and_amax():
    from nexus_b200.ops import _lowp as L
    x = (torch.randn(4096, device="cuda") * 3).bfloat16()
    amax = torch.zeros(1, device="cuda")
    scale = torch.tensor([16.0], device="cuda")
    for dt in (torch.float8_e4m3fn, torch.float8_e5m2):
        q = L.fp8_quantize(x, dt, scale, amax)
        ref = (x.float() * 16).clamp(-torch.finfo(dt).max, torch.finfo(dt).max).to(dt)
        assert torch.equal(q.view(torch.uint8), ref.view(torch.uint8))
        back = L.fp8_dequantize(q, torch.tensor([1 / 16.0], device="cuda"), torch.float32)
        assert torch.allclose(back, ref.float() / 16)
    assert float(amax) == float(x.float().abs().max())
    m = torch.randn(37, 200, device="cuda")
    q, si = L.fp8_quantize_rows(m)
    assert torch.allclose(si, m.abs().amax(1) / 448, rtol=1e-6)
    assert ((q.float() * si[:, None]) - m).abs().max() < 0.07 * m.abs().max()


@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (300, 200, 384), (128, 128, 128)])
def test_fp8_gemm_exact_against_dequantised_reference(m, n, k):
    from nexus_b200.ops import _cuda as K
    from nexus_b200.ops import _lowp as L
    torch.manual_seed(0)
    a, b = torch.randn(m, k, device="cuda"), torch.randn(n, k, device="cuda") * 0.1
    aq, asi = L.fp8_quantize_rows(a)
    bq, bsi = L.fp8_quantize_rows(b)
    amax = torch.zeros(1, device="cuda")
    out = K.gemm(aq, bq, out_dtype=torch.float32, scale_a=asi, scale_b=bsi, amax_out=amax)
    ref = (aq.float() * asi[:, None]) @ (bq.float() * bsi[:, None]).t()
    assert (out - ref).abs().max() < 2e-3 * ref.abs().max()
    assert abs(float(amax) - float(out.abs().max())) < 1e-6
    assert (out - a @ b.t()).norm() / (a @ b.t()).norm() < 0.06
    # E5M2 gradients x E4M3 weights, bias + BF16 output
    gq = L.fp8_quantize(a.bfloat16(), torch.float8_e5m2)
    bias = torch.randn(n, device="cuda").bfloat16()
    o2 = K.gemm(gq, bq, bias=bias, scale_b=bsi)
    r2 = gq.float() @ (bq.float() * bsi[:, None]).t() + bias.float()
    assert (o2.float() - r2).abs().max() < 2e-2 * r2.abs().max()
    y = L.fp8_linear(a.bfloat16(), bq, bsi, bias=bias, act="gelu")
    ry = torch.nn.functional.gelu(a @ b.t() + bias.float(), approximate="tanh")
    assert (y.float() - ry).norm() / ry.norm() < 0.08
    K.check_status()


def test_adamw8_tracks_fp32_adamw_and_delayed_clip():
    from nexus_b200.ops import _cuda as K
    from nexus_b200.ops import _lowp as L
    torch.manual_seed(1)
    n = 5000
    target = torch.randn(n, device="cuda")
    p8 = torch.zeros(n, device="cuda")
    p32 = torch.zeros(n, device="cuda", requires_grad=True)
    sh = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    st8 = L.AdamW8bitState(n, "cuda")
    opt = torch.optim.AdamW([p32], lr=0.05, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.0)
    state = K.opt_state_tensor("cuda")
    clip = torch.ones(1, device="cuda")
    accum = torch.zeros(1, device="cuda", dtype=torch.float64)
    norm = torch.zeros(1, device="cuda")
    for step in range(1, 61):
        raw = K.pack_opt_state(lr=0.05, weight_decay=0.0, beta1=0.9, beta2=0.99, eps=1e-8, max_grad_norm=0.0,
                               loss_scale=1.0, step=step, inv_bias1=1 / (1 - 0.9 ** step), inv_bias2=1 / (1 - 0.99 ** step))
        state.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
        g8 = (p8 - target).contiguous()
        L.grad_sq_accumulate(g8, accum)
        L.adamw8(p8, sh, g8, st8, state, clip=clip, zero_grad=True)
        assert float(g8.abs().max()) == 0.0
        L.delayed_clip_finish(clip, accum, 1e9, norm)
        opt.zero_grad()
        ((p32 - target) ** 2).sum().mul(0.5).backward()
        opt.step()
    assert float(norm) > 0 and float(accum) == 0.0 and float(clip) == 1.0
    e8, e32 = (p8 - target).norm().item(), (p32.detach() - target).norm().item()
    assert e8 < 0.25 * target.norm().item() and abs(e8 - e32) < 0.1 * target.norm().item()
    assert torch.allclose(sh.float(), p8, atol=2e-2)
    assert st8.nbytes() < 0.3 * (8 * n)
    L.delayed_clip_finish(clip, accum.fill_(100.0), 1.0)
    assert abs(float(clip) - 0.1) < 1e-5


@pytest.mark.parametrize("rows,cols", [(130, 200), (256, 1024), (37, 48)])
def test_mx_quantize_matches_reference_bit_for_bit(rows, cols):
    from nexus_b200.ops import _lowp as L
    torch.manual_seed(2)
    x = (torch.randn(rows, cols, device="cuda") * torch.logspace(-3, 3, cols, device="cuda")).bfloat16()
    x[0, :32] = 0  # an all-zero block keeps the scale 1
    for dt in (torch.float8_e4m3fn, torch.float8_e5m2):
        for tr in (False, True):
            q, s = L.mx_quantize(x, dt, transpose=tr)
            rq, rs = L.mx_quantize_reference(x, dt, transpose=tr)
            assert torch.equal(q.view(torch.uint8), rq.view(torch.uint8))
            assert torch.equal(s, rs)
            want = x.t().float() if tr else x.float()
            back = L.mx_dequantize(q, s)
            assert torch.equal(back, L.mx_dequantize_reference(q, s))
            # no saturation: each value is within half a code step (2^-3 relative for E4M3, 2^-2 for E5M2) of its block max
            assert (back - want).abs().max() <= (0.07 if dt == torch.float8_e4m3fn else 0.13) * want.abs().max()


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 1024), (300, 200, 416), (1024, 640, 2048)])
def test_mx_gemm_exact_against_dequantised_reference(m, n, k):
    from nexus_b200.ops import _cuda as K
    from nexus_b200.ops import _lowp as L
    torch.manual_seed(3)
    # column magnitudes over four decades: per-tensor or per-row scales would lose the small columns
    a = torch.randn(m, k, device="cuda") * torch.logspace(-2, 2, k, device="cuda")
    b = torch.randn(n, k, device="cuda") * 0.1
    aq, asf = L.mx_quantize(a)
    bq, bsf = L.mx_quantize(b)
    ref = L.mx_dequantize_reference(aq, asf) @ L.mx_dequantize_reference(bq, bsf).t()
    amax = torch.zeros(1, device="cuda")
    out = L.mx_gemm(aq, asf, bq, bsf, out_dtype=torch.float32, amax_out=amax)
    assert (out - ref).abs().max() < 1e-5 * ref.abs().max()
    assert abs(float(amax) - float(out.abs().max())) < 1e-6 * float(amax)
    assert (out - a @ b.t()).norm() / (a @ b.t()).norm() < 0.05
    # E5M2 gradients x E4M3 weights, bias + GELU, BF16 output
    gq, gsf = L.mx_quantize(a, torch.float8_e5m2)
    bias = torch.randn(n, device="cuda").bfloat16()
    o2 = L.mx_gemm(gq, gsf, bq, bsf, bias=bias, act="gelu", alpha=0.01)
    r2 = torch.nn.functional.gelu(0.01 * (L.mx_dequantize_reference(gq, gsf) @ L.mx_dequantize_reference(bq, bsf).t())
                                  + bias.float(), approximate="tanh")
    assert (o2.float() - r2).abs().max() < 2e-2 * r2.abs().max()
    K.check_status()


def test_mx_gemm_block_scaled_output_feeds_the_next_gemm():
    from nexus_b200.ops import _cuda as K
    from nexus_b200.ops import _lowp as L
    torch.manual_seed(4)
    m, k, h, n = 200, 256, 320, 192
    x = torch.randn(m, k, device="cuda")
    w1 = torch.randn(h, k, device="cuda") * 0.05
    w2 = torch.randn(n, h, device="cuda") * 0.05
    xq, xs = L.mx_quantize(x)
    w1q, w1s = L.mx_quantize(w1)
    w2q, w2s = L.mx_quantize(w2)
    hid = L.mx_gemm(xq, xs, w1q, w1s, act="silu", out_dtype=torch.float32)
    hq, hs = L.mx_gemm(xq, xs, w1q, w1s, act="silu", out_dtype=torch.float8_e4m3fn)
    rq, rs = L.mx_quantize_reference(hid)
    # the epilogue quantiser is the stand-alone quantiser applied to the same FP32 values
    assert torch.equal(hs, rs)
    assert (hq.view(torch.uint8) != rq.view(torch.uint8)).float().mean() < 1e-3
    y = L.mx_gemm(hq, hs, w2q, w2s, out_dtype=torch.float32)
    ref = torch.nn.functional.silu(x @ w1.t()) @ w2.t()
    assert (y - ref).norm() / ref.norm() < 0.06
    K.check_status()


def test_mx_linear_gradients_close_to_fp32():
    from nexus_b200.ops import _cuda as K
    from nexus_b200.ops import _lowp as L
    torch.manual_seed(5)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    b = torch.zeros(384, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    t = torch.randn(4, 96, 384, device="cuda")
    ((L.mx_linear(x, w, b).float() - t) ** 2).mean().backward()
    x2, w2, b2 = (v.detach().float().requires_grad_() for v in (x, w, b))
    ((torch.nn.functional.linear(x2, w2, b2) - t) ** 2).mean().backward()
    for got, want in ((x.grad, x2.grad), (w.grad, w2.grad), (b.grad, b2.grad)):
        assert (got.float() - want).norm() / want.norm() < 0.08
    K.check_status()
