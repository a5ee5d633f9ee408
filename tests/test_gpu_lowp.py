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
