"""tcgen05 flash attention forward/backward vs an FP32 PyTorch reference (causal, window, GQA,
Tq != Tk, packed QKV, head_dim 64 and 128, ragged lengths)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, causal, window, scale):
    B, Tq, H, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    qf, kf, vf = [t.permute(0, 2, 1, 3) for t in (q, k, v)]
    if Hkv != H:
        kf = kf.repeat_interleave(H // Hkv, 1)
        vf = vf.repeat_interleave(H // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    qi = torch.arange(Tq, device=q.device)[:, None] + (Tk - Tq)
    ki = torch.arange(Tk, device=q.device)[None]
    mask = torch.zeros(Tq, Tk, dtype=torch.bool, device=q.device)
    if causal:
        mask |= ki > qi
    if window > 0:
        mask |= ki < qi - window + 1
    s = s.masked_fill(mask, float("-inf"))
    return (torch.softmax(s, -1) @ vf).permute(0, 2, 1, 3), torch.logsumexp(s, -1)


CASES = [
    (1, 128, 128, 1, 1, 64, False, 0, False),
    (2, 256, 256, 3, 3, 64, True, 0, False),
    (2, 1024, 1024, 4, 4, 64, True, 0, True),
    (1, 200, 200, 2, 2, 64, True, 0, False),
    (1, 100, 300, 4, 2, 64, True, 0, False),
    (1, 512, 512, 2, 2, 64, True, 100, False),
    (1, 256, 256, 2, 1, 128, True, 0, False),
    (1, 384, 384, 2, 2, 128, False, 0, False),
    # head_dim 128 runs the two-q-tile forward: several 256-row items per head, ragged ends, window, Tq != Tk
    (2, 1024, 1024, 3, 3, 128, True, 0, True),
    (1, 700, 700, 2, 1, 128, True, 0, False),
    (1, 640, 640, 2, 2, 128, True, 200, False),
    (1, 300, 900, 4, 2, 128, True, 0, False),
]


@pytest.mark.parametrize("B,Tq,Tk,H,Hkv,D,causal,window,packed", CASES)
def test_attention_fwd_bwd(B, Tq, Tk, H, Hkv, D, causal, window, packed):
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(0)
    dev = "cuda"
    if packed:
        qkv = torch.randn(B, Tq, 3, H, D, device=dev).bfloat16()
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    else:
        q = torch.randn(B, Tq, H, D, device=dev).bfloat16()
        k = torch.randn(B, Tk, Hkv, D, device=dev).bfloat16()
        v = torch.randn(B, Tk, Hkv, D, device=dev).bfloat16()
    o, lse = K.attention_fwd(q, k, v, causal=causal, window=window)
    K.check_status()
    qr, kr, vr = [t.float().detach().requires_grad_(True) for t in (q, k, v)]
    oref, lref = _ref(qr, kr, vr, causal, window, D ** -0.5)
    assert (o.float() - oref).abs().max() < 2e-2
    assert (lse - lref).abs().max() < 2e-2
    do = torch.randn_like(o)
    dq, dk, dv = K.attention_bwd(q, k, v, o, lse, do, causal=causal, window=window)
    K.check_status()
    oref.backward(do.float())
    for got, want in ((dq, qr.grad), (dk, kr.grad), (dv, vr.grad)):
        assert (got.float() - want).abs().max() <= 3e-2 * want.abs().max()


@pytest.mark.parametrize("softcap,alibi,causal,window,Tq,Tk,H,Hkv,D", [
    (30.0, False, True, 0, 384, 384, 4, 4, 64),
    (0.0, True, True, 0, 384, 384, 4, 2, 64),
    (20.0, True, True, 100, 300, 300, 2, 2, 64),
    (15.0, True, False, 0, 200, 328, 2, 2, 128),
])
def test_attention_softcap_alibi(softcap, alibi, causal, window, Tq, Tk, H, Hkv, D):
    """Soft-capping and ALiBi inside the tensor-core kernels (forward and both backward kernels) against autograd
    through the FP32 math reference, and through the public fused op."""
    from nexus_b200.fused import ops as F
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(1)
    dev = "cuda"
    q = (torch.randn(2, Tq, H, D, device=dev) * 1.5).bfloat16()
    k = (torch.randn(2, Tk, Hkv, D, device=dev) * 1.5).bfloat16()
    v = torch.randn(2, Tk, Hkv, D, device=dev).bfloat16()
    slopes = (2.0 ** (-torch.arange(1, H + 1, device=dev, dtype=torch.float32))) if alibi else None
    qr, kr, vr = [t.float().detach().requires_grad_(True) for t in (q, k, v)]
    oref = F.attention_reference(qr, kr, vr, causal, window, None, softcap, slopes)
    qg, kg, vg = [t.detach().requires_grad_(True) for t in (q, k, v)]
    o = F.attention(qg, kg, vg, causal, window, None, softcap, slopes)
    K.check_status()
    assert (o.float() - oref).abs().max() < 2e-2
    do = torch.randn_like(o)
    o.backward(do)
    K.check_status()
    oref.backward(do.float())
    for got, want in ((qg.grad, qr.grad), (kg.grad, kr.grad), (vg.grad, vr.grad)):
        assert (got.float() - want).abs().max() <= 3e-2 * want.abs().max()


def test_attention_varlen_on_kernels():
    """Packed variable-length batch: one kernel launch per sequence on strided views; values and gradients against
    the FP32 math on each sequence alone."""
    from nexus_b200.fused import ops as F
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(2)
    dev = "cuda"
    lens = [200, 37, 512, 129]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    H, Hkv, D = 4, 2, 64
    q = torch.randn(cu[-1], H, D, device=dev).bfloat16().requires_grad_(True)
    k = torch.randn(cu[-1], Hkv, D, device=dev).bfloat16().requires_grad_(True)
    v = torch.randn(cu[-1], Hkv, D, device=dev).bfloat16().requires_grad_(True)
    launches = K.launch_count
    out = F.attention_varlen(q, k, v, torch.tensor(cu), causal=True)
    assert K.launch_count - launches == len(lens)          # the kernel path ran, once per sequence
    do = torch.randn_like(out)
    out.backward(do)
    K.check_status()
    qr, kr, vr = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref = torch.cat([F.attention_reference(qr[None, a:b], kr[None, a:b], vr[None, a:b], True)[0]
                     for a, b in zip(cu[:-1], cu[1:])])
    ref.backward(do.float())
    assert (out.float() - ref).abs().max() < 2e-2
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert (got.float() - want).abs().max() <= 3e-2 * want.abs().max()


@pytest.mark.parametrize("Tq,Tk,H,Hkv,D,causal", [(256, 256, 2, 2, 64, True), (130, 203, 4, 2, 64, False),
                                                 (128, 256, 2, 1, 128, True)])
def test_attention_dropout_in_kernels(Tq, Tk, H, Hkv, D, causal):
    """Attention dropout inside the kernels draws the same Philox stream as the FP32 math path, so values and
    gradients can be compared element by element; the kept fraction matches 1 - p."""
    from nexus_b200.fused import ops as F
    from nexus_b200.fused import philox
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(4)
    dev, p, seed, offset = "cuda", 0.2, 1234, 77
    q = torch.randn(2, Tq, H, D, device=dev).bfloat16()
    k = torch.randn(2, Tk, Hkv, D, device=dev).bfloat16()
    v = torch.randn(2, Tk, Hkv, D, device=dev).bfloat16()
    qr, kr, vr = [t.float().detach().requires_grad_(True) for t in (q, k, v)]
    oref = F.attention_reference(qr, kr, vr, causal, 0, None, 0.0, None, p, seed, offset)
    qg, kg, vg = [t.detach().requires_grad_(True) for t in (q, k, v)]
    o = F.attention(qg, kg, vg, causal, 0, None, 0.0, None, p, seed, offset)
    K.check_status()
    assert (o.float() - oref).abs().max() < 3e-2
    do = torch.randn_like(o)
    o.backward(do)
    K.check_status()
    oref.backward(do.float())
    for got, want in ((qg.grad, qr.grad), (kg.grad, kr.grad), (vg.grad, vr.grad)):
        assert (got.float() - want).abs().max() <= 3e-2 * want.abs().max()
    keep = philox.dropout_mask(2 * H * Tq * Tk, p, seed, offset).mean()
    assert abs(keep - (1 - p)) < 5e-3
    o0 = F.attention(q, k, v, causal, 0, None, 0.0, None, 0.0)
    assert (o0.float() - o.float()).abs().max() > 1e-2          # dropout did change the result


def test_two_tile_forward_rows_without_keys():
    """More queries than keys under the bottom-right aligned causal mask: the first Tq - Tk rows see no key and come
    back as zeros with a log-sum-exp of -inf (whole 256-row items and single tiles without work), the others equal the
    reference."""
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(5)
    dev = "cuda"
    B, Tq, Tk, H, D = 1, 900, 300, 2, 128
    q = torch.randn(B, Tq, H, D, device=dev).bfloat16()
    k = torch.randn(B, Tk, H, D, device=dev).bfloat16()
    v = torch.randn(B, Tk, H, D, device=dev).bfloat16()
    o, lse = K.attention_fwd(q, k, v, causal=True)
    K.check_status()
    dead = Tq - Tk
    assert float(o[:, :dead].float().abs().max()) == 0.0
    assert bool(torch.isinf(lse[:, :, :dead]).all()) and float(lse[:, :, :dead].max()) < 0
    oref, lref = _ref(q[:, dead:].float(), k.float(), v.float(), True, 0, D ** -0.5)
    assert (o[:, dead:].float() - oref).abs().max() < 2e-2
    assert (lse[:, :, dead:] - lref).abs().max() < 2e-2


def test_two_tile_forward_merges_key_chunks():
    """The two-q-tile forward (head_dim 128) with a running (output, log-sum-exp) pair: three key/value chunks merged one
    launch at a time equal one softmax over all keys."""
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(7)
    dev = "cuda"
    B, Tq, Tk, H, D = 1, 384, 768, 2, 128
    q = torch.randn(B, Tq, H, D, device=dev).bfloat16()
    k = torch.randn(B, Tk, H, D, device=dev).bfloat16()
    v = torch.randn(B, Tk, H, D, device=dev).bfloat16()
    mo = torch.zeros(B, Tq, H, D, device=dev)
    ml = torch.full((B, H, Tq), float("-inf"), device=dev)
    for c in range(3):
        o, lse = K.attention_fwd(q, k[:, c * 256:(c + 1) * 256], v[:, c * 256:(c + 1) * 256], causal=False,
                                 merge_o=mo, merge_lse=ml)
    K.check_status()
    oref, lref = _ref(q.float(), k.float(), v.float(), False, 0, D ** -0.5)
    assert (o.float() - oref).abs().max() < 2e-2
    assert (lse - lref).abs().max() < 2e-2
    assert (mo - oref).abs().max() < 2e-2


def test_two_tile_forward_forced_at_head_dim_64():
    """NEXUS_B200_ATTN_FWD=2 routes head_dim 64 through the two-q-tile kernel as well (the choice is read once per
    process, so the check runs in a child)."""
    import os
    import subprocess
    import sys
    code = (
        "import torch\n"
        "from nexus_b200.ops import _cuda as K\n"
        "torch.manual_seed(0)\n"
        "q, k, v = [torch.randn(2, 600, 4, 64, device='cuda').bfloat16() for _ in range(3)]\n"
        "o, lse = K.attention_fwd(q, k, v, causal=True)\n"
        "K.check_status()\n"
        "ref = torch.nn.functional.scaled_dot_product_attention(*[t.float().transpose(1, 2) for t in (q, k, v)],"
        " is_causal=True).transpose(1, 2)\n"
        "assert (o.float() - ref).abs().max() < 2e-2, float((o.float() - ref).abs().max())\n"
        "print('ok')\n")
    env = dict(os.environ, NEXUS_B200_ATTN_FWD="2")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]
