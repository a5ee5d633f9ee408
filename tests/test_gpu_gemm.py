"""tcgen05 GEMM vs an FP32 PyTorch reference: every operand layout, both tile widths, tails,
fused epilogues, split-K (deterministic and reduction-based) and the strided batch."""
import itertools

import pytest
import torch

pytestmark = pytest.mark.gpu


def _K():
    from nexus_b200.ops import _cuda as K
    return K


def _operands(M, N, Kd, a_mn, b_mn):
    A = torch.randn(M, Kd, device="cuda").bfloat16()
    B = torch.randn(N, Kd, device="cuda").bfloat16()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    return A, B, a, b


@pytest.mark.parametrize("a_mn,b_mn", list(itertools.product((False, True), repeat=2)))
@pytest.mark.parametrize("bn", (128, 256))
@pytest.mark.parametrize("shape", ((128, 128, 64), (256, 512, 320), (304, 200, 136)))
def test_gemm_layouts(a_mn, b_mn, bn, shape):
    K = _K()
    torch.manual_seed(1)
    M, N, Kd = shape
    A, B, a, b = _operands(M, N, Kd, a_mn, b_mn)
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=bn)
    K.check_status()
    ref = A.float() @ B.float().t()
    assert (out.float() - ref).abs().max() <= 1.5e-2 * ref.abs().max()


@pytest.mark.parametrize("a_mn,b_mn", list(itertools.product((False, True), repeat=2)))
def test_gemm_cta_pair_many_tiles(a_mn, b_mn):
    """256 x 256 tiles over CTA pairs: more tiles than clusters, more k-blocks than stages, ragged M and N."""
    K = _K()
    torch.manual_seed(7)
    M, N, Kd = 5000, 1096, 1096
    A, B, a, b = _operands(M, N, Kd, a_mn, b_mn)
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    K.check_status()
    ref = A.float() @ B.float().t()
    assert (out.float() - ref).abs().max() <= 1.5e-2 * ref.abs().max()
    if not a_mn and not b_mn:   # the same product from single-CTA tiles (128-wide) agrees to rounding
        out1 = K.gemm(a, b, block_n=128)
        assert (out.float() - out1.float()).abs().max() <= 4e-3 * ref.abs().max()


def test_gemm_bias_gelu_aux():
    K = _K()
    torch.manual_seed(2)
    M, N, Kd = 1024, 3072, 768
    A, B, a, b = _operands(M, N, Kd, False, False)
    bias = torch.randn(N, device="cuda")
    aux = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = K.gemm(a, b, bias=bias, act="gelu", aux_out=aux)
    K.check_status()
    pre = A.float() @ B.float().t() + bias
    ref = torch.nn.functional.gelu(pre, approximate="tanh")
    assert (aux.float() - pre).abs().max() <= 1.5e-2 * pre.abs().max()
    assert (out.float() - ref).abs().max() <= 1.5e-2 * ref.abs().max()


def test_gemm_dgelu_residual_accumulate():
    K = _K()
    torch.manual_seed(3)
    M, N, Kd = 512, 768, 1024
    A, B, a, b = _operands(M, N, Kd, False, True)
    pre = torch.randn(M, N, device="cuda").bfloat16()
    out = K.gemm(a, b, b_mn=True, act="dgelu", aux_in=pre)
    K.check_status()
    x = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(x, approximate="tanh").sum().backward()
    ref = (A.float() @ B.float().t()) * x.grad
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    res = torch.randn(M, N, device="cuda")
    bias = torch.randn(N, device="cuda").bfloat16()
    out = K.gemm(a, b, b_mn=True, bias=bias, residual=res, out_dtype=torch.float32)
    ref = A.float() @ B.float().t() + bias.float() + res
    assert (out - ref).abs().max() <= 1e-3 * ref.abs().max()
    acc = torch.randn(M, N, device="cuda")
    ref = acc + A.float() @ B.float().t()
    K.gemm(a, b, b_mn=True, out=acc, accumulate=True)
    K.check_status()
    assert (acc - ref).abs().max() <= 1e-3 * ref.abs().max()


@pytest.mark.parametrize("deterministic", (True, False))
def test_gemm_split_k(deterministic):
    K = _K()
    torch.manual_seed(4)
    M, N, Kd = 768, 768, 4096
    A, B, a, b = _operands(M, N, Kd, True, True)
    acc0 = torch.randn(M, N, device="cuda")
    ref = acc0 + A.float() @ B.float().t()
    outs = []
    for _ in range(2):
        acc = acc0.clone()
        K.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True, split_k=4, deterministic=deterministic)
        K.check_status()
        assert (acc - ref).abs().max() <= 1e-3 * ref.abs().max()
        outs.append(acc)
    if deterministic:
        assert torch.equal(outs[0], outs[1])


def test_gemm_batched():
    K = _K()
    torch.manual_seed(5)
    A = torch.randn(5, 200, 72, device="cuda").bfloat16()
    B = torch.randn(5, 136, 72, device="cuda").bfloat16()
    out = K.gemm(A, B)
    K.check_status()
    ref = torch.einsum("bmk,bnk->bmn", A.float(), B.float())
    assert (out.float() - ref).abs().max() <= 1.5e-2 * ref.abs().max()


def test_gemm_rejects_unaligned_pitch():
    K = _K()
    a = torch.randn(64, 36, device="cuda").bfloat16()  # pitch 36: not a multiple of 8 elements
    b = torch.randn(64, 36, device="cuda").bfloat16()
    with pytest.raises(RuntimeError):
        K.gemm(a, b)


def test_gemm_split_k_with_epilogue_in_the_reduction():
    """Few rows, many K slices: bias + GELU (BF16 out) and bias + in-place FP32 residual come out of the reduction
    pass exactly as from the unsplit GEMM's epilogue, run to run bit-identical."""
    K = _K()
    torch.manual_seed(9)
    M, N, Kd = 64, 768, 3072
    A, B, a, b = _operands(M, N, Kd, False, False)
    bias = torch.randn(N, device="cuda")
    ref = A.float() @ B.float().t() + bias
    o1 = K.gemm(a, b, bias=bias, act="gelu", split_k=0, block_n=128, deterministic=True)
    o2 = K.gemm(a, b, bias=bias, act="gelu", split_k=8, block_n=128, deterministic=True)
    K.check_status()
    want = torch.nn.functional.gelu(ref, approximate="tanh")
    assert (o1.float() - want).abs().max() <= 1.5e-2 * want.abs().max()
    assert (o2.float() - want).abs().max() <= 1.5e-2 * want.abs().max()
    assert torch.equal(o1, K.gemm(a, b, bias=bias, act="gelu", split_k=0, block_n=128, deterministic=True))
    res = torch.randn(M, N, device="cuda")
    want = res + ref
    out = res.clone()
    K.gemm(a, b, bias=bias, residual=out, out=out, out_dtype=torch.float32, split_k=0, block_n=128, deterministic=True)
    K.check_status()
    assert (out - want).abs().max() <= 2e-3 * want.abs().max()
