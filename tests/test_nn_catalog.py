import pytest
import torch

from nexus_b200 import nn


@pytest.mark.parametrize("layer,shape", [
    (lambda: nn.Linear(6, 3, True), (4, 6)), (lambda: nn.Conv1d(2, 4, 3, 1, 1, True), (2, 2, 9)),
    (lambda: nn.Conv2d(2, 4, 3, 1, 1, True), (2, 2, 6, 6)), (lambda: nn.Conv3d(1, 2, 3, 1, 1, True), (1, 1, 4, 4, 4)),
    (lambda: nn.DepthwiseConv2d(3, 3, 1, 1), (2, 3, 5, 5)), (lambda: nn.MultiHeadAttention(8, 2), (2, 5, 8)),
    (lambda: nn.LSTM(4, 6), (2, 5, 4)), (lambda: nn.GRU(4, 6), (2, 5, 4)), (lambda: nn.RNN(4, 6), (2, 5, 4)),
    (lambda: nn.TransformerEncoder(8, 2, 16), (2, 5, 8)), (lambda: nn.TransformerDecoder(8, 2, 16), (2, 5, 8)),
    (lambda: nn.CausalTransformerBlock(8, 2, 16), (2, 5, 8)), (lambda: nn.BatchNorm1d(6), (4, 6)),
    (lambda: nn.BatchNorm2d(3), (2, 3, 4, 4)), (lambda: nn.LayerNorm(6), (4, 6)), (lambda: nn.GroupNorm(2, 4), (2, 4, 3, 3)),
    (lambda: nn.InstanceNorm(3), (2, 3, 4, 4)), (lambda: nn.ReLU(), (3, 3)), (lambda: nn.GELU(), (3, 3)),
    (lambda: nn.SiLU(), (3, 3)), (lambda: nn.Mish(), (3, 3)), (lambda: nn.swish(), (3, 3)), (lambda: nn.Dropout(0.5), (64,)),
    (lambda: nn.MaxPool2d(2), (1, 2, 4, 4)), (lambda: nn.AvgPool2d(2), (1, 2, 4, 4)), (lambda: nn.GlobalAvgPool2d(), (1, 2, 4, 4)),
    (lambda: nn.Flatten(), (2, 3, 4)), (lambda: nn.Reshape([3, 4]), (2, 12)), (lambda: nn.Residual(nn.Linear(4, 4)), (2, 4)),
    (lambda: nn.PositionalEncoding(8, 16, True), (2, 5, 8)),
])
def test_layer_forward_backward_and_spec_round_trip(layer, shape):
    torch.manual_seed(0)
    m = layer()
    x = torch.randn(*shape)
    y = m(x)
    gx = m.backward(torch.ones_like(y))
    assert gx is not None and gx.shape == x.shape
    m2 = nn.make_one(m.nxs_spec())
    assert type(m2) is type(m) or isinstance(m2, nn.Activation)
    assert [p.shape for p in m2.parameters()] == [p.shape for p in m.parameters()]


def test_embedding_and_sequential_backward():
    e = nn.Embedding(10, 4, 0)
    assert e(torch.tensor([[1, 2, 0]])).shape == (1, 3, 4)
    m = nn.Sequential().add(nn.Linear(4, 8, True)).add(nn.ReLU()).add(nn.Linear(8, 2, True))
    x = torch.randn(3, 4)
    y = m(x)
    gx = m.backward(torch.ones_like(y))
    x2 = x.clone().requires_grad_(True)
    m(x2).sum().backward()
    assert torch.allclose(gx, x2.grad) and len(m) == 3


def test_causal_block_is_post_norm_and_causal():
    torch.manual_seed(0)
    blk = nn.CausalTransformerBlock(8, 2, 16)
    blk.eval()
    x = torch.randn(1, 6, 8)
    y = blk(x)
    x2 = x.clone()
    x2[0, 4:] += 1.0
    assert torch.allclose(blk(x2)[0, :4], y[0, :4], atol=1e-6)          # the future does not leak
    assert torch.allclose(y.mean(-1), torch.zeros(1, 6), atol=1e-5)      # output is a LayerNorm output
    enc = nn.TransformerEncoder(8, 2, 16)
    enc.eval()
    assert not torch.allclose(enc(x2)[0, :4], enc(x)[0, :4], atol=1e-6)  # the encoder is not causal
    assert [n.split(".")[0] for n, _ in blk.named_parameters()][::2][:5] == ["attn", "attn", "ln1", "fc1", "fc2"]


def test_graph_merges():
    torch.manual_seed(0)
    a, b = nn.Linear(4, 4), nn.Linear(4, 4)
    g = nn.Graph().add("a", a).add("b", b, ["input"]).add("s", nn.ReLU(), ["a", "b"]).add("c", nn.Linear(8, 2), ["a", "b"], True)
    x = torch.randn(3, 4)
    assert g.merge == {"a": 0, "b": 0, "s": 1, "c": 32}
    assert torch.allclose(g(x), g.nodes["c"](torch.cat([a(x), b(x)], -1)))
    g.set_output("s")
    assert torch.allclose(g(x), torch.relu(a(x) + b(x)))
    gx = g.backward(torch.ones(3, 4))
    assert gx.shape == x.shape


def test_functional_forms_match_torch():
    """`nn.functional`: the stateless operator forms against torch on CPU tensors (the fused ops fall back to their
    FP32 reference statements there): activations, gated activations, norms, attention in torch's layout with
    grouped-query heads, embedding, dropout drawn from the Philox stream."""
    import torch
    from nexus_b200.nn import functional as F
    TF = torch.nn.functional
    torch.manual_seed(0)
    x = torch.randn(5, 16)
    assert torch.allclose(F.gelu(x), TF.gelu(x, approximate="tanh"), atol=1e-6)
    assert torch.allclose(F.gelu(x, approximate="none"), TF.gelu(x), atol=1e-6)
    h = torch.randn(5, 32)
    assert torch.allclose(F.swiglu(h), TF.silu(h[:, :16]) * h[:, 16:], atol=1e-6)
    assert torch.allclose(F.geglu(h), TF.gelu(h[:, :16], approximate="tanh") * h[:, 16:], atol=1e-5)
    g, b = torch.randn(16), torch.randn(16)
    assert torch.allclose(F.layer_norm(x, g, b), TF.layer_norm(x, (16,), g, b), atol=1e-5)
    res = torch.randn(5, 16)
    out = F.residual_layer_norm(x, res, g, b)
    y = out[0] if isinstance(out, tuple) else out
    assert torch.allclose(y, TF.layer_norm(x + res, (16,), g, b), atol=1e-5)
    assert torch.allclose(F.rms_norm(x, g), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * g, atol=1e-5)
    assert torch.allclose(F.softmax(x), torch.softmax(x, -1), atol=1e-6)
    w, bias = torch.randn(8, 16), torch.randn(8)
    assert torch.allclose(F.linear(x, w, bias), TF.linear(x, w, bias), atol=1e-5)
    q, k, v = torch.randn(2, 4, 10, 8), torch.randn(2, 2, 10, 8), torch.randn(2, 2, 10, 8)
    want = TF.scaled_dot_product_attention(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), is_causal=True)
    assert torch.allclose(F.scaled_dot_product_attention(q, k, v, is_causal=True), want, atol=1e-5)
    toks = torch.randint(0, 20, (2, 6))
    table = torch.randn(20, 12)
    assert torch.equal(F.embedding(toks, table), table[toks])
    d1, d2 = F.dropout(x, 0.5, seed=3, offset=10), F.dropout(x, 0.5, seed=3, offset=10)
    assert torch.equal(d1, d2) and 0 < int((d1 == 0).sum()) < x.numel()
    assert torch.equal(F.dropout(x, 0.5, seed=3, offset=10, training=False), x)
