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
