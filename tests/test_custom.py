import math

import pytest
import torch

from nexus_b200.custom import (CallbackList, CustomActivation, CustomCallback, CustomLoss, CustomMetric, CustomModule,
                               CustomOptimizer, MicroTape, Tape)


def test_microtape_gradients():
    t = MicroTape()
    x, y = t.variable(1.5), t.variable(-0.5)
    out = t.log(t.exp(x * y) + t.square(x)) / (t.abs(y) + 2.0) - t.max(x, y) * 3.0 + (-x)
    g = t.gradient(out)
    xt = torch.tensor(1.5, requires_grad=True, dtype=torch.float64)
    yt = torch.tensor(-0.5, requires_grad=True, dtype=torch.float64)
    ref = torch.log(torch.exp(xt * yt) + xt ** 2) / (yt.abs() + 2.0) - torch.maximum(xt, yt) * 3.0 - xt
    ref.backward()
    assert abs(out.value - float(ref)) < 1e-12
    assert abs(g[x.idx] - float(xt.grad)) < 1e-12 and abs(g[y.idx] - float(yt.grad)) < 1e-12


def test_tape_matches_autograd():
    torch.manual_seed(0)
    a, w, b = torch.randn(4, 3), torch.randn(3, 5), torch.randn(1, 5)
    tp = Tape()
    ia, iw, ib = tp.input(a), tp.input(w), tp.input(b)
    out = tp.mul(tp.relu(tp.add(tp.matmul(ia, iw), ib)), tp.add(tp.matmul(ia, iw), ib))
    g = tp.backward(out)
    at, wt, bt = (t.clone().requires_grad_(True) for t in (a, w, b))
    h = at @ wt + bt
    (torch.relu(h) * h).sum().backward()
    assert torch.allclose(g[ia], at.grad, atol=1e-5) and torch.allclose(g[iw], wt.grad, atol=1e-5)
    assert torch.allclose(g[ib], bt.grad, atol=1e-5)


def test_custom_activation_scalar_and_batch():
    swish = CustomActivation("swish", lambda x: x * torch.sigmoid(x))
    x = torch.randn(3, 4, requires_grad=True)
    swish(x).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    (xr * torch.sigmoid(xr)).sum().backward()
    assert torch.allclose(x.grad, xr.grad, atol=1e-3)
    sq = CustomActivation("sq", lambda v: v * v, derivative=lambda v: 2 * v, batch=False)
    y = torch.tensor([1.0, -2.0, 3.0], requires_grad=True)
    sq(y).sum().backward()
    assert y.grad.tolist() == [2.0, -4.0, 6.0]


def test_custom_loss_three_modes_agree():
    p, t = torch.tensor([0.2, -1.0, 2.5]), torch.tensor([0.0, 1.0, 2.0])
    exp = CustomLoss.from_explicit("mse", lambda a, b: (((a - b) ** 2).mean(), 2 * (a - b) / a.numel()))
    num = CustomLoss.from_numeric("mse", lambda a, b: ((a - b) ** 2).mean())

    def prog(tape, pv, tv):
        s = tape.const(0.0)
        for a, b in zip(pv, tv):
            s = s + tape.square(a - b)
        return s / float(len(pv))
    tap = CustomLoss.from_tape("mse", prog)
    l0, g0 = exp.forward_backward(p, t)
    for other in (num, tap):
        l, g = other.forward_backward(p, t)
        assert abs(l - l0) < 1e-5 and torch.allclose(g, g0, atol=1e-3)
    q = p.clone().requires_grad_(True)
    tap(q, t).backward()
    assert torch.allclose(q.grad, g0, atol=1e-6)


def test_metric_optimizer_callbacks_module():
    m = CustomMetric("acc", lambda: [0, 0], lambda s, p, t: [s[0] + int((p.argmax(-1) == t).sum()), s[1] + t.numel()],
                     lambda s: s[0] / max(1, s[1]))
    m.update(torch.tensor([[0.1, 0.9], [0.8, 0.2]]), torch.tensor([1, 1]))
    assert m.result() == 0.5
    m.reset()
    assert m.result() == 0.0
    w = torch.nn.Parameter(torch.tensor([5.0, -3.0]))

    def momentum(p, g, st, step, h):
        st["v"].mul_(h["beta"]).add_(g)
        return p - h["lr"] * st["v"]
    opt = CustomOptimizer([w], momentum, slots=("v",), lr=0.1, beta=0.5)
    for _ in range(60):
        opt.zero_grad()
        (w ** 2).sum().backward()
        opt.step()
    assert w.abs().max() < 1e-3 and opt.state[w]["step"] == 60
    seen = []
    cbs = CallbackList([CustomCallback(on_epoch_end=lambda e, logs: seen.append(e)),
                        CustomCallback(on_epoch_end=lambda e, logs: False if e >= 1 else None)])
    assert cbs.fire("on_epoch_end", 0, {}) is False and cbs.fire("on_epoch_end", 1, {}) is True and seen == [0, 1]
    with pytest.raises(ValueError):
        CustomCallback(on_nothing=lambda: None)
    scale = CustomModule("scale", {"s": (1, 3)}, lambda x, p: x * p["s"],
                         lambda x, p, gy: (gy * p["s"], {"s": (gy * x).sum(0, keepdim=True)}))
    x = torch.randn(4, 3, requires_grad=True)
    scale(x).sum().backward()
    assert torch.allclose(x.grad, scale.slots["s"].detach().expand(4, 3))
    assert torch.allclose(scale.slots["s"].grad, x.detach().sum(0, keepdim=True))
    tp = Tape()
    i = tp.input(x.detach())
    o = tp.module(scale, i)
    scale.slots["s"].grad = None
    g = tp.backward(o)
    assert torch.allclose(g[i], x.grad) and torch.allclose(scale.slots["s"].grad, x.detach().sum(0, keepdim=True))
