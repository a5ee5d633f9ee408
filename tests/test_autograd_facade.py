import pytest
import torch

from nexus_b200 import autograd as ag
from nexus_b200.autograd.checkpoint import SavedBytesCounter, checkpoint


def test_variable_graph_and_hooks():
    x = ag.Variable([[1.0, 2.0], [3.0, 4.0]], requires_grad=True)
    seen = []
    x.register_hook(lambda g: seen.append("hook") or g)
    x.register_post_accumulate_grad_hook(lambda v: seen.append("post"))
    y = ag.sum(ag.mul(x, x))
    assert y.grad_fn().name().startswith("Sum")
    assert any(e.is_valid() for e in y.grad_fn().next_edges())
    y.backward()
    assert x.grad.tolist() == [[2.0, 4.0], [6.0, 8.0]] and seen == ["hook", "post"]
    assert x.grad_accumulator().is_accumulate_grad()
    c = ag.Variable(x)           # copying is a deep copy
    c.tensor.data[0, 0] = 99.0
    assert x.tensor[0, 0] == 1.0 and x.shallow().tensor is x.tensor


def test_grad_modes_and_retain_grad():
    x = ag.Variable([1.0, 2.0], requires_grad=True)
    with ag.NoGradGuard():
        assert not ag.mul(x, x).requires_grad
        with ag.EnableGradGuard():
            assert ag.mul(x, x).requires_grad
    h = ag.mul(x, x)
    h.retain_grad()
    ag.sum(h).backward()
    assert h.grad.tolist() == [1.0, 1.0]


def test_saved_tensor_hooks_and_version_check():
    packed = []
    ag.set_saved_tensors_hooks(lambda t: packed.append(t.shape) or t, lambda t: t)
    try:
        x = ag.Variable([1.0, 2.0], requires_grad=True)
        ag.sum(ag.mul(x, x)).backward()
    finally:
        ag.set_saved_tensors_hooks(None, None)
    assert packed
    t = torch.ones(3)
    s = ag.SavedTensor(t)
    t.add_(1)
    with pytest.raises(RuntimeError, match="modified in place"):
        s.unpack()


def test_anomaly_mode_names_the_failure():
    x = ag.Variable([0.0], requires_grad=True)
    with pytest.raises(ag.AnomalyError):
        with ag.detect_anomaly():
            ag.sum(ag.div(x, x)).backward()


def test_custom_function_and_gradcheck():
    def fwd(ctx, a):
        ctx.save_for_backward(a)
        return a * a * a

    def bwd(ctx, g):
        (a,) = ctx.saved_tensors
        return 3 * a * a * g
    cube = ag.custom_function(fwd, bwd, "Cube")
    x = ag.Variable([1.0, 2.0], requires_grad=True)
    ag.sum(cube(x)).backward()
    assert x.grad.tolist() == [3.0, 12.0]
    assert ag.gradcheck(lambda a: ag.sum(ag.tanh(ag.matmul(a, a))), [ag.Variable(torch.randn(3, 3))])


def test_checkpoint_matches_plain_backward_and_saves_less():
    torch.manual_seed(0)
    lin1, lin2 = torch.nn.Linear(16, 64), torch.nn.Linear(64, 16)
    f = lambda t: lin2(torch.nn.functional.gelu(lin1(t)))
    x = torch.randn(8, 16, requires_grad=True)
    with SavedBytesCounter() as plain:
        f(x).sum().backward()
    g0 = [x.grad.clone(), lin1.weight.grad.clone()]
    x.grad = None
    lin1.weight.grad = None
    with SavedBytesCounter() as ck:
        checkpoint(lambda t: checkpoint(f, t), x).sum().backward()   # nested
    assert torch.equal(x.grad, g0[0]) and torch.equal(lin1.weight.grad, g0[1])
    assert ck.bytes < plain.bytes


def test_module_function_wraps_explicit_backward():
    import torch
    from nexus_b200 import autograd as A

    class Scale:
        def __init__(self):
            self.w, self.gw = torch.tensor(3.0), torch.tensor(0.0)

        def forward(self, x):
            self.x = x
            return x * self.w

        def backward(self, g):
            self.gw = self.gw + (g * self.x).sum()
            return g * self.w
    mod = Scale()
    f = A.module_function(mod)
    x = A.Variable(torch.tensor([1.0, 2.0]), requires_grad=True)
    A.sum(f(x)).backward()
    assert float(mod.gw) == 3.0 and x.grad.tensor.tolist() == [3.0, 3.0]
