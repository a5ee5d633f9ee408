"""Loss functions with ``forward_backward`` (value + gradient w.r.t. the prediction in one call).
`backward_into` variants write the gradient into a caller buffer (no allocation).
Parity: include/nexus/loss and include/nexus/loss/backward_into.hpp of the reference."""
from __future__ import annotations

import torch
import torch.nn.functional as F


class CrossEntropy:
    def __init__(self, label_smoothing: float = 0.0):
        self.label_smoothing = float(label_smoothing)

    def forward(self, logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return F.cross_entropy(logits.float(), target.long(), label_smoothing=self.label_smoothing)

    def forward_backward(self, logits: torch.Tensor, target: torch.Tensor):
        lf = logits.detach().float()
        n, c = lf.shape[0], lf.shape[-1]
        logp = torch.log_softmax(lf, -1)
        s = self.label_smoothing
        q = torch.full_like(lf, s / c)
        q.scatter_(1, target.long()[:, None], 1.0 - s + s / c)
        loss = -(q * logp).sum(-1).mean()
        return loss, (logp.exp() - q) / n

    def backward_into(self, logits, target, out: torch.Tensor) -> torch.Tensor:
        loss, g = self.forward_backward(logits, target)
        out.copy_(g)
        return loss


class _Elementwise:
    def forward_backward(self, pred: torch.Tensor, target: torch.Tensor):
        p = pred.detach().float().requires_grad_(True)
        with torch.enable_grad():
            l = self.forward(p, target.float())
            l.backward()
        return l.detach(), p.grad

    def backward_into(self, pred, target, out):
        loss, g = self.forward_backward(pred, target)
        out.copy_(g)
        return loss


class MSE(_Elementwise):
    def forward(self, pred, target): return F.mse_loss(pred.float(), target.float())


class MAE(_Elementwise):
    def forward(self, pred, target): return F.l1_loss(pred.float(), target.float())


class Huber(_Elementwise):
    def __init__(self, delta: float = 1.0): self.delta = delta
    def forward(self, pred, target): return F.huber_loss(pred.float(), target.float(), delta=self.delta)


class BCE(_Elementwise):
    def forward(self, pred, target): return F.binary_cross_entropy_with_logits(pred.float(), target.float())
