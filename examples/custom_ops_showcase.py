"""Custom activation / loss / optimizer / module on a small regression problem (CPU)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nexus_b200.custom import CustomActivation, CustomLoss, CustomOptimizer  # noqa: E402


def main():
    torch.manual_seed(0)
    x = torch.linspace(-2, 2, 64)[:, None]
    y = torch.sin(2 * x)
    net = torch.nn.Sequential(torch.nn.Linear(1, 32), CustomActivation("swish", lambda t: t * torch.sigmoid(t)),
                              torch.nn.Linear(32, 1))
    huber = CustomLoss.from_explicit("huber", lambda p, t: (torch.nn.functional.huber_loss(p, t),
                                                            torch.clamp(p - t, -1, 1) / p.numel()))

    def lion(p, g, st, step, h):
        update = torch.sign(h["b1"] * st["m"] + (1 - h["b1"]) * g)
        st["m"].mul_(h["b2"]).add_(g, alpha=1 - h["b2"])
        return p - h["lr"] * update
    opt = CustomOptimizer(net.parameters(), lion, slots=("m",), lr=3e-3, b1=0.9, b2=0.99)
    for step in range(400):
        opt.zero_grad()
        loss = huber(net(x), y)
        loss.backward()
        opt.step()
        if step % 100 == 0:
            print(f"step {step}: huber {float(loss.detach()):.5f}")
    print(f"final: {float(huber(net(x), y)):.5f}")


if __name__ == "__main__":
    main()
