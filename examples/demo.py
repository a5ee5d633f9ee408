"""The smallest end-to-end run: a two-layer network on XOR through the `nexus` shell.  Counterpart of apps/demo."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import nexus  # noqa: E402


def main() -> int:
    torch.manual_seed(0)
    x = torch.tensor([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]])
    y = torch.tensor([0, 1, 1, 0])
    net = nexus.nn.Sequential(nexus.nn.Linear(2, 8), nexus.nn.GELU(), nexus.nn.Linear(8, 2))
    opt = torch.optim.Adam(net.parameters(), lr=0.05)
    for _ in range(300):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(net(x), y)
        loss.backward()
        opt.step()
    pred = net(x).argmax(-1)
    print(f"nexus {getattr(nexus, '__version__', '')} xor loss {float(loss.detach()):.4f} predictions {pred.tolist()}")
    return 0 if torch.equal(pred, y) else 1


if __name__ == "__main__":
    sys.exit(main())
