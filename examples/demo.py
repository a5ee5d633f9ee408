"""The smallest end-to-end run: a two-layer network on XOR through the `nexus` shell (flat lists in, a trainer built
with the builder, an archive round trip).  Counterpart of apps/demo."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import nexus  # noqa: E402


def main() -> int:
    features = [0.0, 0.0, 0.0, 1.0, 1.0, 0.0, 1.0, 1.0] * 8
    labels = [0, 1, 1, 0] * 8
    net = nexus.nn.Sequential()
    net.add(nexus.nn.Linear(2, 16, True))
    net.add(nexus.nn.swish())
    net.add(nexus.nn.Linear(16, 2, True))
    trainer = (nexus.train.TrainerBuilder(net).adamw(net, lr=0.05).loss(0.0).execution_policy_cpu().accuracy().build())
    loader = nexus.data.DataLoader(features, labels, 2, 8, True, 0)
    trainer.fit(loader, loader, 60)
    last = trainer.history()[-1]
    x = nexus.Tensor([4, 2])
    x.copy_from(features[:8])
    logits = net.forward(x).to_list()
    pred = [int(logits[2 * i + 1] > logits[2 * i]) for i in range(4)]
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "xor.nxs")
        net.save_nxs(path)
        same = nexus.load(path).forward(x).to_list() == logits
    print(f"nexus {nexus.__version__} xor loss {last.train_loss:.4f} predictions {pred} archive round trip {same}")
    return 0 if pred == [0, 1, 1, 0] and same else 1


if __name__ == "__main__":
    sys.exit(main())
