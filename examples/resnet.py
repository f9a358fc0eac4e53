"""Train a ResNet on synthetic images (role of ``examples/resnet.rs``).

  python examples/resnet.py --model resnet18 --steps 5 --image 64
On a GPU the channels-last bf16 kernel path is used (tcgen05 GEMM convolutions, fused BatchNorm/ReLU/residual)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import torsh_b200 as tb


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet18")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--image", type=int, default=64)
    ap.add_argument("--classes", type=int, default=10)
    a = ap.parse_args(argv)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    model = tb.models.create_model(a.model, num_classes=a.classes).to(dev)
    opt = tb.optim.SGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    x = torch.randn(a.batch, 3, a.image, a.image, device=dev)
    y = torch.randint(0, a.classes, (a.batch,), device=dev)
    losses = []
    for s in range(a.steps):
        loss = torch.nn.functional.cross_entropy(model(x).float(), y)
        opt.zero_grad(); loss.backward(); opt.step()
        losses.append(loss.item())
        print(f"step {s}  loss {losses[-1]:.4f}")
    return losses


if __name__ == "__main__":
    main()
