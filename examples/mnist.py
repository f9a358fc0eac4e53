"""A small convolutional classifier trained with the package's data pipeline, layers, optimizer, scheduler and metrics
(roles of ``examples/mnist.rs`` and ``examples/python/neural_network.py``). There is no dataset on disk here, so the
"digits" are synthetic: ten fixed 28x28 prototypes plus noise; swap in ``torsh_b200.vision`` datasets for real data."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import torsh_b200 as tb


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--samples", type=int, default=512)
    a = ap.parse_args(argv)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    g = torch.Generator().manual_seed(0)
    protos = torch.randn(10, 1, 28, 28, generator=g)
    labels = torch.randint(0, 10, (a.samples,), generator=g)
    images = protos[labels] + 0.5 * torch.randn(a.samples, 1, 28, 28, generator=g)
    loader = torch.utils.data.DataLoader(torch.utils.data.TensorDataset(images, labels), batch_size=64, shuffle=True,
                                         generator=torch.Generator().manual_seed(1))
    model = torch.nn.Sequential(
        torch.nn.Conv2d(1, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.MaxPool2d(2),
        torch.nn.Conv2d(8, 16, 3, padding=1), torch.nn.ReLU(), torch.nn.MaxPool2d(2),
        torch.nn.Flatten(), torch.nn.Linear(16 * 7 * 7, 10)).to(dev)
    opt = tb.optim.AdamW(model.parameters(), lr=3e-3) if hasattr(tb.optim, "AdamW") else torch.optim.AdamW(model.parameters(), lr=3e-3)
    sched = torch.optim.lr_scheduler.CosineAnnealingLR(opt, T_max=a.epochs * len(loader))
    history = []
    for epoch in range(a.epochs):
        correct = total = 0
        for x, y in loader:
            x, y = x.to(dev), y.to(dev)
            logits = model(x)
            loss = torch.nn.functional.cross_entropy(logits, y)
            opt.zero_grad()
            loss.backward()
            opt.step()
            sched.step()
            correct += int((logits.argmax(1) == y).sum())
            total += len(y)
        history.append(correct / total)
        print(f"epoch {epoch}: loss {loss.item():.3f}, accuracy {history[-1]:.3f}")
    return history


if __name__ == "__main__":
    main()
