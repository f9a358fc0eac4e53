"""The ``rstorch`` surface and the fused ops (roles of ``examples/python/tensor_operations.py`` and
``neural_network.py``): the same script runs on CPU and, with kernels, on a B200."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import rstorch
import torsh_b200 as tb


def main(argv=None):
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    a = rstorch.randn(4, 8, device=dev)
    b = rstorch.ones(8, 3, device=dev)
    c = (a @ b).relu().sum()
    print("rstorch:", tuple(a.shape), float(c))
    x = torch.randn(16, 64, device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32, requires_grad=True)
    w = torch.randn(128, 64, device=dev, dtype=x.dtype, requires_grad=True)
    y = tb.ops.linear.linear(x, w, None, gelu=True)            # one GEMM launch with a GELU epilogue on the GPU
    y = tb.ops.norm.layer_norm(y, torch.ones(128, device=dev, dtype=x.dtype), torch.zeros(128, device=dev, dtype=x.dtype))
    y.float().sum().backward()
    print("fused linear+gelu → layer_norm:", tuple(y.shape), "grad norm", float(w.grad.float().norm()))
    net = rstorch.nn.Sequential(rstorch.nn.Linear(8, 16), rstorch.nn.ReLU(), rstorch.nn.Linear(16, 2)).to(dev)
    opt = rstorch.optim.SGD(net.parameters(), lr=0.1)
    for _ in range(3):
        loss = net(a).pow(2).mean()
        opt.zero_grad(); loss.backward(); opt.step()
    print("rstorch.nn loss", loss.item())
    return loss.item()


if __name__ == "__main__":
    main()
