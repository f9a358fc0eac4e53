"""Activation checkpointing (role of ``examples/gradient_checkpointing.rs``): the scheduler picks which blocks to
recompute, and the gradients equal those of the plain run."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from torsh_b200 import autograd as ag


def main(argv=None):
    torch.manual_seed(0)
    blocks = torch.nn.ModuleList([torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.GELU()) for _ in range(8)])
    x = torch.randn(16, 64)

    def run(policy):
        for p in blocks.parameters():
            p.grad = None
        h = x
        for i, b in enumerate(blocks):
            h = ag.checkpoint(b, h) if policy(i) else b(h)
        h.pow(2).mean().backward()
        return torch.cat([p.grad.reshape(-1) for p in blocks.parameters()])

    plain = run(lambda i: False)
    plan = ag.CheckpointScheduler(ag.CheckpointStrategy.SQRT).plan(len(blocks))
    chosen = {i for i, recompute in enumerate(plan) if recompute}
    ckpt = run(lambda i: i in chosen)
    err = float((plain - ckpt).abs().max())
    print(f"checkpointed blocks {sorted(chosen)}; max gradient difference {err:.2e}")
    return err


if __name__ == "__main__":
    main()
