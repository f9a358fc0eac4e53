"""Train a GPT-2-style language model (role of the reference's ``examples/gpt2.rs``).

  python examples/gpt2.py --model gpt2-tiny --steps 20            # CPU or one GPU
On a GPU the step runs through ``CausalLMTrainer`` (flat bf16 parameters with fp32 master weights, fused AdamW,
whole-step CUDA graph); on the CPU it is a plain fp32 optimizer loop over the same model code."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import torsh_b200 as tb
from torsh_b200.data import SyntheticTokenDataset


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2-tiny")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--lr", type=float, default=3e-4)
    a = ap.parse_args(argv)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    model = tb.models.create_model(a.model).to(dev)
    cfg = model.config
    seq = min(a.seq, cfg.n_positions)
    ds = SyntheticTokenDataset(cfg.vocab_size, seq, a.steps * a.batch, seed=0)
    if dev.type == "cuda":
        trainer = tb.engine.CausalLMTrainer(model, lr=a.lr, batch_size=a.batch, seq_len=seq)
        step = trainer.step
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=a.lr)

        def step(x, y):
            loss = model(x, targets=y) if "targets" in model.forward.__code__.co_varnames else torch.nn.functional.cross_entropy(
                model(x).reshape(-1, cfg.vocab_size), y.reshape(-1))
            opt.zero_grad(); loss.backward(); opt.step()
            return loss.item()
    losses = []
    for s in range(a.steps):
        rows = [ds[s * a.batch + i] for i in range(a.batch)]
        x, y = torch.stack([r[0] for r in rows]).to(dev), torch.stack([r[1] for r in rows]).to(dev)
        losses.append(float(step(x, y)))
        if s % 5 == 0 or s + 1 == a.steps:
            print(f"step {s:4d}  loss {losses[-1]:.4f}")
    return losses


if __name__ == "__main__":
    main()
