"""Language-model training from a token file: the native loader cuts batches on worker threads into pinned buffers, and
the trainer runs one step ahead of the loss read (``step_async``), so neither the file nor the loss read stalls the GPU.

  python examples/train_from_tokens.py [--tokens corpus.bin] [--steps 20]
Without ``--tokens`` a synthetic corpus with a repeating pattern is written to a temporary file."""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import numpy as np
import torch

import torsh_b200 as tb
from torsh_b200.data import NativeTokenLoader


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default=None, help="raw uint16 token ids")
    ap.add_argument("--model", default="gpt2-tiny")
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=64)
    a = ap.parse_args(argv)
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = tb.models.create_model(a.model).to(dev)
    path = a.tokens
    if path is None:
        period = np.arange(97, dtype=np.uint16) * 7 % model.config.vocab_size
        path = os.path.join(tempfile.mkdtemp(), "corpus.bin")
        np.tile(period, 400).astype(np.uint16).tofile(path)
    loader = NativeTokenLoader(path, batch=a.batch, seq=a.seq, workers=2, seed=0)
    trainer = tb.engine.CausalLMTrainer(model, lr=1e-3, batch_size=a.batch, seq_len=a.seq, use_graph=dev.type == "cuda")
    losses, pending = [], None
    for _ in range(a.steps):
        x, y = next(loader)
        nxt = trainer.step_async(x, y)           # the loader keeps this buffer for one more batch: the copy is done by then
        if pending is not None:
            losses.append(pending.value())
        pending = nxt
    losses.append(pending.value())
    n_tokens = loader.num_tokens
    loader.close()
    print(f"{n_tokens} tokens | loss {losses[0]:.3f} -> {losses[-1]:.3f} over {len(losses)} steps")
    return losses


if __name__ == "__main__":
    main()
