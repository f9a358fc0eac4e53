"""Tensor and model serialization + training checkpoints (roles of ``tensor_serialization_demo.rs``,
``model_checkpointing.rs``, ``training_with_checkpoints.rs``).

  python examples/checkpointing.py [directory]"""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

import torsh_b200 as tb
from torsh_b200.serialize import model_state as ms
from torsh_b200.serialize import trsh
from torsh_b200.serialize.checkpoint import CheckpointManager, restore_into


def main(argv=None):
    out = (argv or sys.argv[1:] or [tempfile.mkdtemp()])[0]
    os.makedirs(out, exist_ok=True)
    # 1. a tensor in the TRSH container (header + bincode metadata + CRC-32, optional zstd)
    t = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)
    blob = trsh.encode_trsh(t)
    back, _meta = trsh.decode_trsh(blob)
    assert torch.equal(back, t)
    trsh.save_tensor(t, os.path.join(out, "tensor.trsh"))
    assert torch.equal(trsh.load_tensor(os.path.join(out, "tensor.trsh")), t)
    print(f"TRSH: {len(blob)} bytes for a {tuple(t.shape)} f32 tensor")
    # 2. a model state in JSON / binary / safetensors
    model = tb.models.create_model("gpt2-tiny")
    st = ms.model_state(model, architecture="gpt2-tiny")
    for name, save, load in (("json", ms.save_json, ms.load_json), ("trsm", ms.save_binary, ms.load_binary),
                             ("safetensors", ms.save_safetensors, ms.load_safetensors)):
        path = os.path.join(out, f"model.{name}")
        save(st, path)
        assert load(path)["parameters"].keys() == st["parameters"].keys()
        print(f"{name}: {os.path.getsize(path)} bytes")
    # 3. training checkpoints with rotation and resume
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    mgr = CheckpointManager(os.path.join(out, "ckpt"), max_to_keep=2)
    ids = torch.randint(0, model.config.vocab_size, (2, 33))
    for step in range(1, 4):
        loss = model(ids[:, :-1], targets=ids[:, 1:]) if hasattr(model, "forward") else None
        opt.zero_grad(); loss.backward(); opt.step()
        mgr.save(model, opt, global_step=step, metric=loss.item())
    fresh = tb.models.create_model("gpt2-tiny")
    ck = mgr.load()
    restore_into(ck, fresh, strict=True)
    same = all(torch.allclose(a, b) for a, b in zip(model.parameters(), fresh.parameters()))
    print(f"resumed step {ck['metadata']['global_step']}, parameters equal: {same}, files kept: {len(list(mgr.dir.glob('*.torsh')))}")
    return same


if __name__ == "__main__":
    main()
