"""Optimizer checkpoints (``crates/torsh-optim/src/checkpointing.rs:9-60,97-200``): files
``checkpoint_step_{n}.bin`` hold the bincode encoding of ``Checkpoint{metadata{step, timestamp, loss, learning_rate,
epoch, gradient_norm, model_hash}, optimizer_state: Option<bytes>, gradients: Option<map<str, Vec<f32>>>,
model_parameters: Option<map<str, Vec<f32>>>}`` (the reference's "compression" step is the identity, so the bytes on
disk are the plain encoding).  The manager saves every ``checkpoint_frequency`` steps, keeps ``max_checkpoints`` files and
finds existing ones on start-up."""
from __future__ import annotations

import hashlib
import re
import struct
import time
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..serialize import bincode


@dataclass
class CheckpointConfig:
    checkpoint_dir: str = "checkpoints"
    max_checkpoints: int = 5
    checkpoint_frequency: int = 1000
    save_optimizer_state: bool = True
    save_gradients: bool = False
    compress: bool = True
    async_save: bool = True


def _w_f32_vec(w, v):
    a = np.asarray(v, dtype="<f4").reshape(-1)
    w.varu(a.size)
    w.raw(a.tobytes())


def _r_f32_vec(r):
    n = r.varu()
    return np.frombuffer(r.raw(4 * n), dtype="<f4").copy()


def encode(ck: dict) -> bytes:
    w = bincode.Writer()
    m = ck["metadata"]
    w.varu(m["step"]); w.varu(m["timestamp"])
    w.option(m.get("loss"), w.f32); w.f32(m["learning_rate"]); w.option(m.get("epoch"), w.varu)
    w.option(m.get("gradient_norm"), w.f32); w.option(m.get("model_hash"), w.string)
    w.option(ck.get("optimizer_state"), lambda b: (w.varu(len(b)), w.raw(bytes(b))))
    for key in ("gradients", "model_parameters"):
        w.option(ck.get(key), lambda d: w.map(d, w.string, lambda v: _w_f32_vec(w, v)))
    return bytes(w.b)


def decode(buf: bytes) -> dict:
    r = bincode.Reader(buf)
    meta = {"step": r.varu(), "timestamp": r.varu(), "loss": r.option(r.f32), "learning_rate": r.f32(),
            "epoch": r.option(r.varu), "gradient_norm": r.option(r.f32), "model_hash": r.option(r.string)}
    state = r.option(lambda: r.raw(r.varu()))
    grads = r.option(lambda: r.map(r.string, lambda: _r_f32_vec(r)))
    params = r.option(lambda: r.map(r.string, lambda: _r_f32_vec(r)))
    return {"metadata": meta, "optimizer_state": state, "gradients": grads, "model_parameters": params}


def pack_optimizer_state(opt: torch.optim.Optimizer) -> bytes:
    """Flat little-endian record of every fp32 state tensor: ``count | (group, index, key, numel, data)*`` plus ``step``."""
    w = bincode.Writer()
    items = []
    for gi, g in enumerate(opt.param_groups):
        for pi, p in enumerate(g["params"]):
            for k, v in opt.state.get(p, {}).items():
                if isinstance(v, torch.Tensor):
                    items.append((gi, pi, k, v.detach().float().cpu().reshape(-1).numpy()))
                elif isinstance(v, (int, float)):
                    items.append((gi, pi, k, np.asarray([v], dtype="<f4")))
    w.varu(len(items))
    for gi, pi, k, a in items:
        w.varu(gi); w.varu(pi); w.string(k); _w_f32_vec(w, a)
    return bytes(w.b)


def unpack_optimizer_state(opt: torch.optim.Optimizer, blob: bytes) -> None:
    r = bincode.Reader(blob)
    for _ in range(r.varu()):
        gi, pi, k, a = r.varu(), r.varu(), r.string(), _r_f32_vec(r)
        p = opt.param_groups[gi]["params"][pi]
        st = opt.state[p]
        cur = st.get(k)
        if isinstance(cur, torch.Tensor) and cur.numel() == a.size:
            cur.copy_(torch.from_numpy(a).reshape(cur.shape).to(cur.dtype))
        elif a.size == 1 and (cur is None or not isinstance(cur, torch.Tensor) or cur.numel() == 1):
            st[k] = torch.tensor(float(a[0])) if k == "step" else float(a[0])
        else:
            st[k] = torch.from_numpy(a).reshape(p.shape).to(p.device)


class OptimizerCheckpointManager:
    def __init__(self, config: CheckpointConfig | None = None):
        self.cfg = config or CheckpointConfig()
        self.dir = Path(self.cfg.checkpoint_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.current_step, self.last_checkpoint_step = 0, 0
        self.checkpoints: list[tuple[Path, int]] = sorted(
            ((f, int(m.group(1))) for f in self.dir.iterdir() if (m := re.match(r"checkpoint_step_(\d+)\.bin$", f.name))),
            key=lambda t: t[1])
        if self.checkpoints:
            self.last_checkpoint_step = self.checkpoints[-1][1]

    def step(self) -> None:
        self.current_step += 1

    def should_checkpoint(self) -> bool:
        return self.current_step > 0 and self.current_step - self.last_checkpoint_step >= self.cfg.checkpoint_frequency

    def save(self, model: torch.nn.Module | None = None, optimizer=None, loss: float | None = None,
             learning_rate: float | None = None, epoch: int | None = None) -> Path:
        params = grads = None
        gnorm = mhash = None
        if model is not None:
            params = {n: p.detach().float().cpu().reshape(-1).numpy() for n, p in model.named_parameters()}
            h = hashlib.sha256()
            for n in sorted(params):
                h.update(n.encode()); h.update(params[n].tobytes())
            mhash = h.hexdigest()[:16]
            if self.cfg.save_gradients:
                grads = {n: p.grad.detach().float().cpu().reshape(-1).numpy() for n, p in model.named_parameters() if p.grad is not None}
            sq = [p.grad.detach().float().pow(2).sum() for p in model.parameters() if p.grad is not None]
            gnorm = float(torch.stack(sq).sum().sqrt()) if sq else None
        lr = learning_rate if learning_rate is not None else (optimizer.param_groups[0]["lr"] if optimizer is not None else 0.0)
        ck = {"metadata": {"step": self.current_step, "timestamp": int(time.time()), "loss": loss, "learning_rate": lr,
                           "epoch": epoch, "gradient_norm": gnorm, "model_hash": mhash},
              "optimizer_state": pack_optimizer_state(optimizer) if (optimizer is not None and self.cfg.save_optimizer_state) else None,
              "gradients": grads, "model_parameters": params}
        path = self.dir / f"checkpoint_step_{self.current_step}.bin"
        path.write_bytes(encode(ck))
        self.checkpoints.append((path, self.current_step))
        self.last_checkpoint_step = self.current_step
        while len(self.checkpoints) > self.cfg.max_checkpoints:
            old, _ = self.checkpoints.pop(0)
            old.unlink(missing_ok=True)
        return path

    def load_latest(self) -> dict | None:
        return decode(self.checkpoints[-1][0].read_bytes()) if self.checkpoints else None

    def restore(self, ck: dict, model: torch.nn.Module | None = None, optimizer=None) -> None:
        if model is not None and ck.get("model_parameters"):
            with torch.no_grad():
                for n, p in model.named_parameters():
                    if n in ck["model_parameters"]:
                        p.copy_(torch.from_numpy(ck["model_parameters"][n]).reshape(p.shape).to(p.dtype))
        if optimizer is not None and ck.get("optimizer_state"):
            unpack_optimizer_state(optimizer, ck["optimizer_state"])
        self.current_step = ck["metadata"]["step"]

    def statistics(self) -> dict:
        return {"total_checkpoints": len(self.checkpoints), "total_size_bytes": sum(f.stat().st_size for f, _ in self.checkpoints),
                "current_step": self.current_step, "last_checkpoint_step": self.last_checkpoint_step,
                "next_checkpoint_step": self.last_checkpoint_step + self.cfg.checkpoint_frequency}
