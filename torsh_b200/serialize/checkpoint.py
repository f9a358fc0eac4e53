"""Training checkpoints.

* ``ModelCheckpoint`` / ``CheckpointManager``: ``{prefix}_epoch_{e}_step_{s}.torsh`` = gzip(level 6) of the bincode
  encoding of ``{state_dict: {name: [f32]}, parameter_shapes, metadata{model_name, model_version, torsh_version,
  timestamp, epoch, global_step, best_metric, custom}, optimizer_state{optimizer_type, learning_rate,
  momentum_states, velocity_states, step_counts, custom_state}, training_stats}``; ``{prefix}_best.torsh``; at most
  5 files are kept (``crates/torsh-nn/src/checkpoint.rs:24-157,204-207,354-438``).
* ``DistributedCheckpointManager``: ``checkpoint_step_{step}_rank_{rank}.json`` with ``TrainingCheckpoint{step, epoch,
  model_state, optimizer_state, scheduler_state, rng_states, loss, metrics, config, timestamp, version,
  distributed_meta{world_size, rank, dp_size, tp_size, pp_size, fsdp_sharding}}``, verified by re-loading after the
  write, latest = max step parsed from the file names, rotation (``crates/torsh-distributed/src/fault_tolerance.rs:
  91-135,214-409``). Sharded (FSDP / TP) states are written per rank and re-sharded on load when the world size changed.
"""
from __future__ import annotations

import gzip
import json
import re
import time
from pathlib import Path

import numpy as np
import torch

from ..core.error import TorshDistributedError, TorshError
from . import bincode

TORSH_VERSION = "0.1.3"


def _w_f32_map(w: bincode.Writer, d: dict):
    def vec(v):
        a = np.asarray(v, dtype="<f4").reshape(-1)
        w.varu(a.size)
        w.raw(a.tobytes())
    w.map(d, w.string, vec)


def _r_f32_map(r: bincode.Reader) -> dict:
    return r.map(r.string, lambda: np.frombuffer(r.raw(4 * r.varu()), dtype="<f4").copy())


def encode_checkpoint(ck: dict) -> bytes:
    w = bincode.Writer()
    _w_f32_map(w, ck["state_dict"])
    w.map(ck["parameter_shapes"], w.string, lambda s: w.seq(list(s), w.varu))
    m = ck["metadata"]
    w.string(m["model_name"]); w.string(m["model_version"]); w.string(m["torsh_version"]); w.varu(int(m["timestamp"]))
    w.varu(int(m["epoch"])); w.varu(int(m["global_step"]))
    w.option(m.get("best_metric"), w.f64)
    w.map(m.get("custom", {}), w.string, w.string)
    o = ck.get("optimizer_state")

    def opt(o):
        w.string(o["optimizer_type"]); w.f64(float(o["learning_rate"]))
        _w_f32_map(w, o.get("momentum_states", {})); _w_f32_map(w, o.get("velocity_states", {}))
        w.map(o.get("step_counts", {}), w.string, w.varu)
        w.map(o.get("custom_state", {}), w.string, w.string)
    w.option(o, opt)
    w.map(ck.get("training_stats", {}), w.string, w.f64)
    return gzip.compress(w.bytes(), compresslevel=6)


def decode_checkpoint(buf: bytes) -> dict:
    r = bincode.Reader(gzip.decompress(buf))
    ck = {"state_dict": _r_f32_map(r), "parameter_shapes": r.map(r.string, lambda: r.seq(r.varu))}
    ck["metadata"] = {"model_name": r.string(), "model_version": r.string(), "torsh_version": r.string(),
                      "timestamp": r.varu(), "epoch": r.varu(), "global_step": r.varu(),
                      "best_metric": r.option(r.f64), "custom": r.map(r.string, r.string)}

    def opt():
        return {"optimizer_type": r.string(), "learning_rate": r.f64(), "momentum_states": _r_f32_map(r),
                "velocity_states": _r_f32_map(r), "step_counts": r.map(r.string, r.varu),
                "custom_state": r.map(r.string, r.string)}
    ck["optimizer_state"] = r.option(opt)
    ck["training_stats"] = r.map(r.string, r.f64)
    return ck


def checkpoint_from(model: torch.nn.Module, optimizer=None, *, epoch: int = 0, global_step: int = 0,
                    best_metric: float | None = None, stats: dict | None = None, model_name: str | None = None) -> dict:
    sd = {n: p.detach().float().cpu().numpy().reshape(-1) for n, p in model.named_parameters()}
    shapes = {n: list(p.shape) for n, p in model.named_parameters()}
    ck = {"state_dict": sd, "parameter_shapes": shapes,
          "metadata": {"model_name": model_name or type(model).__name__, "model_version": "1.0.0",
                       "torsh_version": TORSH_VERSION, "timestamp": int(time.time()), "epoch": epoch,
                       "global_step": global_step, "best_metric": best_metric, "custom": {}},
          "optimizer_state": None, "training_stats": dict(stats or {})}
    if optimizer is not None:
        names = {id(p): n for n, p in model.named_parameters()}
        mom, vel, steps = {}, {}, {}
        for p, st in getattr(optimizer, "state", {}).items():
            n = names.get(id(p))
            if n is None:
                continue
            if "exp_avg" in st:
                mom[n] = st["exp_avg"].float().cpu().numpy().reshape(-1)
            if "momentum_buffer" in st:
                mom[n] = st["momentum_buffer"].float().cpu().numpy().reshape(-1)
            if "exp_avg_sq" in st:
                vel[n] = st["exp_avg_sq"].float().cpu().numpy().reshape(-1)
            if "step" in st:
                steps[n] = int(st["step"])
        ck["optimizer_state"] = {"optimizer_type": type(optimizer).__name__, "learning_rate": optimizer.param_groups[0]["lr"],
                                 "momentum_states": mom, "velocity_states": vel, "step_counts": steps, "custom_state": {}}
    return ck


def restore_into(ck: dict, model: torch.nn.Module, optimizer=None, strict: bool = True) -> None:
    own = dict(model.named_parameters())
    missing = [k for k in own if k not in ck["state_dict"]]
    unexpected = [k for k in ck["state_dict"] if k not in own]
    if strict and (missing or unexpected):
        raise TorshError.invalid_argument(f"checkpoint mismatch: missing {missing}, unexpected {unexpected}")
    with torch.no_grad():
        for n, p in own.items():
            if n in ck["state_dict"]:
                p.copy_(torch.from_numpy(np.asarray(ck["state_dict"][n])).reshape(ck["parameter_shapes"][n]).to(p.dtype))
    o = ck.get("optimizer_state")
    if optimizer is not None and o is not None:
        for g in optimizer.param_groups:
            g["lr"] = o["learning_rate"]
        for n, p in own.items():
            st = optimizer.state[p]
            if n in o["momentum_states"]:
                key = "momentum_buffer" if o["optimizer_type"] == "SGD" else "exp_avg"
                st[key] = torch.from_numpy(o["momentum_states"][n]).reshape(p.shape).to(p.device)
            if n in o["velocity_states"]:
                st["exp_avg_sq"] = torch.from_numpy(o["velocity_states"][n]).reshape(p.shape).to(p.device)
            if n in o["step_counts"]:
                st["step"] = torch.tensor(float(o["step_counts"][n]))


class CheckpointManager:
    def __init__(self, directory, prefix: str = "checkpoint", max_to_keep: int = 5, mode: str = "min"):
        self.dir, self.prefix, self.max_to_keep, self.mode = Path(directory), prefix, max_to_keep, mode
        self.dir.mkdir(parents=True, exist_ok=True)
        self.best = None

    def path(self, epoch, step) -> Path:
        return self.dir / f"{self.prefix}_epoch_{epoch}_step_{step}.torsh"

    def save(self, model, optimizer=None, *, epoch=0, global_step=0, metric: float | None = None, stats=None) -> Path:
        ck = checkpoint_from(model, optimizer, epoch=epoch, global_step=global_step, best_metric=metric, stats=stats)
        blob = encode_checkpoint(ck)
        p = self.path(epoch, global_step)
        p.write_bytes(blob)
        if metric is not None and (self.best is None or (metric < self.best if self.mode == "min" else metric > self.best)):
            self.best = metric
            (self.dir / f"{self.prefix}_best.torsh").write_bytes(blob)
        self._rotate()
        return p

    def _files(self):
        pat = re.compile(rf"{re.escape(self.prefix)}_epoch_(\d+)_step_(\d+)\.torsh$")
        out = []
        for f in self.dir.iterdir():
            m = pat.match(f.name)
            if m:
                out.append((int(m.group(2)), int(m.group(1)), f))
        return sorted(out)

    def _rotate(self):
        files = self._files()
        for _, _, f in files[:-self.max_to_keep] if len(files) > self.max_to_keep else []:
            f.unlink()

    def latest(self) -> Path | None:
        files = self._files()
        return files[-1][2] if files else None

    def load(self, path=None) -> dict:
        path = Path(path) if path else self.latest()
        if path is None:
            raise TorshError.io_error("no checkpoint found")
        return decode_checkpoint(path.read_bytes())


class DistributedCheckpointManager:
    def __init__(self, directory, rank: int = 0, world_size: int = 1, max_to_keep: int = 5, dp_size=1, tp_size=1, pp_size=1,
                 fsdp_sharding: bool = False):
        self.dir, self.rank, self.world, self.max_to_keep = Path(directory), rank, world_size, max_to_keep
        self.mesh = dict(dp_size=dp_size, tp_size=tp_size, pp_size=pp_size, fsdp_sharding=fsdp_sharding)
        self.dir.mkdir(parents=True, exist_ok=True)

    def _path(self, step, rank=None) -> Path:
        return self.dir / f"checkpoint_step_{step}_rank_{self.rank if rank is None else rank}.json"

    @staticmethod
    def _enc(t):
        if isinstance(t, torch.Tensor):
            return {"__tensor__": True, "dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape),
                    "data": t.detach().float().cpu().reshape(-1).tolist()}
        if isinstance(t, dict):
            return {str(k): DistributedCheckpointManager._enc(v) for k, v in t.items()}
        if isinstance(t, (list, tuple)):
            return [DistributedCheckpointManager._enc(v) for v in t]
        return t

    @staticmethod
    def _dec(o):
        if isinstance(o, dict) and o.get("__tensor__"):
            return torch.tensor(o["data"], dtype=torch.float32).reshape(o["shape"]).to(getattr(torch, o["dtype"]))
        if isinstance(o, dict):
            return {k: DistributedCheckpointManager._dec(v) for k, v in o.items()}
        if isinstance(o, list):
            return [DistributedCheckpointManager._dec(v) for v in o]
        return o

    def save(self, step: int, epoch: int, model_state: dict, optimizer_state: dict | None = None, scheduler_state=None,
             loss: float = 0.0, metrics: dict | None = None, config: dict | None = None) -> Path:
        doc = {"step": step, "epoch": epoch, "model_state": self._enc(model_state), "optimizer_state": self._enc(optimizer_state or {}),
               "scheduler_state": self._enc(scheduler_state or {}),
               "rng_states": {"torch": torch.get_rng_state().tolist()}, "loss": loss, "metrics": metrics or {}, "config": config or {},
               "timestamp": int(time.time()), "version": TORSH_VERSION,
               "distributed_meta": {"world_size": self.world, "rank": self.rank, "process_group_info": "world", **self.mesh}}
        p = self._path(step)
        tmp = p.with_suffix(".tmp")
        tmp.write_text(json.dumps(doc, indent=2))
        tmp.replace(p)
        try:  # verify-after-save
            back = json.loads(p.read_text())
            assert back["step"] == step and back["distributed_meta"]["rank"] == self.rank
        except Exception as e:
            raise TorshDistributedError.checkpoint_error(f"verification of {p} failed: {e}") from e
        self._rotate()
        return p

    def steps(self) -> list[int]:
        pat = re.compile(rf"checkpoint_step_(\d+)_rank_{self.rank}\.json$")
        return sorted(int(m.group(1)) for f in self.dir.iterdir() if (m := pat.match(f.name)))

    def latest_step(self) -> int | None:
        s = self.steps()
        return s[-1] if s else None

    def _rotate(self):
        s = self.steps()
        for step in s[:-self.max_to_keep] if len(s) > self.max_to_keep else []:
            self._path(step).unlink(missing_ok=True)

    def load(self, step: int | None = None, rank: int | None = None) -> dict:
        step = self.latest_step() if step is None else step
        if step is None:
            raise TorshDistributedError.checkpoint_error("no checkpoint found")
        try:
            doc = json.loads(self._path(step, rank).read_text())
        except (OSError, json.JSONDecodeError) as e:
            raise TorshDistributedError.checkpoint_error(f"cannot read checkpoint for step {step}: {e}") from e
        for k in ("model_state", "optimizer_state", "scheduler_state"):
            doc[k] = self._dec(doc[k])
        return doc

    def load_resharded_flat(self, step: int, key: str, old_world: int) -> torch.Tensor:
        """Concatenates the flat shard ``model_state[key]`` of every old rank and returns this rank's slice for
        the current world size (FSDP flat-shard resharding)."""
        full = torch.cat([self.load(step, r)["model_state"][key].reshape(-1) for r in range(old_world)])
        n = full.numel() // self.world
        return full[self.rank * n:(self.rank + 1) * n].clone()
