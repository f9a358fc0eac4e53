"""Training checkpoints.

* ``ModelCheckpoint`` / ``CheckpointManager``: ``{prefix}_epoch_{e}_step_{s}.torsh`` (default prefix ``model``) =
  gzip(level 6) of the bincode encoding of ``{state_dict: {name: [f32]}, parameter_shapes, metadata{model_name,
  model_version, torsh_version, timestamp: RFC 3339 string, epoch?, global_step?, best_metric?, custom},
  optimizer_state?{optimizer_type, learning_rate, momentum_states, velocity_states, step_counts, custom_state: {name:
  [f32]}}, training_stats?{six f64 histories, custom_metrics}}`` with the field types of the reference struct;
  ``{prefix}_best.torsh``; at most 5 files are kept (``crates/torsh-nn/src/checkpoint.rs:24-157,204-207,354-438``).
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


def _w_f32_vec(w: bincode.Writer, v):
    a = np.asarray(v, dtype="<f4").reshape(-1)
    w.varu(a.size)
    w.raw(a.tobytes())


def _w_f32_map(w: bincode.Writer, d: dict):
    w.map(d, w.string, lambda v: _w_f32_vec(w, v))


def _r_f32_vec(r: bincode.Reader):
    return np.frombuffer(r.raw(4 * r.varu()), dtype="<f4").copy()


def _r_f32_map(r: bincode.Reader) -> dict:
    return r.map(r.string, lambda: _r_f32_vec(r))


_STATS_LISTS = ("train_losses", "val_losses", "train_accuracies", "val_accuracies", "learning_rates", "epoch_durations")


def _rfc3339(ts) -> str:
    if isinstance(ts, str):
        return ts
    return time.strftime("%Y-%m-%dT%H:%M:%S", time.gmtime(float(ts))) + "+00:00"


def encode_checkpoint(ck: dict) -> bytes:
    """``ModelCheckpoint`` in the field order and types of ``crates/torsh-nn/src/checkpoint.rs:24-113``:
    ``state_dict: HashMap<String, Vec<f32>>``, ``parameter_shapes: HashMap<String, Vec<usize>>``, ``metadata``
    (``timestamp: String`` in RFC 3339, ``epoch`` / ``global_step: Option<usize>``, ``best_metric: Option<f64>``,
    ``custom: HashMap<String, String>``), ``optimizer_state: Option<OptimizerState>`` (``custom_state:
    HashMap<String, Vec<f32>>``) and ``training_stats: Option<TrainingStats>`` (six ``Vec<f64>`` and
    ``custom_metrics: HashMap<String, Vec<f64>>``), bincode "standard" configuration, then gzip level 6. Map entries
    are written in key order (any order decodes)."""
    w = bincode.Writer()
    _w_f32_map(w, ck["state_dict"])
    w.map(ck["parameter_shapes"], w.string, lambda s: w.seq(list(s), w.varu))
    m = ck["metadata"]
    w.string(m["model_name"]); w.string(m["model_version"]); w.string(m["torsh_version"]); w.string(_rfc3339(m["timestamp"]))
    w.option(m.get("epoch"), lambda v: w.varu(int(v)))
    w.option(m.get("global_step"), lambda v: w.varu(int(v)))
    w.option(m.get("best_metric"), w.f64)
    w.map(m.get("custom", {}), w.string, w.string)

    def opt(o):
        w.string(o["optimizer_type"]); w.f64(float(o["learning_rate"]))
        _w_f32_map(w, o.get("momentum_states", {})); _w_f32_map(w, o.get("velocity_states", {}))
        w.map(o.get("step_counts", {}), w.string, w.varu)
        _w_f32_map(w, o.get("custom_state", {}))
    w.option(ck.get("optimizer_state"), opt)

    def stats(t):
        for k in _STATS_LISTS:
            w.seq([float(x) for x in t.get(k, [])], w.f64)
        w.map(t.get("custom_metrics", {}), w.string, lambda v: w.seq([float(x) for x in v], w.f64))
    w.option(ck.get("training_stats"), stats)
    return gzip.compress(w.bytes(), compresslevel=6)


def decode_checkpoint(buf: bytes) -> dict:
    r = bincode.Reader(gzip.decompress(buf))
    ck = {"state_dict": _r_f32_map(r), "parameter_shapes": r.map(r.string, lambda: r.seq(r.varu))}
    ck["metadata"] = {"model_name": r.string(), "model_version": r.string(), "torsh_version": r.string(),
                      "timestamp": r.string(), "epoch": r.option(r.varu), "global_step": r.option(r.varu),
                      "best_metric": r.option(r.f64), "custom": r.map(r.string, r.string)}

    def opt():
        return {"optimizer_type": r.string(), "learning_rate": r.f64(), "momentum_states": _r_f32_map(r),
                "velocity_states": _r_f32_map(r), "step_counts": r.map(r.string, r.varu),
                "custom_state": _r_f32_map(r)}
    ck["optimizer_state"] = r.option(opt)

    def stats():
        t = {k: r.seq(r.f64) for k in _STATS_LISTS}
        t["custom_metrics"] = r.map(r.string, lambda: r.seq(r.f64))
        return t
    ck["training_stats"] = r.option(stats)
    return ck


def _flat_optimizer_state(model: torch.nn.Module, optimizer) -> dict | None:
    """``OptimizerState`` of the flat fused optimizers (:class:`FlatAdamW` and the FSDP variants): per-parameter slices
    of the moments, plus the fp32 master weights under ``custom_state["master.<name>"]`` and the step count."""
    flat = getattr(optimizer, "flat", None)
    if flat is None or not hasattr(flat, "offsets") or not hasattr(flat, "exp_avg"):
        return None
    names = {id(p): n for n, p in model.named_parameters()}
    mom, vel, steps, custom = {}, {}, {}, {}
    for p, o in zip(flat.params, flat.offsets):
        n = names.get(id(p))
        if n is None:
            continue
        k = p.numel()
        mom[n] = flat.exp_avg[o:o + k].detach().float().cpu().numpy()
        vel[n] = flat.exp_avg_sq[o:o + k].detach().float().cpu().numpy()
        custom["master." + n] = flat.master[o:o + k].detach().float().cpu().numpy()
        steps[n] = int(optimizer.step_count)
    return {"optimizer_type": type(optimizer).__name__, "learning_rate": optimizer.param_groups[0]["lr"],
            "momentum_states": mom, "velocity_states": vel, "step_counts": steps, "custom_state": custom}


def checkpoint_from(model: torch.nn.Module, optimizer=None, *, epoch: int = 0, global_step: int = 0,
                    best_metric: float | None = None, stats: dict | None = None, model_name: str | None = None) -> dict:
    sd = {n: p.detach().float().cpu().numpy().reshape(-1) for n, p in model.named_parameters()}
    shapes = {n: list(p.shape) for n, p in model.named_parameters()}
    ck = {"state_dict": sd, "parameter_shapes": shapes,
          "metadata": {"model_name": model_name or type(model).__name__, "model_version": "1.0.0",
                       "torsh_version": TORSH_VERSION, "timestamp": _rfc3339(time.time()), "epoch": epoch,
                       "global_step": global_step, "best_metric": best_metric, "custom": {}},
          "optimizer_state": None, "training_stats": _as_training_stats(stats)}
    flat_state = _flat_optimizer_state(model, optimizer) if optimizer is not None else None
    if flat_state is not None:
        ck["optimizer_state"] = flat_state
    elif optimizer is not None:
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


def _as_training_stats(stats) -> dict | None:
    """Accepts the reference's ``TrainingStats`` layout or a plain ``{metric: value}`` map (stored as one-element
    ``custom_metrics`` histories)."""
    if not stats:
        return None
    if any(k in stats for k in _STATS_LISTS) or "custom_metrics" in stats:
        return {**{k: list(stats.get(k, [])) for k in _STATS_LISTS}, "custom_metrics": dict(stats.get("custom_metrics", {}))}
    return {**{k: [] for k in _STATS_LISTS},
            "custom_metrics": {k: (list(v) if isinstance(v, (list, tuple)) else [float(v)]) for k, v in stats.items()}}


def _restore_flat(ck: dict, model: torch.nn.Module, optimizer) -> bool:
    """Restore into a flat fused optimizer: master weights first, then the bf16 copy from them, then the moments and
    the step count. Returns False when ``optimizer`` is not a flat optimizer."""
    flat = getattr(optimizer, "flat", None)
    if flat is None or not hasattr(flat, "offsets") or not hasattr(flat, "exp_avg"):
        return False
    o = ck.get("optimizer_state") or {}
    names = {id(p): n for n, p in model.named_parameters()}
    dev = flat.master.device
    with torch.no_grad():
        for p, off in zip(flat.params, flat.offsets):
            n = names.get(id(p))
            if n is None:
                continue
            k = p.numel()
            src = o.get("custom_state", {}).get("master." + n)
            if src is None and n in ck["state_dict"]:
                src = ck["state_dict"][n]
            if src is not None:
                flat.master[off:off + k].copy_(torch.from_numpy(np.asarray(src, dtype=np.float32)).to(dev))
                flat.lowp[off:off + k].copy_(flat.master[off:off + k])
            if n in o.get("momentum_states", {}):
                flat.exp_avg[off:off + k].copy_(torch.from_numpy(np.asarray(o["momentum_states"][n])).to(dev))
            if n in o.get("velocity_states", {}):
                flat.exp_avg_sq[off:off + k].copy_(torch.from_numpy(np.asarray(o["velocity_states"][n])).to(dev))
    if o.get("step_counts"):
        optimizer.step_count = int(max(o["step_counts"].values()))
    if "learning_rate" in o:
        optimizer.set_lr(o["learning_rate"])
    return True


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
    if optimizer is not None and _restore_flat(ck, model, optimizer):
        return
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
    def __init__(self, directory, prefix: str = "model", max_to_keep: int = 5, mode: str = "min"):
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
