"""Command line (``crates/torsh-cli/src/main.rs:69-108``): ``python -m torsh_b200.cli <command>`` with the reference's
command tree — ``model`` / ``train`` / ``dataset`` / ``benchmark`` / ``hub`` / ``dev`` / ``info`` / ``init`` /
``update`` / ``completions``.  Configuration comes from ``--config`` or the ``TORSH_CONFIG`` environment variable
(JSON, YAML or TOML; sections ``general``, ``model``, ``training``, ``hub``, ``benchmark``, ``dev`` as in
``crates/torsh-cli/src/config.rs``).  Where the reference's ``train`` command steps a mock loop over host arrays, this
one builds a model from the registry and trains it through :class:`torsh_b200.engine.CausalLMTrainer` (language models)
or a plain optimizer loop, writing checkpoints with ``serialize.CheckpointManager``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

DEFAULT_CONFIG = {
    "general": {"output_dir": "./outputs", "cache_dir": "~/.cache/torsh", "default_device": "cuda", "num_workers": 4,
                "memory_limit_gb": None, "show_progress": True, "default_dtype": "bf16"},
    "model": {"default_format": "trsh"},
    "training": {"epochs": 1, "batch_size": 8, "learning_rate": 3e-4, "checkpoint_every": 100, "mixed_precision": True},
    "hub": {"cache_dir": "~/.cache/torsh/hub", "url": None},
    "benchmark": {"iterations": 20, "warmup": 3},
    "dev": {"template_dir": None},
}


def load_config(path: str | None) -> dict:
    cfg = json.loads(json.dumps(DEFAULT_CONFIG))
    path = path or os.environ.get("TORSH_CONFIG")
    if not path:
        return cfg
    text = Path(path).read_text()
    if path.endswith((".yaml", ".yml")):
        import yaml
        user = yaml.safe_load(text) or {}
    elif path.endswith(".toml"):
        import tomllib
        user = tomllib.loads(text)
    else:
        user = json.loads(text)
    for sec, vals in user.items():
        cfg.setdefault(sec, {}).update(vals if isinstance(vals, dict) else {})
    return cfg


def _emit(obj, as_json: bool):
    if as_json:
        print(json.dumps(obj, indent=1, default=str))
        return
    if isinstance(obj, dict):
        w = max((len(str(k)) for k in obj), default=0)
        for k, v in obj.items():
            print(f"{str(k):<{w}}  {v}")
    elif isinstance(obj, list):
        for v in obj:
            print(v)
    else:
        print(obj)


def _device(name: str | None, cfg: dict):
    import torch
    name = name or cfg["general"]["default_device"]
    if name.startswith("cuda") and not torch.cuda.is_available():
        name = "cpu"
    return torch.device(name)


def _t(v):
    """Tensor of a model-state entry (``{"shape", "dtype", "data"}``) or of anything tensor-like."""
    import torch
    if isinstance(v, dict):
        return torch.tensor(v["data"], dtype=torch.float32).reshape(v["shape"])
    return torch.as_tensor(v)


def _entry(t) -> dict:
    t = t.detach().float().cpu()
    return {"shape": list(t.shape), "dtype": "f32", "data": t.reshape(-1).tolist(), "requires_grad": True}


def _load_state(path: str) -> dict:
    from .serialize import model_state as ms
    p = str(path)
    if p.endswith(".json"):
        return ms.load_json(p)
    if p.endswith(".safetensors"):
        return ms.load_safetensors(p)
    if p.endswith((".pt", ".pth")):
        import torch
        sd = torch.load(p, map_location="cpu", weights_only=True)
        return {"parameters": {k: _entry(v) for k, v in sd.items()}, "config": {}, "metadata": {"architecture": "unknown"}}
    return ms.load_binary(p)


def _save_state(state: dict, path: str) -> None:
    from .serialize import model_state as ms
    p = str(path)
    if p.endswith(".json"):
        ms.save_json(state, p)
    elif p.endswith(".safetensors"):
        ms.save_safetensors(state, p)
    elif p.endswith((".pt", ".pth")):
        import torch
        dt = state.get("_torch_dtype")
        torch.save({k: _t(v).to(dt) if dt else _t(v) for k, v in state["parameters"].items()}, p)
    else:
        ms.save_binary(state, p)


# ----------------------------------------------------------------------------------------------- model

def cmd_model(a, cfg):
    import torch
    from . import models
    if a.action == "list":
        return models.list_models()
    if a.action == "create":
        from .serialize.model_state import model_state
        m = models.create_model(a.name)
        _save_state(model_state(m, architecture=a.name), a.output)
        return {"saved": a.output, "parameters": sum(p.numel() for p in m.parameters())}
    if a.action == "inspect":
        if a.path in models.list_models():
            from .nn.summary import summary
            return summary(models.create_model(a.path))
        st = _load_state(a.path)
        params = st["parameters"]
        total = sum(int(_t(v).numel()) for v in params.values())
        rows = {k: f"{tuple(_t(v).shape)} {v.get('dtype', 'f32') if isinstance(v, dict) else _t(v).dtype}"
                for k, v in list(params.items())[: a.limit]}
        return {"architecture": st.get("metadata", {}).get("architecture"), "tensors": len(params), "parameters": total,
                "size_mb": round(total * 4 / 2**20, 2), **rows}
    if a.action == "convert":
        st = _load_state(a.path)
        if a.dtype:
            # the TRSM / JSON / safetensors model-state formats hold f32 only (as in the reference); a narrower
            # dtype rounds the values through it and, for a .pt output, is also the stored dtype
            dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[a.dtype]
            st["parameters"] = {k: _entry(_t(v).to(dt)) for k, v in st["parameters"].items()}
            st["_torch_dtype"] = dt
        if not str(a.output).endswith((".pt", ".pth")):
            st.pop("_torch_dtype", None)
        _save_state(st, a.output)
        return {"converted": a.path, "to": a.output}
    if a.action == "validate":
        st = _load_state(a.path)
        bad = [k for k, v in st["parameters"].items() if not torch.isfinite(_t(v).float()).all()]
        return {"tensors": len(st["parameters"]), "non_finite": bad, "valid": not bad}
    if a.action == "quantize":
        from . import quantization as Q
        st = _load_state(a.path)
        out, report = {}, {}
        for k, v in st["parameters"].items():
            v = _t(v)
            if v.dim() >= 2 and v.is_floating_point():
                q, qp = Q.quantize_per_channel(v.float(), 0, a.bits)
                report[k] = round(Q.sqnr_db(v.float(), Q.dequantize(q, qp)), 2)
                out[k + ".qweight"], out[k + ".scale"] = _entry(q), _entry(qp.scale)
            else:
                out[k] = _entry(v)
        st["parameters"] = out
        _save_state(st, a.output)
        return {"quantized": len(report), "min_sqnr_db": min(report.values(), default=None), "output": a.output}
    if a.action == "benchmark":
        from .utils import benchmark
        dev = _device(a.device, cfg)
        m = models.create_model(a.path).to(dev)
        if dev.type == "cuda":
            m = m.to(torch.bfloat16)
        x = _example_input(m, a.batch, a.seq, dev)
        with torch.no_grad():
            r = benchmark(lambda: m(x), warmup=cfg["benchmark"]["warmup"], iters=a.iters)
        return {"model": a.path, "device": str(dev), **r}
    if a.action == "prune":
        st = _load_state(a.path)
        kept = total = 0
        for k, v in st["parameters"].items():
            t = _t(v).float()
            if t.dim() >= 2:
                if a.structured:                                                   # whole output rows, smallest L2 norm first
                    norms = t.flatten(1).norm(dim=1)
                    n_drop = int(a.sparsity * len(norms))
                    mask = torch.ones_like(norms, dtype=torch.bool)
                    if n_drop:
                        mask[norms.argsort()[:n_drop]] = False
                    t = t * mask.reshape(-1, *[1] * (t.dim() - 1))
                else:
                    n_drop = int(a.sparsity * t.numel())
                    if n_drop:
                        t = t * (t.abs() > t.abs().flatten().kthvalue(n_drop).values)
                st["parameters"][k] = _entry(t)
                kept += int((t != 0).sum()); total += t.numel()
        _save_state(st, a.output)
        return {"pruned": a.path, "output": a.output, "sparsity": round(1 - kept / max(total, 1), 4), "structured": bool(a.structured)}
    if a.action == "optimize":
        # folds every "<prefix>.weight" / "<bn>.running_mean, running_var, weight, bias" pair named with --fold "conv=bn" and
        # drops buffers that inference does not need
        st = _load_state(a.path)
        params, folded = st["parameters"], []
        for pair in (a.fold or "").split(","):
            if "=" not in pair:
                continue
            conv, bn = pair.split("=")
            w, mean, var = _t(params[conv + ".weight"]).float(), _t(params[bn + ".running_mean"]).float(), _t(params[bn + ".running_var"]).float()
            g = _t(params[bn + ".weight"]).float() if bn + ".weight" in params else torch.ones_like(mean)
            beta = _t(params[bn + ".bias"]).float() if bn + ".bias" in params else torch.zeros_like(mean)
            b = _t(params[conv + ".bias"]).float() if conv + ".bias" in params else torch.zeros_like(mean)
            scale = g / torch.sqrt(var + 1e-5)
            params[conv + ".weight"] = _entry(w * scale.reshape(-1, *[1] * (w.dim() - 1)))
            params[conv + ".bias"] = _entry((b - mean) * scale + beta)
            for suffix in (".running_mean", ".running_var", ".weight", ".bias", ".num_batches_tracked"):
                params.pop(bn + suffix, None)
            folded.append(conv)
        dropped = [k for k in list(params) if k.endswith("num_batches_tracked")]
        for k in dropped:
            params.pop(k)
        _save_state(st, a.output)
        return {"optimized": a.path, "output": a.output, "folded": folded, "dropped": dropped}
    if a.action == "compress":
        import gzip
        raw = Path(a.path).read_bytes()
        Path(a.output).write_bytes(gzip.compress(raw, compresslevel=a.level))
        return {"compressed": a.path, "output": a.output, "bytes": len(raw), "compressed_bytes": Path(a.output).stat().st_size, "ratio": round(len(raw) / max(Path(a.output).stat().st_size, 1), 3)}
    if a.action == "extract":
        import fnmatch
        st = _load_state(a.path)
        pats = (a.pattern or "*").split(",")
        st["parameters"] = {k: v for k, v in st["parameters"].items() if any(fnmatch.fnmatch(k, p_) for p_ in pats)}
        if not st["parameters"]:
            raise SystemExit(f"no tensor matches {a.pattern!r}")
        _save_state(st, a.output)
        return {"extracted": len(st["parameters"]), "output": a.output, "names": sorted(st["parameters"])[: a.limit]}
    if a.action == "merge":
        paths = [a.path, *(a.others or [])]
        states = [_load_state(p_) for p_ in paths]
        weights = [float(w) for w in a.weights.split(",")] if a.weights else [1.0 / len(states)] * len(states)
        if len(weights) != len(states):
            raise SystemExit("one weight per model is required")
        keys = set(states[0]["parameters"])
        if any(set(s_["parameters"]) != keys for s_ in states[1:]):
            raise SystemExit("the models do not have the same tensors")
        merged = states[0]
        merged["parameters"] = {k: _entry(sum(w * _t(s_["parameters"][k]).float() for w, s_ in zip(weights, states))) for k in sorted(keys)}
        _save_state(merged, a.output)
        return {"merged": paths, "weights": weights, "output": a.output}
    raise SystemExit(f"unknown model action {a.action}")


def _example_input(m, batch, seq, dev):
    import torch
    cfg = getattr(m, "config", None)
    if cfg is not None and hasattr(cfg, "vocab_size"):
        return torch.randint(0, cfg.vocab_size, (batch, min(seq, getattr(cfg, "n_positions", seq))), device=dev)
    dt = next(m.parameters()).dtype
    return torch.randn(batch, 3, 224, 224, device=dev, dtype=dt)


# ----------------------------------------------------------------------------------------------- train

def _run_file(out: Path) -> Path:
    return out / "run.json"


def cmd_train(a, cfg):
    import torch
    out = Path(a.output or cfg["general"]["output_dir"])
    if a.action == "monitor":
        f = _run_file(out)
        return json.loads(f.read_text()) if f.exists() else {"status": "no run found", "dir": str(out)}
    if a.action == "stop":
        out.mkdir(parents=True, exist_ok=True)
        (out / "STOP").write_text("stop requested\n")
        return {"stop_requested": str(out / "STOP")}
    from . import models
    from .data import SyntheticTokenDataset
    from .serialize.checkpoint import CheckpointManager
    out.mkdir(parents=True, exist_ok=True)
    (out / "STOP").unlink(missing_ok=True)
    tc = cfg["training"]
    dev = _device(a.device, cfg)
    model = models.create_model(a.model, **(json.loads(a.model_args) if a.model_args else {})).to(dev)
    lm = hasattr(getattr(model, "config", None), "vocab_size")
    bs, lr = a.batch_size or tc["batch_size"], a.lr or tc["learning_rate"]
    mgr = CheckpointManager(out / "checkpoints", max_to_keep=3)
    step0 = 0
    if dev.type == "cuda" and lm:
        from .engine import CausalLMTrainer
        seq_len = min(a.seq, getattr(model.config, "n_positions", a.seq))
        trainer = CausalLMTrainer(model, lr=lr, batch_size=bs, seq_len=seq_len, use_graph=False)
        step_fn = lambda ids, tgt: trainer.step(ids, tgt)
        opt = trainer.opt   # flat fused AdamW: checkpoints carry its master weights, moments and step count
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=lr)

        def step_fn(x, y):
            logits = model(x)
            logits = logits[0] if isinstance(logits, tuple) else logits
            loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), y.reshape(-1))
            opt.zero_grad(set_to_none=True); loss.backward(); opt.step()
            return loss.item()
    if a.action == "resume":
        if mgr.latest() is not None:
            from .serialize.checkpoint import restore_into
            ck = mgr.load()
            restore_into(ck, model, opt, strict=False)
            step0 = ck["metadata"]["global_step"]
    seq = min(a.seq, getattr(model.config, "n_positions", a.seq)) if lm else a.seq
    host_batches = dev.type == "cuda" and lm   # the trainer copies each batch from (pinned) host memory itself
    if lm:
        ds = SyntheticTokenDataset(model.config.vocab_size, seq, a.steps * bs, seed=0)
    history, t0 = [], time.time()
    for step in range(step0, step0 + a.steps):
        if (out / "STOP").exists():
            break
        if lm:
            rows = [ds[(step - step0) * bs + i] for i in range(bs)]
            x = torch.stack([r[0] for r in rows]); y = torch.stack([r[1] for r in rows])
            x, y = (x.pin_memory(), y.pin_memory()) if host_batches else (x.to(dev), y.to(dev))
        else:
            x = torch.randn(bs, 3, a.image, a.image, device=dev); y = torch.randint(0, 10, (bs,), device=dev)
        loss = float(step_fn(x, y))
        history.append(loss)
        if (step + 1) % a.log_every == 0 or step + 1 == step0 + a.steps:
            _run_file(out).write_text(json.dumps({"status": "running", "step": step + 1, "loss": loss,
                                                  "elapsed_s": round(time.time() - t0, 2), "model": a.model}))
        if (step + 1) % tc["checkpoint_every"] == 0 or step + 1 == step0 + a.steps:
            mgr.save(model, opt, global_step=step + 1, metric=loss)
    res = {"status": "finished", "step": step0 + len(history), "first_loss": history[0] if history else None,
           "loss": history[-1] if history else None, "elapsed_s": round(time.time() - t0, 2), "model": a.model,
           "device": str(dev)}
    _run_file(out).write_text(json.dumps(res))
    return res


# ----------------------------------------------------------------------------------------------- dataset

def cmd_dataset(a, cfg):
    import torch
    if a.action == "download":
        # The reference fetches archives over HTTP; with no network a synthetic set of the same shape is written.
        shapes = {"mnist": ((1, 28, 28), 10), "cifar10": ((3, 32, 32), 10), "cifar100": ((3, 32, 32), 100)}
        if a.name not in shapes:
            raise SystemExit(f"dataset {a.name!r}: only synthetic {sorted(shapes)} are available offline")
        shp, nc = shapes[a.name]
        g = torch.Generator().manual_seed(0)
        Path(a.output).mkdir(parents=True, exist_ok=True)
        f = Path(a.output) / f"{a.name}_synthetic.pt"
        torch.save({"x": torch.rand(a.samples, *shp, generator=g), "y": torch.randint(0, nc, (a.samples,), generator=g)}, f)
        return {"written": str(f), "samples": a.samples, "synthetic": True}
    d = torch.load(a.path, weights_only=True)
    if a.action == "analyze":
        x, y = d["x"].float(), d["y"]
        return {"samples": len(y), "shape": tuple(x.shape[1:]), "mean": round(x.mean().item(), 4), "std": round(x.std().item(), 4),
                "classes": int(y.max()) + 1, "class_counts": torch.bincount(y).tolist()}
    if a.action == "split":
        n = len(d["y"])
        perm = torch.randperm(n, generator=torch.Generator().manual_seed(a.seed))
        cut = [int(n * a.train), int(n * (a.train + a.val))]
        Path(a.output).mkdir(parents=True, exist_ok=True)
        for name, idx in zip(("train", "val", "test"), (perm[: cut[0]], perm[cut[0]: cut[1]], perm[cut[1]:])):
            torch.save({k: v[idx] for k, v in d.items()}, Path(a.output) / f"{name}.pt")
        return {"train": cut[0], "val": cut[1] - cut[0], "test": n - cut[1]}
    if a.action == "preprocess":
        x = d["x"].float()
        mean, std = x.mean((0, 2, 3), keepdim=True), x.std((0, 2, 3), keepdim=True).clamp(min=1e-6)
        torch.save({"x": (x - mean) / std, "y": d["y"]}, a.output)
        return {"normalized": a.output, "mean": mean.flatten().tolist(), "std": std.flatten().tolist()}
    raise SystemExit(f"unknown dataset action {a.action}")


# ----------------------------------------------------------------------------------------------- benchmark

def cmd_benchmark(a, cfg):
    if a.action == "run":
        import torch
        from .utils import benchmark
        dev = _device(a.device, cfg)
        res = {}
        n = 4096 if dev.type == "cuda" else 256
        dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
        x, w = torch.randn(n, n, device=dev, dtype=dt), torch.randn(n, n, device=dev, dtype=dt)
        suites = {
            "ops": {"matmul": lambda: x @ w, "add": lambda: x + w, "gelu": lambda: torch.nn.functional.gelu(x),
                    "softmax": lambda: torch.softmax(x.float(), -1), "layer_norm": lambda: torch.nn.functional.layer_norm(x, (n,))},
            "memory": {"copy": lambda: x.clone(), "transpose": lambda: x.t().contiguous()},
        }
        if dev.type == "cuda":
            from . import ops
            suites["ops"].update({"tb_gemm": lambda: ops.gemm.matmul(x, w), "tb_gelu": lambda: ops.elementwise.gelu(x),
                                  "tb_layer_norm": lambda: ops.norm.layer_norm(x, torch.ones(n, device=dev, dtype=dt), None)})
        for suite, fns in suites.items():
            if a.suite not in ("all", suite):
                continue
            for name, fn in fns.items():
                res[f"{suite}.{name}"] = benchmark(fn, warmup=a.warmup, iters=a.iters)
        Path(a.output).parent.mkdir(parents=True, exist_ok=True)
        Path(a.output).write_text(json.dumps({"device": str(dev), "results": res}, indent=1))
        return {k: f"{v['median_ms']:.4f} ms" for k, v in res.items()}
    if a.action == "compare":
        base, new = (json.loads(Path(p).read_text())["results"] for p in (a.baseline, a.candidate))
        return {k: f"{base[k]['median_ms'] / new[k]['median_ms']:.2f}x" for k in base if k in new}
    if a.action == "report":
        r = json.loads(Path(a.results).read_text())
        lines = ["| benchmark | median ms | min ms |", "|---|---|---|"] + [
            f"| {k} | {v['median_ms']:.4f} | {v['min_ms']:.4f} |" for k, v in r["results"].items()]
        Path(a.output).write_text("\n".join(lines) + "\n")
        return {"report": a.output, "rows": len(r["results"])}
    raise SystemExit(f"unknown benchmark action {a.action}")


# ----------------------------------------------------------------------------------------------- hub / dev / misc

def cmd_hub(a, cfg):
    from . import hub
    reg = hub.LocalHub(os.path.expanduser(a.cache or cfg["hub"]["cache_dir"]))
    if a.action == "list":
        return reg.list()
    if a.action == "search":
        return reg.search(a.query)
    if a.action == "upload":
        return reg.publish(a.name, a.path, version=a.version)
    if a.action == "download":
        return {"path": str(reg.fetch(a.name, a.version, a.output))}
    raise SystemExit(f"unknown hub action {a.action}")


_TEMPLATES = {
    "model": '''"""{name}: a model defined with torsh_b200."""
import torch
import torsh_b200 as tb


class {cls}(torch.nn.Module):
    def __init__(self, width: int = 256, classes: int = 10):
        super().__init__()
        self.net = torch.nn.Sequential(tb.nn.Linear(width, width), torch.nn.GELU(), tb.nn.Linear(width, classes))

    def forward(self, x):
        return self.net(x)
''',
    "train": '''"""Training script for {name}."""
import torch
import torsh_b200 as tb

model = tb.models.create_model("gpt2")
trainer = tb.engine.CausalLMTrainer(model.cuda(), lr=3e-4)
''',
}


def cmd_dev(a, cfg):
    if a.action == "codegen":
        if a.template not in _TEMPLATES:
            raise SystemExit(f"templates: {sorted(_TEMPLATES)}")
        Path(a.output).mkdir(parents=True, exist_ok=True)
        f = Path(a.output) / f"{a.name}.py"
        f.write_text(_TEMPLATES[a.template].format(name=a.name, cls=a.name.title().replace("_", "")))
        return {"generated": str(f)}
    if a.action == "test":
        import subprocess
        root = Path(__file__).resolve().parent.parent
        return subprocess.call([sys.executable, "-m", "pytest", str(root / "tests"), "-q", "-m", a.marker])
    if a.action == "debug":
        import torch
        st = _load_state(a.path)
        rep = {}
        for k, v in st["parameters"].items():
            v = _t(v).float()
            rep[k] = f"mean={v.mean():.3e} std={v.std():.3e} absmax={v.abs().max():.3e} nan={int(torch.isnan(v).sum())}"
        return rep
    if a.action == "profile":
        import torch
        from . import models
        from .utils.profiler import Profiler
        dev = _device(a.device, cfg)
        m = models.create_model(a.model).to(dev)
        x = _example_input(m, 2, 64, dev)
        prof = Profiler()
        with torch.no_grad():
            for i in range(a.iters):
                with prof.scope(f"forward_{i}", "model"):
                    m(x)
        prof.export_chrome_trace(a.output)
        return {"trace": a.output, "events": len(prof.events)}
    raise SystemExit(f"unknown dev action {a.action}")


def cmd_info(a, cfg):
    from .utils import collect_env
    return collect_env()


def cmd_init(a, cfg):
    root = Path(a.path)
    (root / "src").mkdir(parents=True, exist_ok=True)
    (root / "torsh.json").write_text(json.dumps(DEFAULT_CONFIG, indent=1))
    (root / "src" / "model.py").write_text(_TEMPLATES["model"].format(name=root.name, cls="Model"))
    (root / "src" / "train.py").write_text(_TEMPLATES["train"].format(name=root.name))
    return {"project": str(root), "files": ["torsh.json", "src/model.py", "src/train.py"]}


def cmd_update(a, cfg):
    from . import __version__
    return {"version": __version__, "update": "no package index is reachable; rebuild native libraries with "
                                              "`python -m torsh_b200._build`"}


def cmd_completions(a, cfg):
    cmds = "model train dataset benchmark hub dev info init update completions"
    if a.shell == "bash":
        return f'complete -W "{cmds}" torsh'
    if a.shell == "zsh":
        return f"compdef '_arguments \"1: :({cmds})\"' torsh"
    if a.shell == "fish":
        return "\n".join(f"complete -c torsh -n __fish_use_subcommand -a {c}" for c in cmds.split())
    raise SystemExit("shells: bash zsh fish")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="torsh", description="torsh_b200 command line")
    p.add_argument("--config"); p.add_argument("--json", action="store_true"); p.add_argument("-v", "--verbose", action="count", default=0)
    p.add_argument("--no-color", action="store_true")
    sub = p.add_subparsers(dest="command", required=True)

    m = sub.add_parser("model"); m.add_argument("action", choices=["list", "create", "inspect", "convert", "validate", "quantize", "benchmark", "prune", "optimize", "compress", "extract", "merge"])
    m.add_argument("path", nargs="?"); m.add_argument("others", nargs="*"); m.add_argument("--sparsity", type=float, default=0.5); m.add_argument("--structured", action="store_true")
    m.add_argument("--fold"); m.add_argument("--level", type=int, default=6); m.add_argument("--pattern"); m.add_argument("--weights"); m.add_argument("-o", "--output"); m.add_argument("--name"); m.add_argument("--dtype", choices=["f32", "f16", "bf16"])
    m.add_argument("--bits", type=int, default=8); m.add_argument("--limit", type=int, default=20); m.add_argument("--device")
    m.add_argument("--batch", type=int, default=2); m.add_argument("--seq", type=int, default=128); m.add_argument("--iters", type=int, default=10)

    t = sub.add_parser("train"); t.add_argument("action", choices=["start", "resume", "monitor", "stop"])
    t.add_argument("--model", default="gpt2"); t.add_argument("--model-args"); t.add_argument("--output"); t.add_argument("--device")
    t.add_argument("--steps", type=int, default=10); t.add_argument("--batch-size", type=int); t.add_argument("--lr", type=float)
    t.add_argument("--seq", type=int, default=128); t.add_argument("--image", type=int, default=64); t.add_argument("--log-every", type=int, default=10)

    d = sub.add_parser("dataset"); d.add_argument("action", choices=["download", "preprocess", "analyze", "split"])
    d.add_argument("path", nargs="?"); d.add_argument("--name", default="mnist"); d.add_argument("-o", "--output", default="./data")
    d.add_argument("--samples", type=int, default=1024); d.add_argument("--train", type=float, default=0.8); d.add_argument("--val", type=float, default=0.1)
    d.add_argument("--seed", type=int, default=42)

    b = sub.add_parser("benchmark"); b.add_argument("action", choices=["run", "compare", "report"])
    b.add_argument("--suite", default="all"); b.add_argument("-o", "--output", default="./outputs/benchmark.json"); b.add_argument("--device")
    b.add_argument("--iters", type=int, default=20); b.add_argument("--warmup", type=int, default=3)
    b.add_argument("--baseline"); b.add_argument("--candidate"); b.add_argument("--results")

    h = sub.add_parser("hub"); h.add_argument("action", choices=["download", "upload", "list", "search"])
    h.add_argument("name", nargs="?"); h.add_argument("--path"); h.add_argument("--version"); h.add_argument("--query", default="")
    h.add_argument("-o", "--output"); h.add_argument("--cache")

    v = sub.add_parser("dev"); v.add_argument("action", choices=["codegen", "test", "debug", "profile"])
    v.add_argument("path", nargs="?"); v.add_argument("--template", default="model"); v.add_argument("--name", default="my_model")
    v.add_argument("-o", "--output", default="./generated"); v.add_argument("--marker", default="not gpu"); v.add_argument("--model", default="gpt2")
    v.add_argument("--device"); v.add_argument("--iters", type=int, default=3)

    sub.add_parser("info")
    i = sub.add_parser("init"); i.add_argument("path")
    sub.add_parser("update")
    c = sub.add_parser("completions"); c.add_argument("shell")
    return p


_COMMANDS = {"model": cmd_model, "train": cmd_train, "dataset": cmd_dataset, "benchmark": cmd_benchmark, "hub": cmd_hub,
             "dev": cmd_dev, "info": cmd_info, "init": cmd_init, "update": cmd_update, "completions": cmd_completions}


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    cfg = load_config(a.config)
    res = _COMMANDS[a.command](a, cfg)
    if isinstance(res, int):
        return res
    _emit(res, a.json)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
