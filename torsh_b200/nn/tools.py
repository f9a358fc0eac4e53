"""Model-level tools of ``crates/torsh-nn/src``: numerical stability testing (``numerical_stability.rs``), deployment
export with optimisation and benchmarks (``export.rs``), conversion of other frameworks' checkpoints and layer naming
(``conversion.rs``), a local model zoo with weight records (``model_zoo.rs``), graph-level network optimisation report
(``optimization.rs``), per-layer update policies (``parameter_updates.rs``) and activation / gradient recording hooks
(``hooks/``, ``diagnostics/``)."""
from __future__ import annotations

import copy
import hashlib
import json
import math
import re
import time
from pathlib import Path
from typing import Callable, Sequence

import torch
from torch import nn


# ================================================================================================ numerical stability
class StabilityTester:
    """Runs a module under a set of stress inputs (zeros, tiny, huge, mixed-scale, extreme-sign, constant) and dtypes,
    and checks outputs and gradients for NaN / Inf, plus sensitivity to a small input perturbation."""

    CASES = {"zeros": lambda s: torch.zeros(s), "tiny": lambda s: torch.randn(s) * 1e-30, "huge": lambda s: torch.randn(s) * 1e4,
             "mixed_scale": lambda s: torch.randn(s) * torch.logspace(-6, 4, s[-1]), "constant": lambda s: torch.full(s, 3.0),
             "negative_huge": lambda s: -torch.rand(s) * 1e4, "normal": lambda s: torch.randn(s)}

    def __init__(self, dtypes=(torch.float32,), perturbation: float = 1e-3, seed: int = 0):
        self.dtypes, self.eps, self.seed = dtypes, perturbation, seed

    def test(self, module: nn.Module, input_shape: Sequence[int]) -> dict:
        results, module = [], copy.deepcopy(module).eval()
        for dt in self.dtypes:
            m = copy.deepcopy(module).to(dt)
            for name, make in self.CASES.items():
                torch.manual_seed(self.seed)
                x = make(tuple(input_shape)).to(dt).requires_grad_(True)
                rec = {"case": name, "dtype": str(dt).replace("torch.", "")}
                try:
                    y = m(x)
                    rec["output_finite"] = bool(torch.isfinite(y).all())
                    y.float().sum().backward()
                    grads = [p.grad for p in m.parameters() if p.grad is not None] + ([x.grad] if x.grad is not None else [])
                    rec["grad_finite"] = all(bool(torch.isfinite(g).all()) for g in grads)
                    with torch.no_grad():
                        y2 = m(x.detach() * (1 + self.eps))
                        rec["relative_sensitivity"] = float((y2 - y).float().norm() / (y.float().norm() * self.eps).clamp(min=1e-30)) if rec["output_finite"] else math.inf
                    m.zero_grad()
                except Exception as e:                                         # a crash is a finding, not a test failure
                    rec.update(output_finite=False, grad_finite=False, error=repr(e))
                rec["passed"] = rec.get("output_finite", False) and rec.get("grad_finite", False)
                results.append(rec)
        failed = [r for r in results if not r["passed"]]
        return {"results": results, "passed": not failed, "failed_cases": [(r["case"], r["dtype"]) for r in failed],
                "worst_sensitivity": max((r.get("relative_sensitivity", 0) for r in results if math.isfinite(r.get("relative_sensitivity", 0))), default=0.0)}


# ================================================================================================ export / deployment
class DeploymentOptimizer:
    """Inference preparation: eval mode, conv+bn folding through the graph tools when the module traces, dropout removal,
    optional dtype cast and ``requires_grad`` off."""

    def optimize(self, model: nn.Module, dtype: torch.dtype | None = None) -> tuple[nn.Module, dict]:
        from .. import fx as tfx, fx_tools
        m = copy.deepcopy(model).eval()
        report = {"folded_conv_bn": 0, "fused_activation": 0, "removed_dropout": 0, "traced": False}
        for name, child in list(m.named_modules()):
            if isinstance(child, (nn.Dropout, nn.Dropout1d, nn.Dropout2d, nn.Dropout3d, nn.AlphaDropout)):
                parent = m.get_submodule(name.rpartition(".")[0]) if "." in name else m
                setattr(parent, name.rpartition(".")[2], nn.Identity())
                report["removed_dropout"] += 1
        try:
            gm = tfx.symbolic_trace(m)
            report["folded_conv_bn"] = fx_tools.fold_conv_bn(gm)
            report["fused_activation"] = fx_tools.fuse_module_activation(gm)
            m, report["traced"] = gm, True
        except Exception as e:
            report["trace_error"] = type(e).__name__
        if dtype is not None:
            m = m.to(dtype)
        for p in m.parameters():
            p.requires_grad_(False)
        return m, report


class ModelExporter:
    """Writes a model in one of the package's formats (``state`` binary model state, ``safetensors``, ``json``, ``onnx``
    through the built-in ONNX writer, ``torchscript`` trace) and records size, time and a checksum."""

    def export(self, model: nn.Module, path, fmt: str = "safetensors", example_inputs=None, architecture: str | None = None) -> dict:
        from ..serialize import model_state as ms
        path, t0 = Path(path), time.perf_counter()
        if fmt in ("state", "safetensors", "json"):
            st = ms.model_state(model, architecture=architecture)
            {"state": ms.save_binary, "safetensors": ms.save_safetensors, "json": ms.save_json}[fmt](st, path)
        elif fmt == "onnx":
            from .. import onnx_io
            onnx_io.export_onnx(model, example_inputs, path)
        elif fmt == "torchscript":
            torch.jit.trace(model.eval(), example_inputs).save(str(path))
        else:
            raise ValueError(f"unknown export format {fmt!r}")
        data = path.read_bytes()
        return {"format": fmt, "path": str(path), "bytes": len(data), "sha256": hashlib.sha256(data).hexdigest(), "seconds": time.perf_counter() - t0,
                "parameters": sum(p.numel() for p in model.parameters())}

    def benchmark(self, model: nn.Module, example_inputs, formats=("state", "safetensors", "json"), out_dir=".") -> list[dict]:
        return sorted((self.export(model, Path(out_dir) / f"model.{f}", f, example_inputs) for f in formats), key=lambda r: r["bytes"])


# ================================================================================================ conversion
_TF_RULES = [(r"/", "."), (r"\.kernel$", ".weight"), (r"\.gamma$", ".weight"), (r"\.beta$", ".bias"), (r"\.moving_mean$", ".running_mean"),
             (r"\.moving_variance$", ".running_var"), (r":0$", "")]


class ModelConverter:
    """Checkpoint conversion into this package's naming and layouts.

    ``from_tensorflow``: ``scope/layer/kernel:0`` names to dotted ``weight`` / ``bias`` names; dense kernels ``[in, out]`` are
    transposed, convolution kernels ``[kh, kw, in, out]`` permuted to ``[out, in, kh, kw]``.
    ``rename``: regex rules for any source.  ``fit``: loads a converted state into a model, reports missing, unexpected and
    shape-mismatched entries instead of raising."""

    def from_tensorflow(self, weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        out = {}
        for name, t in weights.items():
            is_kernel = re.search(r"/kernel(:0)?$", name) is not None
            new = name
            for pat, rep in [(r":0$", ""), *_TF_RULES]:
                new = re.sub(pat, rep, new)
            t = torch.as_tensor(t)
            if is_kernel and t.dim() == 2:
                t = t.t()
            elif is_kernel and t.dim() == 4:
                t = t.permute(3, 2, 0, 1)
            elif is_kernel and t.dim() == 3:
                t = t.permute(2, 1, 0)
            out[new] = t.contiguous()
        return out

    def rename(self, state: dict, rules: Sequence[tuple[str, str]]) -> dict:
        out = {}
        for k, v in state.items():
            for pat, rep in rules:
                k = re.sub(pat, rep, k)
            out[k] = v
        return out

    def fit(self, model: nn.Module, state: dict) -> dict:
        own = model.state_dict()
        ok = {k: v for k, v in state.items() if k in own and tuple(own[k].shape) == tuple(v.shape)}
        report = {"loaded": sorted(ok), "missing": sorted(set(own) - set(state)), "unexpected": sorted(set(state) - set(own)),
                  "shape_mismatch": sorted(k for k in state if k in own and tuple(own[k].shape) != tuple(state[k].shape))}
        model.load_state_dict({**own, **{k: v.to(own[k].dtype) for k, v in ok.items()}})
        return report

    def describe(self, model: nn.Module) -> list[dict]:
        return [{"name": n, "type": type(m).__name__, "parameters": sum(p.numel() for p in m.parameters(recurse=False))} for n, m in model.named_modules() if n]


class MigrationHelper:
    """Source-level hints for code written against other APIs: maps call names to this package's and lists what has no
    counterpart."""

    MAP = {"torch.nn.Linear": "torsh_b200.nn.Linear", "torch.nn.LayerNorm": "torsh_b200.nn.LayerNorm", "torch.optim.AdamW": "torsh_b200.optim.AdamW",
           "torch.optim.SGD": "torsh_b200.optim.SGD", "torch.nn.functional.scaled_dot_product_attention": "torsh_b200.nn.functional.scaled_dot_product_attention",
           "torch.nn.parallel.DistributedDataParallel": "torsh_b200.parallel.ddp.DistributedDataParallel", "torch.utils.data.DataLoader": "torsh_b200.data.DataLoader",
           "tf.keras.layers.Dense": "torsh_b200.nn.Linear", "tf.keras.layers.LayerNormalization": "torsh_b200.nn.LayerNorm", "tf.keras.optimizers.Adam": "torsh_b200.optim.Adam"}

    def migrate_source(self, source: str) -> tuple[str, list[str]]:
        notes = []
        for old, new in sorted(self.MAP.items(), key=lambda kv: -len(kv[0])):
            if old in source:
                source = source.replace(old, new)
                notes.append(f"{old} -> {new}")
        unknown = sorted(set(re.findall(r"\btf\.[\w.]+", source)))
        return source, notes + [f"no mapping for {u}" for u in unknown]


# ================================================================================================ model zoo
class ModelZoo:
    """Registry of constructors with configurations and weight files on disk (``<root>/<name>/<version>.safetensors`` with
    a JSON record holding the checksum); nothing is downloaded."""

    def __init__(self, root):
        self.root, self.builders = Path(root), {}
        self.root.mkdir(parents=True, exist_ok=True)

    def register(self, name: str, builder: Callable[..., nn.Module], default_config: dict | None = None, description: str = ""):
        self.builders[name] = {"builder": builder, "config": default_config or {}, "description": description}

    def list_models(self): return sorted(self.builders)
    def _dir(self, name): return self.root / name

    def save_weights(self, name: str, model: nn.Module, version: str = "v1", metrics: dict | None = None) -> dict:
        from ..serialize import model_state as ms
        d = self._dir(name)
        d.mkdir(exist_ok=True)
        ms.save_safetensors(ms.model_state(model, architecture=name), d / f"{version}.safetensors")
        info = {"name": name, "version": version, "sha256": hashlib.sha256((d / f"{version}.safetensors").read_bytes()).hexdigest(),
                "parameters": sum(p.numel() for p in model.parameters()), "metrics": metrics or {}}
        (d / f"{version}.json").write_text(json.dumps(info))
        return info

    def available_weights(self, name): return sorted(p.stem for p in self._dir(name).glob("*.json")) if self._dir(name).exists() else []

    def create(self, name: str, pretrained: str | None = None, **overrides) -> nn.Module:
        from ..serialize import model_state as ms
        b = self.builders[name]
        model = b["builder"](**{**b["config"], **overrides})
        if pretrained:
            info = json.loads((self._dir(name) / f"{pretrained}.json").read_text())
            path = self._dir(name) / f"{pretrained}.safetensors"
            if hashlib.sha256(path.read_bytes()).hexdigest() != info["sha256"]:
                raise IOError(f"{name}/{pretrained}: weight file does not match its recorded checksum")
            ms.load_model_state(model, ms.load_safetensors(path))
        return model


# ================================================================================================ network optimisation report
class NetworkOptimizer:
    """Static report over a module tree: parameter and activation memory per layer for one example input, FLOPs of linear
    and convolution layers, and findings (layers that dominate, conv+bn pairs, very wide activations)."""

    def analyze(self, model: nn.Module, example_input: torch.Tensor) -> dict:
        rows, hooks = [], []
        def hook(name):
            def fn(m, inp, out):
                if isinstance(out, torch.Tensor):
                    flops = 0
                    if isinstance(m, nn.Linear):
                        flops = 2 * out.numel() * m.in_features
                    elif isinstance(m, (nn.Conv1d, nn.Conv2d, nn.Conv3d)):
                        flops = 2 * out.numel() * (m.in_channels // m.groups) * math.prod(m.kernel_size)
                    rows.append({"name": name, "type": type(m).__name__, "params": sum(p.numel() for p in m.parameters(recurse=False)),
                                 "activation_bytes": out.numel() * out.element_size(), "flops": flops})
            return fn
        for n, m in model.named_modules():
            if n and not list(m.children()):
                hooks.append(m.register_forward_hook(hook(n)))
        with torch.no_grad():
            model.eval()(example_input)
        for h in hooks:
            h.remove()
        total_f, total_a = sum(r["flops"] for r in rows) or 1, sum(r["activation_bytes"] for r in rows) or 1
        findings = [f"{r['name']} holds {r['flops'] / total_f:.0%} of the FLOPs" for r in rows if r["flops"] / total_f > 0.5]
        findings += [f"{r['name']} holds {r['activation_bytes'] / total_a:.0%} of the activation memory" for r in rows if r["activation_bytes"] / total_a > 0.5]
        names = [r["type"] for r in rows]
        findings += [f"{rows[i]['name']} + {rows[i + 1]['name']}: convolution followed by batch norm can be folded" for i in range(len(rows) - 1)
                     if names[i].startswith("Conv") and names[i + 1].startswith("BatchNorm")]
        return {"layers": rows, "total_flops": sum(r["flops"] for r in rows), "total_params": sum(r["params"] for r in rows),
                "total_activation_bytes": sum(r["activation_bytes"] for r in rows), "findings": findings}


# ================================================================================================ per-layer update policies
class LayerSpecificOptimizers:
    """Parameter groups by name pattern with their own learning-rate multiplier, weight decay and freeze flag (first match
    wins); ``layerwise_decay`` assigns ``base_lr * decay^(depth from the top)`` to numbered blocks."""

    def __init__(self, model: nn.Module, rules: Sequence[tuple[str, dict]] = (), default: dict | None = None):
        self.model, self.rules, self.default = model, list(rules), default or {}

    def param_groups(self, base_lr: float, weight_decay: float = 0.0) -> list[dict]:
        groups: dict[tuple, dict] = {}
        for name, p in self.model.named_parameters():
            cfg = next((c for pat, c in self.rules if re.search(pat, name)), self.default)
            if cfg.get("freeze"):
                p.requires_grad_(False)
                continue
            key = (cfg.get("lr_mult", 1.0), cfg.get("weight_decay", weight_decay))
            g = groups.setdefault(key, {"params": [], "lr": base_lr * key[0], "weight_decay": key[1], "names": []})
            g["params"].append(p); g["names"].append(name)
        return list(groups.values())

    @staticmethod
    def layerwise_decay(model: nn.Module, base_lr: float, decay: float = 0.8, block_pattern: str = r"\.(\d+)\.") -> list[dict]:
        depth = lambda n: int(m.group(1)) if (m := re.search(block_pattern, n)) else None
        top = max((d for n, _ in model.named_parameters() if (d := depth(n)) is not None), default=0)
        groups: dict[float, dict] = {}
        for n, p in model.named_parameters():
            d = depth(n)
            lr = base_lr * decay ** (top - d if d is not None else (top + 1 if n.startswith(("embed", "wte", "wpe", "patch")) else 0))
            groups.setdefault(lr, {"params": [], "lr": lr, "names": []})
            groups[lr]["params"].append(p); groups[lr]["names"].append(n)
        return sorted(groups.values(), key=lambda g: g["lr"])


class ParameterUpdater:
    """Applies gradient updates with clipping by value and by norm, weight-norm bounds and an exponential moving average
    copy of the parameters; counts what it clipped."""

    def __init__(self, params, lr: float, clip_value: float | None = None, clip_norm: float | None = None, max_weight_norm: float | None = None, ema_decay: float | None = None):
        self.params, self.lr, self.cv, self.cn, self.mw, self.ema_decay = list(params), lr, clip_value, clip_norm, max_weight_norm, ema_decay
        self.ema = [p.detach().clone() for p in self.params] if ema_decay else None
        self.stats = {"steps": 0, "value_clipped": 0, "norm_clipped": 0, "weights_rescaled": 0}

    @torch.no_grad()
    def step(self):
        ps = [p for p in self.params if p.grad is not None]
        if self.cv is not None:
            for p in ps:
                self.stats["value_clipped"] += int((p.grad.abs() > self.cv).sum())
                p.grad.clamp_(-self.cv, self.cv)
        if self.cn is not None and float(torch.nn.utils.clip_grad_norm_(ps, self.cn)) > self.cn:
            self.stats["norm_clipped"] += 1
        for p in ps:
            p.add_(p.grad, alpha=-self.lr)
            if self.mw is not None and p.dim() > 1:
                n = p.flatten(1).norm(dim=1).reshape(-1, *[1] * (p.dim() - 1))
                over = n > self.mw
                if over.any():
                    p.mul_(torch.where(over, self.mw / n.clamp(min=1e-12), torch.ones_like(n)))
                    self.stats["weights_rescaled"] += int(over.sum())
        if self.ema is not None:
            for e, p in zip(self.ema, self.params):
                e.mul_(self.ema_decay).add_(p.detach(), alpha=1 - self.ema_decay)
        self.stats["steps"] += 1

    def swap_in_ema(self):
        """Exchanges the live parameters with their averages (call again to swap back)."""
        with torch.no_grad():
            for e, p in zip(self.ema, self.params):
                tmp = p.detach().clone()
                p.copy_(e)
                e.copy_(tmp)


# ================================================================================================ recording hooks
class ActivationRecorder:
    """Forward and backward hooks on the leaf modules that match ``pattern``: records mean, standard deviation, share of
    zeros and maximum of each output (and gradient norms), and flags dead or saturated layers."""

    def __init__(self, model: nn.Module, pattern: str = ".*"):
        self.stats, self.grads, self.handles = {}, {}, []
        for name, m in model.named_modules():
            if name and not list(m.children()) and re.search(pattern, name):
                self.handles.append(m.register_forward_hook(self._fwd(name)))
                self.handles.append(m.register_full_backward_hook(self._bwd(name)))

    def _fwd(self, name):
        def fn(m, inp, out):
            if isinstance(out, torch.Tensor):
                o = out.detach().float()
                self.stats[name] = {"mean": float(o.mean()), "std": float(o.std()) if o.numel() > 1 else 0.0, "zero_fraction": float((o == 0).float().mean()),
                                    "abs_max": float(o.abs().max()), "saturated": float((o.abs() > 0.99 * o.abs().max().clamp(min=1e-12)).float().mean())}
        return fn

    def _bwd(self, name):
        def fn(m, gin, gout):
            if gout and gout[0] is not None:
                self.grads[name] = float(gout[0].detach().float().norm())
        return fn

    def findings(self, dead_threshold: float = 0.95) -> list[str]:
        out = [f"{n}: {s['zero_fraction']:.0%} of outputs are zero" for n, s in self.stats.items() if s["zero_fraction"] >= dead_threshold]
        out += [f"{n}: gradient norm {g:.2e} vanishes" for n, g in self.grads.items() if g < 1e-8]
        out += [f"{n}: outputs reach {s['abs_max']:.2e}" for n, s in self.stats.items() if s["abs_max"] > 1e4]
        return out

    def remove(self):
        for h in self.handles:
            h.remove()
        self.handles.clear()
