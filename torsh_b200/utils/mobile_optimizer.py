"""Model preparation for constrained targets and layer-level bottleneck profiling (``crates/torsh-utils/src/mobile_optimizer/``,
``bottleneck.rs``).

``optimize_for_mobile`` applies, in order and as configured: dropout removal, convolution / batch-norm folding, magnitude
pruning to a size target, dynamic INT8 or fp16 weight storage for linear layers, and reports what each step did to size
and to the output error on a calibration batch.  ``profile_bottlenecks`` times every leaf module forward (and backward)
over repeated runs and ranks them; memory per layer comes from output sizes."""
from __future__ import annotations

import copy
import os
import time
from dataclasses import dataclass, field

import torch
from torch import nn


PLATFORMS = {
    "ios": {"preferred_dtype": torch.float16, "quantization": "fp16", "alignment": 16, "max_model_mb": 200},
    "android": {"preferred_dtype": torch.float32, "quantization": "dynamic_int8", "alignment": 8, "max_model_mb": 100},
    "edge": {"preferred_dtype": torch.float32, "quantization": "dynamic_int8", "alignment": 4, "max_model_mb": 16},
    "server": {"preferred_dtype": torch.bfloat16, "quantization": "none", "alignment": 64, "max_model_mb": 1 << 20},
}


@dataclass
class MobileOptimizerConfig:
    platform: str = "android"
    remove_dropout: bool = True
    fold_batch_norm: bool = True
    quantization: str | None = None            # None -> the platform's choice; "none" | "fp16" | "dynamic_int8"
    prune_sparsity: float = 0.0
    size_target_mb: float | None = None
    preserve_modules: tuple[str, ...] = ()


class Int8DynamicLinear(nn.Module):
    """Weights stored as INT8 with one scale per output row; activations are quantised per call (per row, symmetric), the
    product is accumulated in INT32 and rescaled."""

    def __init__(self, lin: nn.Linear):
        super().__init__()
        w = lin.weight.detach().float()
        scale = w.abs().amax(1).clamp(min=1e-12) / 127
        self.register_buffer("qweight", (w / scale[:, None]).round().clamp(-127, 127).to(torch.int8))
        self.register_buffer("scale", scale)
        self.bias = None if lin.bias is None else nn.Parameter(lin.bias.detach().clone(), requires_grad=False)
        self.in_features, self.out_features = lin.in_features, lin.out_features

    def forward(self, x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1]).float()
        xs = x2.abs().amax(1, keepdim=True).clamp(min=1e-12) / 127
        xq = (x2 / xs).round().clamp(-127, 127)
        acc = xq @ self.qweight.float().t()                                     # exact: |sum| < 2^24 for K up to ~1000
        y = acc * xs * self.scale
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, -1).to(x.dtype)


class _HalfStorage(nn.Module):
    """Runs a half-precision model on inputs of any floating dtype and returns that dtype."""

    def __init__(self, inner): super().__init__(); self.inner = inner
    def forward(self, x): return self.inner(x.half()).to(x.dtype)


def model_size_bytes(model: nn.Module) -> int:
    return sum(t.numel() * t.element_size() for t in list(model.parameters()) + list(model.buffers()))


def _replace(model, name, new):
    parent = model.get_submodule(name.rpartition(".")[0]) if "." in name else model
    setattr(parent, name.rpartition(".")[2], new)


def optimize_for_mobile(model: nn.Module, config: MobileOptimizerConfig | None = None, calibration: torch.Tensor | None = None):
    """Returns ``(optimised model, report)``; the input model is not modified."""
    cfg = config or MobileOptimizerConfig()
    plat = PLATFORMS[cfg.platform]
    m = copy.deepcopy(model).eval()
    ref = m(calibration).detach() if calibration is not None else None
    steps, size0 = [], model_size_bytes(m)

    def log(step, **kw):
        rec = {"step": step, "bytes": model_size_bytes(m), **kw}
        if ref is not None:
            with torch.no_grad():
                out = m(calibration)
            rec["relative_error"] = float((out.float() - ref.float()).norm() / ref.float().norm().clamp(min=1e-12))
        steps.append(rec)

    if cfg.remove_dropout:
        n = 0
        for name, c in list(m.named_modules()):
            if isinstance(c, (nn.Dropout, nn.Dropout1d, nn.Dropout2d, nn.Dropout3d, nn.AlphaDropout)) and name not in cfg.preserve_modules:
                _replace(m, name, nn.Identity()); n += 1
        log("remove_dropout", removed=n)
    if cfg.fold_batch_norm:
        n = 0
        for name, seq in [(n_, c) for n_, c in m.named_modules() if isinstance(c, nn.Sequential)] + ([("", m)] if isinstance(m, nn.Sequential) else []):
            keys = list(seq._modules)
            for a, b in zip(keys, keys[1:]):
                conv, bn = seq._modules[a], seq._modules[b]
                if isinstance(conv, (nn.Conv1d, nn.Conv2d, nn.Conv3d)) and isinstance(bn, (nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d)) and bn.track_running_stats:
                    seq._modules[a], seq._modules[b] = torch.nn.utils.fusion.fuse_conv_bn_eval(conv, bn), nn.Identity()
                    n += 1
        log("fold_batch_norm", folded=n)
    sparsity = cfg.prune_sparsity
    if sparsity > 0:
        ws = [p for n_, p in m.named_parameters() if p.dim() > 1 and not any(n_.startswith(k) for k in cfg.preserve_modules)]
        allw = torch.cat([w.detach().abs().flatten() for w in ws])
        thr = allw.kthvalue(max(1, int(sparsity * allw.numel()))).values
        with torch.no_grad():
            for w in ws:
                w.mul_((w.abs() > thr).to(w.dtype))
        log("prune", sparsity=float(sum((w == 0).sum() for w in ws) / sum(w.numel() for w in ws)))
    quant = cfg.quantization or plat["quantization"]
    if quant == "fp16":
        m = _HalfStorage(m.half())
        log("fp16")
    elif quant == "dynamic_int8":
        n = 0
        for name, c in list(m.named_modules()):
            if isinstance(c, nn.Linear) and name not in cfg.preserve_modules:
                _replace(m, name, Int8DynamicLinear(c)); n += 1
        log("dynamic_int8", layers=n)
    final = model_size_bytes(m)
    report = {"platform": cfg.platform, "original_bytes": size0, "optimized_bytes": final, "compression": size0 / max(final, 1), "steps": steps,
              "fits_target": cfg.size_target_mb is None or final <= cfg.size_target_mb * 2 ** 20, "fits_platform": final <= plat["max_model_mb"] * 2 ** 20}
    return m, report


def export_optimized_model(model: nn.Module, path, example: torch.Tensor | None = None, fmt: str = "state_dict") -> dict:
    """``state_dict`` (tensors incl. INT8 buffers via ``torch.save``) or ``torchscript`` (traced with ``example``)."""
    if fmt == "torchscript":
        torch.jit.trace(model, example).save(str(path))
    else:
        torch.save(model.state_dict(), path)
    return {"path": str(path), "bytes": os.path.getsize(path), "format": fmt}


def benchmark_mobile_model(model: nn.Module, example: torch.Tensor, warmup: int = 3, iters: int = 20, threads: int | None = None) -> dict:
    prev = torch.get_num_threads()
    if threads:
        torch.set_num_threads(threads)
    try:
        with torch.no_grad():
            for _ in range(warmup):
                model(example)
            t = []
            for _ in range(iters):
                t0 = time.perf_counter()
                model(example)
                t.append(time.perf_counter() - t0)
    finally:
        torch.set_num_threads(prev)
    t.sort()
    return {"mean_ms": 1e3 * sum(t) / len(t), "p50_ms": 1e3 * t[len(t) // 2], "p95_ms": 1e3 * t[min(len(t) - 1, int(0.95 * len(t)))], "throughput_per_s": example.shape[0] * len(t) / sum(t),
            "model_bytes": model_size_bytes(model), "threads": threads or prev}


# ---- bottleneck profiling ---------------------------------------------------------------------------------------------------
@dataclass
class BottleneckReport:
    layers: list = field(default_factory=list)
    total_forward_ms: float = 0.0
    total_backward_ms: float = 0.0
    hotspots: list = field(default_factory=list)
    memory_peak_layer: str = ""
    recommendations: list = field(default_factory=list)

    def render(self) -> str:
        lines = [f"{'layer':30s} {'type':18s} {'fwd ms':>9s} {'bwd ms':>9s} {'share':>7s} {'out MiB':>9s}"]
        for l in self.layers:
            lines.append(f"{l['name'][:30]:30s} {l['type'][:18]:18s} {l['forward_ms']:9.3f} {l['backward_ms']:9.3f} {l['share']:7.1%} {l['output_bytes'] / 2 ** 20:9.3f}")
        lines.append(f"total forward {self.total_forward_ms:.3f} ms, backward {self.total_backward_ms:.3f} ms")
        lines += [f"* {r}" for r in self.recommendations]
        return "\n".join(lines)


def profile_bottlenecks(model: nn.Module, example: torch.Tensor, iters: int = 5, backward: bool = True, clock=time.perf_counter) -> BottleneckReport:
    """Per-leaf-module timing through forward pre / post hooks and full backward hooks; on a CUDA model every timestamp is
    taken after a device synchronise, so times are device times including launch gaps."""
    sync = torch.cuda.synchronize if example.is_cuda else (lambda: None)
    fwd, bwd, out_bytes, types, t0 = {}, {}, {}, {}, {}
    handles = []
    for name, mod in model.named_modules():
        if name and not list(mod.children()):
            types[name] = type(mod).__name__
            def pre(m, inp, name=name):
                sync(); t0[name] = clock()
            def post(m, inp, out, name=name):
                sync()
                fwd[name] = fwd.get(name, 0.0) + clock() - t0[name]
                if isinstance(out, torch.Tensor):
                    out_bytes[name] = out.numel() * out.element_size()
            def bpre(m, gout, name=name):
                sync(); t0["b:" + name] = clock()
            def bpost(m, gin, gout, name=name):
                sync()
                if "b:" + name in t0:
                    bwd[name] = bwd.get(name, 0.0) + clock() - t0["b:" + name]
            handles += [mod.register_forward_pre_hook(pre), mod.register_forward_hook(post), mod.register_full_backward_pre_hook(bpre), mod.register_full_backward_hook(bpost)]
    was_training = model.training
    try:
        for _ in range(iters):
            x = example.clone().requires_grad_(backward and example.is_floating_point())
            out = model(x)
            if backward:
                out.float().sum().backward()
                model.zero_grad(set_to_none=True)
    finally:
        for h in handles:
            h.remove()
        model.train(was_training)
    total = sum(fwd.values()) + sum(bwd.values()) or 1.0
    layers = sorted(({"name": n, "type": types[n], "forward_ms": 1e3 * fwd.get(n, 0) / iters, "backward_ms": 1e3 * bwd.get(n, 0) / iters,
                      "share": (fwd.get(n, 0) + bwd.get(n, 0)) / total, "output_bytes": out_bytes.get(n, 0)} for n in types if n in fwd), key=lambda l: -l["share"])
    rep = BottleneckReport(layers, 1e3 * sum(fwd.values()) / iters, 1e3 * sum(bwd.values()) / iters, [l["name"] for l in layers[:3]],
                           max(out_bytes, key=out_bytes.get) if out_bytes else "")
    for l in layers[:3]:
        if l["share"] > 0.4:
            rep.recommendations.append(f"{l['name']} ({l['type']}) takes {l['share']:.0%} of the step: the first place to optimise")
    small = [l for l in layers if l["forward_ms"] < 0.02 and l["type"] in ("ReLU", "GELU", "Dropout", "LayerNorm", "Sigmoid", "Tanh", "SiLU")]
    if len(small) >= 3:
        rep.recommendations.append(f"{len(small)} tiny element-wise layers: fuse them into their producers or capture the step in a CUDA graph")
    return rep
