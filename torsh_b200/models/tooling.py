"""Model tooling (``crates/torsh-models/src``): configuration objects and a factory with named presets (``config.rs``,
``builder.rs``), lazy and streaming weight loading from safetensors files (``lazy_loading.rs``), validation with hold-out /
k-fold / stratified strategies, confusion matrices and correctness checks (``validation.rs``), multi-model comparison with
ANOVA, pairwise tests, rankings and trade-offs (``comparison.rs``), inference benchmarking with latency percentiles
(``benchmark.rs``) and optimisation recommendations (``optimization.rs``)."""
from __future__ import annotations

import csv
import html
import io
import json
import math
import mmap
import statistics
import struct
import time
from collections import OrderedDict
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable, Iterator, Sequence

import numpy as np
import torch
from torch import nn

# ================================================================================================ configs and factory
@dataclass
class VisionModelConfig:
    architecture: str = "resnet"
    num_classes: int = 1000
    in_channels: int = 3
    depths: Sequence[int] = (2, 2, 2, 2)
    widths: Sequence[int] = (64, 128, 256, 512)
    patch_size: int = 16
    image_size: int = 224
    embed_dim: int = 768
    num_heads: int = 12
    dropout: float = 0.0

    def validate(self):
        if self.architecture not in ("resnet", "vit", "mlp_mixer"):
            raise ValueError(f"unknown vision architecture {self.architecture!r}")
        if self.architecture == "resnet" and len(self.depths) != len(self.widths):
            raise ValueError("depths and widths must have the same length")
        if self.architecture == "vit" and (self.image_size % self.patch_size or self.embed_dim % self.num_heads):
            raise ValueError("image size must be a multiple of the patch size and the embedding of the head count")
        return self


@dataclass
class NlpModelConfig:
    architecture: str = "gpt"
    vocab_size: int = 50257
    max_position: int = 1024
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    intermediate: int | None = None
    dropout: float = 0.1
    num_labels: int = 2

    def validate(self):
        if self.architecture not in ("gpt", "bert"):
            raise ValueError(f"unknown NLP architecture {self.architecture!r}")
        if self.hidden % self.heads:
            raise ValueError("hidden size must be divisible by the number of heads")
        return self


VISION_PRESETS = {"resnet18": VisionModelConfig("resnet", depths=(2, 2, 2, 2)), "resnet34": VisionModelConfig("resnet", depths=(3, 4, 6, 3)), "vit_base": VisionModelConfig("vit", embed_dim=768, num_heads=12, depths=(12,)),
                  "vit_small": VisionModelConfig("vit", embed_dim=384, num_heads=6, depths=(12,)), "vit_tiny": VisionModelConfig("vit", embed_dim=192, num_heads=3, depths=(12,))}
NLP_PRESETS = {"gpt2": NlpModelConfig("gpt"), "gpt2_medium": NlpModelConfig("gpt", hidden=1024, layers=24, heads=16), "bert_base": NlpModelConfig("bert", vocab_size=30522, max_position=512),
               "bert_large": NlpModelConfig("bert", vocab_size=30522, max_position=512, hidden=1024, layers=24, heads=16)}


class _BasicBlock(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.c1, self.b1, self.c2, self.b2 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False), nn.BatchNorm2d(cout), nn.Conv2d(cout, cout, 3, 1, 1, bias=False), nn.BatchNorm2d(cout)
        self.short = None if stride == 1 and cin == cout else nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))
    def forward(self, x):
        y = self.b2(self.c2(torch.relu(self.b1(self.c1(x)))))
        return torch.relu(y + (x if self.short is None else self.short(x)))


class _ViT(nn.Module):
    def __init__(self, c: VisionModelConfig):
        super().__init__()
        n = (c.image_size // c.patch_size) ** 2
        self.patch = nn.Conv2d(c.in_channels, c.embed_dim, c.patch_size, c.patch_size)
        self.cls, self.pos = nn.Parameter(torch.zeros(1, 1, c.embed_dim)), nn.Parameter(torch.randn(1, n + 1, c.embed_dim) * 0.02)
        self.blocks = nn.TransformerEncoder(nn.TransformerEncoderLayer(c.embed_dim, c.num_heads, 4 * c.embed_dim, c.dropout, "gelu", batch_first=True, norm_first=True), c.depths[0], enable_nested_tensor=False)
        self.norm, self.head = nn.LayerNorm(c.embed_dim), nn.Linear(c.embed_dim, c.num_classes)
    def forward(self, x):
        t = self.patch(x).flatten(2).transpose(1, 2)
        t = torch.cat([self.cls.expand(len(t), -1, -1), t], 1) + self.pos
        return self.head(self.norm(self.blocks(t))[:, 0])


class _Transformer(nn.Module):
    def __init__(self, c: NlpModelConfig):
        super().__init__()
        self.c = c
        self.tok, self.pos = nn.Embedding(c.vocab_size, c.hidden), nn.Embedding(c.max_position, c.hidden)
        self.blocks = nn.TransformerEncoder(nn.TransformerEncoderLayer(c.hidden, c.heads, c.intermediate or 4 * c.hidden, c.dropout, "gelu", batch_first=True, norm_first=c.architecture == "gpt"), c.layers, enable_nested_tensor=False)
        self.norm = nn.LayerNorm(c.hidden)
        self.head = nn.Linear(c.hidden, c.vocab_size, bias=False) if c.architecture == "gpt" else nn.Linear(c.hidden, c.num_labels)
        if c.architecture == "gpt":
            self.head.weight = self.tok.weight
    def forward(self, ids):
        h = self.tok(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device))
        mask = nn.Transformer.generate_square_subsequent_mask(ids.shape[1], device=ids.device) if self.c.architecture == "gpt" else None
        h = self.norm(self.blocks(h, mask=mask, is_causal=mask is not None))
        return self.head(h) if self.c.architecture == "gpt" else self.head(h[:, 0])


class ModelFactory:
    """Builds models from named presets or explicit configurations; new presets can be registered."""

    def __init__(self): self.vision, self.nlp = dict(VISION_PRESETS), dict(NLP_PRESETS)
    def add_config(self, domain: str, name: str, config): getattr(self, domain)[name] = config.validate()
    def list_all_models(self) -> dict: return {"vision": sorted(self.vision), "nlp": sorted(self.nlp)}

    def build_vision_model_from_config(self, c: VisionModelConfig) -> nn.Module:
        c.validate()
        if c.architecture == "vit":
            return _ViT(c)
        if c.architecture == "mlp_mixer":
            n, d = (c.image_size // c.patch_size) ** 2, c.embed_dim
            return nn.Sequential(nn.Conv2d(c.in_channels, d, c.patch_size, c.patch_size), nn.Flatten(2), nn.Linear(n, n), nn.GELU(), nn.LayerNorm(n), _Mean(-1), nn.Linear(d, c.num_classes))
        layers, cin = [nn.Conv2d(c.in_channels, c.widths[0], 3, 1, 1, bias=False), nn.BatchNorm2d(c.widths[0]), nn.ReLU()], c.widths[0]
        for i, (dep, w) in enumerate(zip(c.depths, c.widths)):
            for j in range(dep):
                layers.append(_BasicBlock(cin, w, 2 if j == 0 and i > 0 else 1)); cin = w
        return nn.Sequential(*layers, nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Dropout(c.dropout), nn.Linear(cin, c.num_classes))

    def build_nlp_model_from_config(self, c: NlpModelConfig) -> nn.Module: return _Transformer(c.validate())
    def build_vision_model(self, name: str, **overrides): return self.build_vision_model_from_config(VisionModelConfig(**{**asdict(self.vision[name]), **overrides}))
    def build_nlp_model(self, name: str, **overrides): return self.build_nlp_model_from_config(NlpModelConfig(**{**asdict(self.nlp[name]), **overrides}))

    def get_model_info(self, domain: str, name: str) -> dict | None:
        cfg = getattr(self, domain).get(name)
        if cfg is None:
            return None
        with torch.device("meta"):
            m = self.build_vision_model_from_config(cfg) if domain == "vision" else self.build_nlp_model_from_config(cfg)
        n = sum(p.numel() for p in {id(p): p for p in m.parameters()}.values())
        return {"name": name, "domain": domain, "architecture": cfg.architecture, "parameters": n, "fp32_mb": n * 4 / 2 ** 20, "bf16_mb": n * 2 / 2 ** 20, "config": asdict(cfg)}


class _Mean(nn.Module):
    def __init__(self, dim): super().__init__(); self.dim = dim
    def forward(self, x): return x.mean(self.dim)


def compare_configs(a, b) -> dict:
    da, db = asdict(a), asdict(b)
    return {k: (da.get(k), db.get(k)) for k in sorted(set(da) | set(db)) if da.get(k) != db.get(k)}


# ================================================================================================ safetensors: write, lazy load, stream
_ST = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool}
_ST_REV = {v: k for k, v in _ST.items()}


def write_safetensors(tensors: dict[str, torch.Tensor], path, metadata: dict | None = None) -> None:
    header, off = {}, 0
    for name in sorted(tensors):
        t = tensors[name]
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _ST_REV[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}; off += n
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj))); f.write(hj)
        for name in sorted(tensors):
            f.write(tensors[name].detach().contiguous().cpu().view(torch.uint8).numpy().tobytes())


@dataclass
class CacheStats:
    hits: int = 0
    misses: int = 0
    evictions: int = 0
    bytes_cached: int = 0
    capacity: int = 0
    def hit_rate(self): return self.hits / (self.hits + self.misses) if self.hits + self.misses else 0.0
    def utilization(self): return self.bytes_cached / self.capacity if self.capacity else 0.0


class LazyModelLoader:
    """Reads only the header at open time; a tensor's bytes are mapped from the file when it is first asked for and kept in
    a least-recently-used cache bounded in bytes."""

    def __init__(self, path, max_cache_bytes: int = 1 << 30):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        header = json.loads(self._f.read(n))
        self.metadata = header.pop("__metadata__", {})
        self.header, self.base = header, 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.cache: OrderedDict[str, torch.Tensor] = OrderedDict()
        self.stats = CacheStats(capacity=max_cache_bytes)

    def tensor_names(self) -> list[str]: return sorted(self.header)
    def tensor_metadata(self, name: str): h = self.header.get(name); return None if h is None else (tuple(h["shape"]), _ST[h["dtype"]])
    def is_cached(self, name: str) -> bool: return name in self.cache
    def cache_stats(self) -> CacheStats: return self.stats

    def _read(self, name: str) -> torch.Tensor:
        h = self.header[name]
        a, b = h["data_offsets"]
        raw = torch.frombuffer(bytearray(self._mm[self.base + a:self.base + b]), dtype=torch.uint8) if b > a else torch.empty(0, dtype=torch.uint8)
        return raw.view(_ST[h["dtype"]]).reshape(h["shape"])

    def get_tensor(self, name: str) -> torch.Tensor:
        if name not in self.header:
            raise KeyError(f"no tensor named {name!r}; available: {', '.join(self.tensor_names()[:5])}...")
        if name in self.cache:
            self.stats.hits += 1; self.cache.move_to_end(name)
            return self.cache[name]
        self.stats.misses += 1
        t = self._read(name)
        size = t.numel() * t.element_size()
        if size <= self.stats.capacity:
            while self.stats.bytes_cached + size > self.stats.capacity and self.cache:
                _, old = self.cache.popitem(last=False)
                self.stats.bytes_cached -= old.numel() * old.element_size(); self.stats.evictions += 1
            self.cache[name] = t; self.stats.bytes_cached += size
        return t

    def clear_cache(self): self.cache.clear(); self.stats.bytes_cached = 0

    def load_into(self, module: nn.Module, strict: bool = True, prefix: str = "") -> dict:
        """Copies tensors into a module parameter by parameter (peak extra memory: one tensor)."""
        own = dict(module.state_dict(keep_vars=True))
        missing = [k for k in own if prefix + k not in self.header]
        unexpected = [k for k in self.header if k.removeprefix(prefix) not in own]
        if strict and (missing or unexpected):
            raise KeyError(f"missing {missing[:3]}, unexpected {unexpected[:3]}")
        with torch.no_grad():
            for k, p in own.items():
                if prefix + k in self.header:
                    p.copy_(self._read(prefix + k))
        return {"missing": missing, "unexpected": unexpected}

    def stream_tensors(self, callback: Callable[[str, torch.Tensor], None]):
        """Every tensor once, in file order, without caching."""
        for name in sorted(self.header, key=lambda k: self.header[k]["data_offsets"][0]):
            callback(name, self._read(name))

    def stream_tensor_chunks(self, name: str, chunk_bytes: int) -> Iterator[torch.Tensor]:
        h = self.header[name]
        a, b = h["data_offsets"]
        es = torch.empty(0, dtype=_ST[h["dtype"]]).element_size()
        step = max(es, chunk_bytes // es * es)
        for s in range(a, b, step):
            yield torch.frombuffer(bytearray(self._mm[self.base + s:self.base + min(b, s + step)]), dtype=torch.uint8).view(_ST[h["dtype"]])

    def close(self): self.cache.clear(); self._mm.close(); self._f.close()
    def __enter__(self): return self
    def __exit__(self, *a): self.close()


# ================================================================================================ validation
class ConfusionMatrix:
    def __init__(self, num_classes: int): self.k, self.m = num_classes, torch.zeros(num_classes, num_classes, dtype=torch.long)
    def update(self, pred: torch.Tensor, target: torch.Tensor): self.m += torch.bincount(target * self.k + pred, minlength=self.k * self.k).reshape(self.k, self.k); return self

    def class_metrics(self) -> list[dict]:
        tp, col, row = self.m.diag().double(), self.m.sum(0).double(), self.m.sum(1).double()
        p, r = tp / col.clamp_min(1), tp / row.clamp_min(1)
        f1 = 2 * p * r / (p + r).clamp_min(1e-12)
        return [{"class": i, "precision": float(p[i]), "recall": float(r[i]), "f1": float(f1[i]), "support": int(row[i])} for i in range(self.k)]

    def summary(self, average: str = "macro") -> dict:
        cm = self.class_metrics()
        acc = float(self.m.diag().sum()) / max(int(self.m.sum()), 1)
        if average == "micro":
            return {"accuracy": acc, "precision": acc, "recall": acc, "f1": acc}
        w = [c["support"] for c in cm] if average == "weighted" else [1] * self.k
        agg = lambda key: sum(c[key] * wi for c, wi in zip(cm, w)) / max(sum(w), 1)
        return {"accuracy": acc, "precision": agg("precision"), "recall": agg("recall"), "f1": agg("f1")}


def make_splits(n: int, strategy: str = "kfold", k: int = 5, test_fraction: float = 0.2, labels: torch.Tensor | None = None, seed: int = 0, repeats: int = 1) -> list[tuple[torch.Tensor, torch.Tensor]]:
    """``holdout``, ``kfold``, ``stratified`` (k folds preserving class proportions), ``bootstrap`` (train with replacement, test
    on the rest), ``time_series`` (expanding window) or ``leave_one_out``."""
    g = torch.Generator().manual_seed(seed)
    if strategy == "holdout":
        p = torch.randperm(n, generator=g); c = int(round(n * (1 - test_fraction)))
        return [(p[:c], p[c:])]
    if strategy == "leave_one_out":
        return [(torch.cat([torch.arange(i), torch.arange(i + 1, n)]), torch.tensor([i])) for i in range(n)]
    if strategy == "time_series":
        fold = n // (k + 1)
        return [(torch.arange((i + 1) * fold), torch.arange((i + 1) * fold, min(n, (i + 2) * fold))) for i in range(k)]
    if strategy == "bootstrap":
        out = []
        for _ in range(k):
            tr = torch.randint(n, (n,), generator=g)
            mask = torch.ones(n, dtype=torch.bool); mask[tr] = False
            out.append((tr, mask.nonzero().flatten()))
        return out
    out = []
    for _ in range(repeats):
        if strategy == "stratified":
            fold_of = torch.empty(n, dtype=torch.long)
            for c in labels.unique():
                idx = (labels == c).nonzero().flatten()
                idx = idx[torch.randperm(len(idx), generator=g)]
                fold_of[idx] = torch.arange(len(idx)) % k
        elif strategy == "kfold":
            fold_of = torch.empty(n, dtype=torch.long); fold_of[torch.randperm(n, generator=g)] = torch.arange(n) % k
        else:
            raise ValueError(strategy)
        out += [((fold_of != f).nonzero().flatten(), (fold_of == f).nonzero().flatten()) for f in range(k)]
    return out


class ModelValidator:
    """Trains a fresh model per split (``make_model`` and ``train`` are the caller's) and evaluates it on the held-out part;
    results are summarised per metric with mean, deviation and a t-based confidence interval."""

    def __init__(self, strategy: str = "kfold", k: int = 5, task: str = "classification", seed: int = 0, **split_kw): self.strategy, self.k, self.task, self.seed, self.kw = strategy, k, task, seed, split_kw

    def _metrics(self, out: torch.Tensor, y: torch.Tensor) -> dict:
        if self.task == "classification":
            cm = ConfusionMatrix(out.shape[1]).update(out.argmax(1), y)
            return {**cm.summary("macro"), "loss": float(torch.nn.functional.cross_entropy(out, y))}
        err = out.squeeze(-1) - y
        return {"mse": float(err.pow(2).mean()), "mae": float(err.abs().mean()), "r2": float(1 - err.pow(2).sum() / (y - y.mean()).pow(2).sum().clamp_min(1e-12))}

    def validate(self, make_model: Callable[[], nn.Module], train: Callable[[nn.Module, torch.Tensor, torch.Tensor], None], x: torch.Tensor, y: torch.Tensor) -> dict:
        from scipy import stats
        splits = make_splits(len(x), self.strategy, self.k, labels=y if self.strategy == "stratified" else None, seed=self.seed, **self.kw)
        rows = []
        for tr, te in splits:
            m = make_model(); train(m, x[tr], y[tr]); m.eval()
            with torch.no_grad():
                rows.append({**self._metrics(m(x[te]), y[te]), "train_size": len(tr), "test_size": len(te)})
        summary = {}
        for key in rows[0]:
            if key.endswith("_size"):
                continue
            v = [r[key] for r in rows]
            mean, sd = statistics.fmean(v), statistics.stdev(v) if len(v) > 1 else 0.0
            half = stats.t.ppf(0.975, len(v) - 1) * sd / math.sqrt(len(v)) if len(v) > 1 else 0.0
            summary[key] = {"mean": mean, "std": sd, "min": min(v), "max": max(v), "ci95": (mean - half, mean + half)}
        return {"splits": rows, "summary": summary}


def tensors_close(a: torch.Tensor, b: torch.Tensor, rtol: float = 1e-5, atol: float = 1e-8, max_mismatch_fraction: float = 0.0) -> bool:
    if a.shape != b.shape:
        return False
    bad = ~torch.isclose(a.double(), b.double(), rtol=rtol, atol=atol, equal_nan=True)
    return float(bad.float().mean()) <= max_mismatch_fraction


def validate_model_correctness(model: nn.Module, reference: nn.Module | Callable, inputs: Sequence[torch.Tensor], **tol) -> dict:
    model.eval()
    with torch.no_grad():
        outs = [(model(i), reference(i)) for i in inputs]
    errs = [float((a.double() - b.double()).abs().max()) for a, b in outs]
    return {"passed": all(tensors_close(a, b, **tol) for a, b in outs), "max_abs_error": max(errs), "cases": len(inputs)}


# ================================================================================================ benchmark and comparison
def benchmark_model(model: nn.Module, example: torch.Tensor, warmup: int = 3, iterations: int = 20, batch_sizes: Sequence[int] | None = None) -> dict:
    from ..utils.bench_suite import Timer
    model.eval()
    timer, out = Timer(example.device.type), {}
    n_params = sum(p.numel() for p in model.parameters())
    for bs in batch_sizes or (example.shape[0],):
        x = example[:1].expand(bs, *example.shape[1:]).contiguous()
        with torch.no_grad():
            for _ in range(warmup):
                model(x)
            ts = sorted(timer.measure(lambda: model(x)) for _ in range(iterations))
        q = lambda p: ts[min(len(ts) - 1, int(p * len(ts)))]
        out[bs] = {"mean_ms": statistics.fmean(ts) * 1e3, "p50_ms": q(0.5) * 1e3, "p90_ms": q(0.9) * 1e3, "p99_ms": q(0.99) * 1e3, "throughput": bs / statistics.fmean(ts)}
    return {"parameters": n_params, "size_mb": sum(p.numel() * p.element_size() for p in model.parameters()) / 2 ** 20, "latency": out}


def one_way_anova(groups: Sequence[Sequence[float]]) -> dict:
    from scipy import stats
    k, n = len(groups), sum(len(g) for g in groups)
    grand = sum(sum(g) for g in groups) / n
    ssb = sum(len(g) * (statistics.fmean(g) - grand) ** 2 for g in groups)
    ssw = sum(sum((v - statistics.fmean(g)) ** 2 for v in g) for g in groups)
    f = (ssb / (k - 1)) / (ssw / (n - k)) if ssw > 0 else math.inf
    return {"f": f, "p": float(stats.f.sf(f, k - 1, n - k)), "df_between": k - 1, "df_within": n - k, "eta_squared": ssb / (ssb + ssw) if ssb + ssw else 0.0}


class ModelComparator:
    """Per-model samples of a quality metric (for example accuracy per fold) plus measured latency and size: ANOVA over the
    quality samples, pairwise Welch tests with Holm correction, a ranking per dimension, an overall ranking from weighted
    normalised scores, and the Pareto-optimal set of (quality, latency)."""

    def __init__(self, weights: dict | None = None, alpha: float = 0.05): self.w, self.alpha, self.models = weights or {"quality": 0.5, "latency": 0.3, "size": 0.2}, alpha, {}
    def add(self, name: str, quality_samples: Sequence[float], latency_ms: float, size_mb: float): self.models[name] = {"quality": list(quality_samples), "latency": latency_ms, "size": size_mb}; return self

    def compare(self) -> dict:
        from scipy import stats
        names = list(self.models)
        q = {n: statistics.fmean(self.models[n]["quality"]) for n in names}
        anova = one_way_anova([self.models[n]["quality"] for n in names]) if len(names) > 1 else None
        pairs = []
        for i, a in enumerate(names):
            for b in names[i + 1:]:
                t, p = stats.ttest_ind(self.models[a]["quality"], self.models[b]["quality"], equal_var=False)
                pairs.append({"a": a, "b": b, "diff": q[a] - q[b], "p": float(p)})
        for rank, pr in enumerate(sorted(pairs, key=lambda r: r["p"])):                # Holm step-down
            pr["p_adjusted"] = min(1.0, pr["p"] * (len(pairs) - rank))
        run = 0.0
        for pr in sorted(pairs, key=lambda r: r["p"]):
            run = max(run, pr["p_adjusted"]); pr["p_adjusted"] = run
            pr["significant"] = pr["p_adjusted"] < self.alpha
            pr["preferred"] = (pr["a"] if pr["diff"] > 0 else pr["b"]) if pr["significant"] else "no clear preference"
        norm = lambda vals, invert: {n: ((max(vals.values()) - v) if invert else (v - min(vals.values()))) / ((max(vals.values()) - min(vals.values())) or 1.0) for n, v in vals.items()}
        parts = {"quality": norm(q, False), "latency": norm({n: self.models[n]["latency"] for n in names}, True), "size": norm({n: self.models[n]["size"] for n in names}, True)}
        score = {n: sum(self.w[d] * parts[d][n] for d in parts) for n in names}
        pareto = [n for n in names if not any(q[m] >= q[n] and self.models[m]["latency"] <= self.models[n]["latency"] and (q[m] > q[n] or self.models[m]["latency"] < self.models[n]["latency"]) for m in names)]
        return {"quality": q, "anova": anova, "pairwise": pairs, "rankings": {d: sorted(names, key=lambda n: -parts[d][n]) for d in parts}, "overall": sorted(names, key=lambda n: -score[n]), "scores": score, "pareto": pareto}

    def export_csv(self, results: dict) -> str:
        buf = io.StringIO(); w = csv.writer(buf)
        w.writerow(["model", "quality", "latency_ms", "size_mb", "score", "pareto"])
        for n in results["overall"]:
            w.writerow([n, f"{results['quality'][n]:.6g}", self.models[n]["latency"], self.models[n]["size"], f"{results['scores'][n]:.4f}", n in results["pareto"]])
        return buf.getvalue()

    def html_report(self, results: dict, title: str = "Model comparison") -> str:
        rows = "".join(f"<tr><td>{html.escape(n)}</td><td>{results['quality'][n]:.4f}</td><td>{self.models[n]['latency']:.3g}</td><td>{self.models[n]['size']:.3g}</td><td>{results['scores'][n]:.3f}</td><td>{'yes' if n in results['pareto'] else ''}</td></tr>" for n in results["overall"])
        pw = "".join(f"<tr><td>{html.escape(p['a'])} vs {html.escape(p['b'])}</td><td>{p['diff']:+.4f}</td><td>{p['p_adjusted']:.3g}</td><td>{html.escape(p['preferred'])}</td></tr>" for p in results["pairwise"])
        an = f"<p>ANOVA: F = {results['anova']['f']:.3g}, p = {results['anova']['p']:.3g}</p>" if results["anova"] else ""
        return f"<html><body><h1>{html.escape(title)}</h1><table><tr><th>model</th><th>quality</th><th>latency ms</th><th>size MB</th><th>score</th><th>Pareto</th></tr>{rows}</table>{an}<h2>Pairwise</h2><table>{pw}</table></body></html>"


def optimization_recommendations(bench: dict, targets: dict) -> list[dict]:
    """From a :func:`benchmark_model` result and targets (``latency_ms``, ``size_mb``, ``throughput``): what to try, most
    valuable first."""
    recs = []
    lat = min(v["p50_ms"] for v in bench["latency"].values())
    if "size_mb" in targets and bench["size_mb"] > targets["size_mb"]:
        ratio = bench["size_mb"] / targets["size_mb"]
        recs.append({"priority": "high", "action": "bf16 weights" if ratio <= 2 else "int8 weight quantisation" if ratio <= 4 else "int4 quantisation or pruning plus distillation", "reason": f"model is {ratio:.1f}x the size target"})
    if "latency_ms" in targets and lat > targets["latency_ms"]:
        recs.append({"priority": "high", "action": "fuse element-wise chains and GEMM epilogues; run bf16 on tensor cores; capture the step in a CUDA graph", "reason": f"median latency {lat:.3g} ms exceeds {targets['latency_ms']:g} ms"})
    best = max(bench["latency"].items(), key=lambda kv: kv[1]["throughput"])
    if "throughput" in targets and best[1]["throughput"] < targets["throughput"]:
        recs.append({"priority": "medium", "action": f"raise the batch size beyond {best[0]} or shard across GPUs", "reason": f"peak throughput {best[1]['throughput']:.3g}/s below {targets['throughput']:g}/s"})
    if len(bench["latency"]) > 1:
        bs = sorted(bench["latency"])
        if bench["latency"][bs[-1]]["throughput"] < 1.2 * bench["latency"][bs[0]]["throughput"]:
            recs.append({"priority": "low", "action": "batching does not help: the model is already compute-bound at the smallest batch", "reason": "throughput is flat in the batch size"})
    return recs
