"""Benchmark harness and analysis (``crates/torsh-benches/src``): runner with device-event timing and L2 flushing
(``lib.rs``, ``utils.rs``), data generators, statistics / bottleneck / complexity analysis (``benchmark_analysis.rs``,
``advanced_analysis.rs``), result cache (``benchmark_cache.rs``, ``cached_runner.rs``), comparisons with significance
(``benchmark_comparison.rs``), output validation against reference implementations (``benchmark_validation.rs``), CI
gating with JUnit / Markdown artifacts (``ci_integration.rs``), change-point and trend regression detection
(``regression_detection.rs``), scalability sweeps with Amdahl fits (``scalability.rs``), system information
(``system_info.rs``), SVG charts, HTML reports and dashboards (``visualization.rs``, ``html_reporting.rs``,
``performance_dashboards.rs``), library comparisons (``numpy_comparisons.rs``, ``pytorch_comparisons.rs``), precision,
quantisation and pruning benchmarks (``precision_benchmarks.rs``), edge-deployment benchmarks (``edge_deployment.rs``,
``mobile_benchmarks.rs``) and hardware probes (``hardware_benchmarks.rs``)."""
from __future__ import annotations

import hashlib
import html
import json
import math
import os
import platform
import statistics
import sys
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Sequence

import torch


# ================================================================================================ runner
@dataclass
class BenchConfig:
    name: str
    sizes: Sequence[int] = (1024,)
    warmup: int = 3
    iterations: int = 10
    dtype: torch.dtype = torch.float32
    device: str = "cpu"
    flush_l2: bool = True
    metadata: dict = field(default_factory=dict)

    def key(self) -> str: return hashlib.sha256(json.dumps([self.name, list(self.sizes), self.warmup, self.iterations, str(self.dtype), self.device, self.metadata], sort_keys=True, default=str).encode()).hexdigest()[:16]


@dataclass
class BenchResult:
    name: str
    size: int
    times: list
    flops: float | None = None
    bytes: float | None = None
    metadata: dict = field(default_factory=dict)

    @property
    def mean(self): return statistics.fmean(self.times)
    @property
    def median(self): return statistics.median(self.times)
    @property
    def std(self): return statistics.stdev(self.times) if len(self.times) > 1 else 0.0
    @property
    def min(self): return min(self.times)
    def throughput(self): return self.size / self.median
    def gflops(self): return None if self.flops is None else self.flops / self.median / 1e9
    def gbps(self): return None if self.bytes is None else self.bytes / self.median / 1e9
    def to_dict(self): return {**asdict(self), "mean": self.mean, "median": self.median, "std": self.std, "min": self.min}


class Timer:
    """Times a callable: CUDA events on the current stream for device work (synchronised on both sides), the host's
    monotonic clock otherwise."""

    def __init__(self, device: str = "cpu"): self.cuda = str(device).startswith("cuda") and torch.cuda.is_available()

    def measure(self, fn: Callable[[], Any]) -> float:
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(); a.record(); fn(); b.record(); torch.cuda.synchronize()
            return a.elapsed_time(b) * 1e-3
        t0 = time.perf_counter(); fn()
        return time.perf_counter() - t0


class BenchRunner:
    """Runs objects with ``setup(size, config) -> state``, ``run(state)`` and optional ``flops(size)`` / ``bytes(size)``.  Between
    timed iterations on a GPU a buffer larger than the 126 MB L2 is rewritten so every iteration starts cold."""

    def __init__(self): self.results: list[BenchResult] = []

    def run(self, bench, config: BenchConfig) -> list[BenchResult]:
        timer, out = Timer(config.device), []
        flush = torch.empty(160 << 20, dtype=torch.uint8, device=config.device) if timer.cuda and config.flush_l2 else None
        for size in config.sizes:
            state = bench.setup(size, config)
            for _ in range(config.warmup):
                bench.run(state)
            times = []
            for _ in range(config.iterations):
                if flush is not None:
                    flush.zero_()
                times.append(timer.measure(lambda: bench.run(state)))
            out.append(BenchResult(config.name, size, times, getattr(bench, "flops", lambda s: None)(size), getattr(bench, "bytes", lambda s: None)(size), {"device": config.device, "dtype": str(config.dtype)}))
        self.results += out
        return out


class FunctionBench:
    def __init__(self, make_inputs: Callable, fn: Callable, flops: Callable | None = None, nbytes: Callable | None = None):
        self.make, self.fn = make_inputs, fn
        if flops:
            self.flops = flops
        if nbytes:
            self.bytes = nbytes
    def setup(self, size, config): return self.make(size, config)
    def run(self, state): return self.fn(*state)


class DataGenerator:
    def __init__(self, seed: int = 0): self.g = torch.Generator().manual_seed(seed)

    def tensor(self, shape, distribution: str = "normal", dtype=torch.float32, device="cpu", sparsity: float = 0.0, **kw) -> torch.Tensor:
        if distribution == "normal":
            x = torch.randn(shape, generator=self.g) * kw.get("std", 1.0) + kw.get("mean", 0.0)
        elif distribution == "uniform":
            x = torch.rand(shape, generator=self.g) * (kw.get("high", 1.0) - kw.get("low", 0.0)) + kw.get("low", 0.0)
        elif distribution == "lognormal":
            x = torch.randn(shape, generator=self.g).exp()
        elif distribution == "sequential":
            x = torch.arange(math.prod(shape), dtype=torch.float32).reshape(shape)
        elif distribution == "constant":
            x = torch.full(shape, float(kw.get("value", 1.0)))
        else:
            raise ValueError(distribution)
        if sparsity:
            x = x * (torch.rand(shape, generator=self.g) >= sparsity)
        return x.to(dtype).to(device)


class MemoryMonitor:
    def __init__(self, device="cpu"): self.device, self.samples = device, []
    def sample(self, label=""):
        import psutil
        b = torch.cuda.memory_allocated() if str(self.device).startswith("cuda") and torch.cuda.is_available() else psutil.Process().memory_info().rss
        self.samples.append((time.perf_counter(), b, label)); return b
    def peak(self): return max(b for _, b, _ in self.samples)
    def growth(self): return self.samples[-1][1] - self.samples[0][1]


# ================================================================================================ analysis
def summarize(times: Sequence[float], confidence_z: float = 1.96) -> dict:
    v = sorted(times); n = len(v)
    mean, sd = statistics.fmean(v), (statistics.stdev(v) if n > 1 else 0.0)
    q = lambda p: v[0] if n == 1 else v[int(p * (n - 1))] + (p * (n - 1) - int(p * (n - 1))) * (v[min(int(p * (n - 1)) + 1, n - 1)] - v[int(p * (n - 1))])
    q1, q3 = q(0.25), q(0.75)
    lo, hi = q1 - 1.5 * (q3 - q1), q3 + 1.5 * (q3 - q1)
    return {"n": n, "mean": mean, "median": q(0.5), "std": sd, "cv": sd / mean if mean else 0.0, "min": v[0], "max": v[-1], "p95": q(0.95), "p99": q(0.99), "iqr": q3 - q1,
            "ci": (mean - confidence_z * sd / math.sqrt(n), mean + confidence_z * sd / math.sqrt(n)), "outliers": [t for t in times if t < lo or t > hi]}


class BenchmarkAnalyzer:
    """Places results on a roofline given the machine's peaks, names the bottleneck, rates the efficiency and suggests what
    to change."""

    def __init__(self, peak_gflops: float, peak_gbps: float): self.pf, self.pb = peak_gflops, peak_gbps

    def analyze(self, r: BenchResult) -> dict:
        s = summarize(r.times)
        out = {"name": r.name, "size": r.size, "stats": s, "stable": s["cv"] < 0.05}
        if r.flops and r.bytes:
            intensity, ridge = r.flops / r.bytes, self.pf / self.pb
            roof = min(self.pf, intensity * self.pb)
            eff = r.gflops() / roof
            out.update(intensity=intensity, ridge=ridge, bottleneck="memory" if intensity < ridge else "compute", roofline_gflops=roof, efficiency=eff,
                       rating="excellent" if eff > 0.8 else "good" if eff > 0.6 else "fair" if eff > 0.3 else "poor")
            rec = []
            if eff < 0.3 and s["median"] < 2e-5:
                out["bottleneck"] = "launch"; rec.append("the call is launch-bound: batch more work per launch or capture the loop in a CUDA graph")
            elif out["bottleneck"] == "memory" and eff < 0.6:
                rec.append("memory-bound below 60 % of bandwidth: fuse with the producer, widen loads to 16 bytes, check coalescing")
            elif out["bottleneck"] == "compute" and eff < 0.6:
                rec.append("compute-bound below 60 % of peak: larger tiles, deeper pipeline, keep the tensor cores fed")
            if not out["stable"]:
                rec.append(f"coefficient of variation {s['cv']:.1%}: raise iterations or isolate the machine")
            out["recommendations"] = rec
        return out


COMPLEXITY_CLASSES = {"O(1)": lambda n: 1.0, "O(log n)": lambda n: math.log2(n), "O(n)": lambda n: n, "O(n log n)": lambda n: n * math.log2(n), "O(n^2)": lambda n: n ** 2, "O(n^3)": lambda n: n ** 3}


def fit_complexity(sizes: Sequence[int], times: Sequence[float]) -> dict:
    """Least-squares fit of ``t = a f(n) + b`` (``a, b >= 0``) for each candidate class; the class with the smallest relative residual wins.  The log-log
    slope is reported as well."""
    import numpy as np
    n, t = np.asarray(sizes, float), np.asarray(times, float)
    fits = {}
    for name, f in COMPLEXITY_CLASSES.items():
        x = np.array([f(v) for v in n])
        A = np.stack([x, np.ones_like(x)], 1)
        coef, *_ = np.linalg.lstsq(A, t, rcond=None)
        if coef[0] < 0 or coef[1] < 0:
            a = max(float(x @ t / (x @ x)), 0.0); coef = np.array([a, 0.0])
        fits[name] = float(np.sqrt(np.mean(((A @ coef - t) / t) ** 2)))
    slope = float(np.polyfit(np.log(n), np.log(t), 1)[0])
    best = min(fits, key=fits.get)
    return {"class": best, "residuals": fits, "loglog_slope": slope}


# ================================================================================================ cache
class BenchmarkCache:
    """Results on disk keyed by benchmark config and environment fingerprint; entries expire after ``ttl`` seconds."""

    def __init__(self, root, ttl: float = 24 * 3600, environment: dict | None = None, clock=time.time):
        self.root, self.ttl, self.clock = Path(root), ttl, clock
        self.root.mkdir(parents=True, exist_ok=True)
        self.env = hashlib.sha256(json.dumps(environment or {}, sort_keys=True).encode()).hexdigest()[:8]
        self.stats = {"hits": 0, "misses": 0, "expired": 0}

    def _path(self, config: BenchConfig): return self.root / f"{config.key()}-{self.env}.json"

    def get(self, config: BenchConfig):
        p = self._path(config)
        if not p.exists():
            self.stats["misses"] += 1; return None
        d = json.loads(p.read_text())
        if self.clock() - d["stored_at"] > self.ttl:
            self.stats["expired"] += 1; p.unlink(); return None
        self.stats["hits"] += 1
        return [BenchResult(**r) for r in d["results"]]

    def put(self, config: BenchConfig, results: Sequence[BenchResult]): self._path(config).write_text(json.dumps({"stored_at": self.clock(), "results": [asdict(r) for r in results]}))
    def clear(self): [p.unlink() for p in self.root.glob("*.json")]


class CachedBenchRunner(BenchRunner):
    def __init__(self, cache: BenchmarkCache): super().__init__(); self.cache = cache
    def run(self, bench, config):
        hit = self.cache.get(config)
        if hit is not None:
            return hit
        res = super().run(bench, config); self.cache.put(config, res)
        return res


# ================================================================================================ comparison
def welch_t(a: Sequence[float], b: Sequence[float]) -> tuple[float, float]:
    """Welch's t statistic and two-sided p-value (normal approximation above 30 degrees of freedom, Student t below)."""
    ma, mb, va, vb = statistics.fmean(a), statistics.fmean(b), statistics.variance(a), statistics.variance(b)
    se = math.sqrt(va / len(a) + vb / len(b)) or 1e-300
    t = (ma - mb) / se
    df = (va / len(a) + vb / len(b)) ** 2 / max((va / len(a)) ** 2 / (len(a) - 1) + (vb / len(b)) ** 2 / (len(b) - 1), 1e-300)
    from scipy import stats
    return t, float(2 * stats.t.sf(abs(t), df))


class BenchmarkComparator:
    def __init__(self, alpha: float = 0.05, min_effect: float = 0.02): self.alpha, self.min_effect = alpha, min_effect

    def compare(self, baseline: BenchResult, candidate: BenchResult) -> dict:
        speedup = baseline.median / candidate.median
        t, p = welch_t(baseline.times, candidate.times) if min(len(baseline.times), len(candidate.times)) > 1 else (0.0, 1.0)
        sig = p < self.alpha and abs(speedup - 1) > self.min_effect
        return {"name": candidate.name, "size": candidate.size, "speedup": speedup, "p_value": p, "significant": sig, "verdict": "faster" if sig and speedup > 1 else "slower" if sig else "equivalent"}

    def compare_sets(self, baseline: Sequence[BenchResult], candidate: Sequence[BenchResult]) -> dict:
        base = {(r.name, r.size): r for r in baseline}
        rows = [self.compare(base[(r.name, r.size)], r) for r in candidate if (r.name, r.size) in base]
        geo = math.exp(statistics.fmean(math.log(r["speedup"]) for r in rows)) if rows else 1.0
        return {"rows": rows, "geomean_speedup": geo, "faster": sum(r["verdict"] == "faster" for r in rows), "slower": sum(r["verdict"] == "slower" for r in rows), "equivalent": sum(r["verdict"] == "equivalent" for r in rows)}


# ================================================================================================ validation
class BenchmarkValidator:
    """Checks that what a benchmark timed is the right computation: output against a float64 reference, determinism across
    runs, stability of timings."""

    def __init__(self, rtol: float = 1e-4, atol: float = 1e-6, max_cv: float = 0.1): self.rtol, self.atol, self.max_cv = rtol, atol, max_cv

    def numerical_accuracy(self, out: torch.Tensor, ref: torch.Tensor) -> dict:
        o, r = out.double(), ref.double()
        err = (o - r).abs()
        rel = err / r.abs().clamp_min(1e-30)
        return {"max_abs": float(err.max()), "max_rel": float(rel[r.abs() > self.atol].max()) if (r.abs() > self.atol).any() else 0.0, "rmse": float(err.pow(2).mean().sqrt()),
                "ok": bool(torch.allclose(o, r, rtol=self.rtol, atol=self.atol)), "non_finite": int((~torch.isfinite(o)).sum())}

    def validate(self, name: str, fn: Callable, reference: Callable, inputs: Sequence[torch.Tensor], times: Sequence[float] | None = None) -> dict:
        issues = []
        out, out2 = fn(*inputs), fn(*inputs)
        acc = self.numerical_accuracy(out, reference(*[i.double() if i.is_floating_point() else i for i in inputs]))
        if not acc["ok"]:
            issues.append({"severity": "error", "category": "accuracy", "message": f"max abs error {acc['max_abs']:.3g}, max rel {acc['max_rel']:.3g}"})
        if acc["non_finite"]:
            issues.append({"severity": "error", "category": "overflow", "message": f"{acc['non_finite']} non-finite outputs"})
        if not torch.equal(out, out2):
            issues.append({"severity": "warning", "category": "determinism", "message": "two runs on the same inputs differ"})
        if times is not None and summarize(times)["cv"] > self.max_cv:
            issues.append({"severity": "warning", "category": "consistency", "message": f"timing cv {summarize(times)['cv']:.1%} above {self.max_cv:.0%}"})
        return {"name": name, "accuracy": acc, "issues": issues, "status": "failed" if any(i["severity"] == "error" for i in issues) else "warning" if issues else "passed"}


def cancellation_risk(a: torch.Tensor, b: torch.Tensor) -> float:
    """Fraction of entries where ``a - b`` loses more than half of the significand bits."""
    d, m = (a - b).abs(), torch.maximum(a.abs(), b.abs())
    bits = torch.finfo(a.dtype).bits - {torch.float32: 9, torch.float64: 12, torch.float16: 6, torch.bfloat16: 9}[a.dtype]
    return float(((d > 0) & (d < m * 2.0 ** (-bits / 2))).float().mean())


# ================================================================================================ CI gating
@dataclass
class CIConfig:
    warn_slowdown: float = 0.05
    fail_slowdown: float = 0.15
    min_speedup_note: float = 0.05
    require_significance: bool = True


class CIBenchmarkRunner:
    def __init__(self, config: CIConfig | None = None): self.cfg, self.cmp = config or CIConfig(), BenchmarkComparator()

    def evaluate(self, baseline: Sequence[BenchResult], candidate: Sequence[BenchResult]) -> dict:
        rows = []
        for r in self.cmp.compare_sets(baseline, candidate)["rows"]:
            slow = 1 / r["speedup"] - 1
            real = r["significant"] or not self.cfg.require_significance
            status = "fail" if real and slow > self.cfg.fail_slowdown else "warn" if real and slow > self.cfg.warn_slowdown else "improved" if real and -slow > self.cfg.min_speedup_note else "pass"
            rows.append({**r, "slowdown": slow, "status": status})
        overall = "fail" if any(r["status"] == "fail" for r in rows) else "warn" if any(r["status"] == "warn" for r in rows) else "pass"
        return {"status": overall, "exit_code": 1 if overall == "fail" else 0, "rows": rows}

    @staticmethod
    def junit_xml(decision: dict, suite: str = "benchmarks") -> str:
        cases = []
        for r in decision["rows"]:
            body = f'<failure message="{r["slowdown"]:+.1%} slower (p={r["p_value"]:.3g})"/>' if r["status"] == "fail" else ""
            cases.append(f'  <testcase classname="{suite}" name="{html.escape(r["name"])}[{r["size"]}]">{body}</testcase>')
        fails = sum(r["status"] == "fail" for r in decision["rows"])
        return f'<?xml version="1.0"?>\n<testsuite name="{suite}" tests="{len(cases)}" failures="{fails}">\n' + "\n".join(cases) + "\n</testsuite>\n"

    @staticmethod
    def markdown(decision: dict) -> str:
        icon = {"pass": "ok", "warn": "WARN", "fail": "FAIL", "improved": "faster"}
        rows = "\n".join(f"| {r['name']} | {r['size']} | {r['speedup']:.3f}x | {r['p_value']:.3g} | {icon[r['status']]} |" for r in decision["rows"])
        return f"### Benchmarks: {decision['status'].upper()}\n\n| benchmark | size | speedup | p | status |\n|---|---|---|---|---|\n{rows}\n"

    @staticmethod
    def annotations(decision: dict) -> list[str]:
        return [f"::{'error' if r['status'] == 'fail' else 'warning'} title=benchmark {r['name']}::{r['slowdown']:+.1%} slower at size {r['size']}" for r in decision["rows"] if r["status"] in ("fail", "warn")]


# ================================================================================================ regression detection over history
class AdvancedRegressionDetector:
    """History of one metric (lower is better): CUSUM change point, Mann-Kendall trend, severity of the latest level against
    the level before the change."""

    def __init__(self, min_history: int = 8, threshold_sigmas: float = 4.0): self.min_history, self.k = min_history, threshold_sigmas

    @staticmethod
    def change_point(v: Sequence[float]) -> tuple[int, float]:
        mean = statistics.fmean(v)
        s, cum = 0.0, []
        for x in v:
            s += x - mean; cum.append(s)
        i = max(range(len(cum) - 1), key=lambda j: abs(cum[j]))
        return i + 1, abs(cum[i])

    @staticmethod
    def mann_kendall(v: Sequence[float]) -> tuple[float, float]:
        n = len(v)
        s = sum((v[j] > v[i]) - (v[j] < v[i]) for i in range(n) for j in range(i + 1, n))
        var = n * (n - 1) * (2 * n + 5) / 18
        z = (s - (s > 0) + (s < 0)) / math.sqrt(var) if var else 0.0
        return z, math.erfc(abs(z) / math.sqrt(2))

    def analyze(self, history: Sequence[float]) -> dict:
        if len(history) < self.min_history:
            return {"status": "insufficient_history"}
        cp, _ = self.change_point(history)
        before, after = history[:cp], history[cp:]
        out = {"trend_z": (mk := self.mann_kendall(history))[0], "trend_p": mk[1], "trend": "degrading" if mk[1] < 0.05 and mk[0] > 0 else "improving" if mk[1] < 0.05 else "stable"}
        if len(before) >= 3 and len(after) >= 2:
            sd = statistics.stdev(before) or 1e-12 * abs(statistics.fmean(before)) or 1e-12
            shift = statistics.fmean(after) - statistics.fmean(before)
            rel = shift / statistics.fmean(before)
            if abs(shift) > self.k * sd / math.sqrt(min(len(before), len(after))) and abs(rel) > 0.02:
                out.update(change_point=cp, shift=rel, kind="regression" if shift > 0 else "improvement", severity="critical" if rel > 0.5 else "major" if rel > 0.2 else "moderate" if rel > 0.1 else "minor")
                out["status"] = out["kind"]
                return out
        out["status"] = "stable"
        return out


# ================================================================================================ scalability
def size_progression(kind: str, start: int, stop: int, steps: int = 8) -> list[int]:
    if kind == "linear":
        return [round(start + i * (stop - start) / (steps - 1)) for i in range(steps)]
    if kind == "exponential":
        return sorted({round(start * (stop / start) ** (i / (steps - 1))) for i in range(steps)})
    if kind == "power_of_two":
        return [1 << p for p in range(math.ceil(math.log2(start)), math.floor(math.log2(stop)) + 1)]
    raise ValueError(kind)


def amdahl_fit(workers: Sequence[int], times: Sequence[float]) -> dict:
    """Serial fraction ``s`` of ``T(p) = T1 (s + (1 - s) / p)`` by least squares; also per-point speedup and efficiency."""
    import numpy as np
    p, t = np.asarray(workers, float), np.asarray(times, float)
    t1 = t[p == p.min()][0] * p.min()
    y, x = t / t1 - 1 / p, 1 - 1 / p
    s = float(np.clip((x @ y) / max(x @ x, 1e-30), 0, 1))
    speed = t[0] * p[0] / t / p.min() if p.min() == 1 else t[0] / t
    return {"serial_fraction": s, "max_speedup": 1 / s if s > 0 else math.inf, "speedup": speed.tolist(), "efficiency": (speed / (p / p.min())).tolist()}


class ScalabilityTestSuite:
    def __init__(self, runner: BenchRunner | None = None): self.runner = runner or BenchRunner()

    def size_sweep(self, bench, config: BenchConfig) -> dict:
        res = self.runner.run(bench, config)
        sizes, times = [r.size for r in res], [r.median for r in res]
        per = [t / s for s, t in zip(sizes, times)]
        return {"results": res, "complexity": fit_complexity(sizes, times) if len(sizes) >= 3 else None, "time_per_element": per, "knee": self._knee(sizes, per)}

    @staticmethod
    def _knee(sizes, per):
        """First size at which the cost per element jumps by more than 50 % over the best seen so far (a working set leaving a
        cache level)."""
        best = per[0]
        for s, p in zip(sizes[1:], per[1:]):
            if p > 1.5 * best:
                return s
            best = min(best, p)
        return None

    @staticmethod
    def weak_scaling(workers: Sequence[int], throughput: Sequence[float]) -> list[float]: return [t / (throughput[0] * w / workers[0]) for w, t in zip(workers, throughput)]


# ================================================================================================ system information
def system_info() -> dict:
    import psutil
    info = {"platform": platform.platform(), "machine": platform.machine(), "python": sys.version.split()[0], "torch": torch.__version__, "cpu_count": os.cpu_count(), "physical_cores": psutil.cpu_count(logical=False),
            "memory_gb": round(psutil.virtual_memory().total / 2 ** 30, 1), "cuda_build": torch.version.cuda, "threads": torch.get_num_threads(), "gpus": []}
    try:
        import cpuinfo
        info["cpu"] = cpuinfo.get_cpu_info().get("brand_raw")
    except Exception:
        info["cpu"] = platform.processor()
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            info["gpus"].append({"name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count, "memory_gb": round(p.total_memory / 2 ** 30, 1)})
    info["fingerprint"] = hashlib.sha256(json.dumps({k: info[k] for k in ("machine", "cpu", "cpu_count", "torch", "cuda_build", "gpus")}, sort_keys=True).encode()).hexdigest()[:12]
    return info


# ================================================================================================ charts, reports, dashboards
class Chart:
    """Self-contained SVG line or bar chart with optional log axes."""
    PALETTE = ("#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b")

    def __init__(self, title: str, kind: str = "line", x_label: str = "", y_label: str = "", log_x: bool = False, log_y: bool = False, width: int = 640, height: int = 360):
        self.title, self.kind, self.xl, self.yl, self.lx, self.ly, self.w, self.h, self.series, self.notes = title, kind, x_label, y_label, log_x, log_y, width, height, [], []

    def add_series(self, name: str, xs: Sequence, ys: Sequence[float]): self.series.append((name, list(xs), list(ys))); return self
    def annotate(self, x, y, text): self.notes.append((x, y, text)); return self

    def to_svg(self) -> str:
        L, R, T, B = 60, 20, 30, 45
        pw, ph = self.w - L - R, self.h - T - B
        fx = (lambda v: math.log10(v)) if self.lx else float
        fy = (lambda v: math.log10(v)) if self.ly else float
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{self.w}" height="{self.h}" font-family="sans-serif" font-size="11">', f'<text x="{self.w / 2}" y="16" text-anchor="middle" font-size="14">{html.escape(self.title)}</text>',
               f'<rect x="{L}" y="{T}" width="{pw}" height="{ph}" fill="none" stroke="#888"/>']
        ys_all = [fy(y) for _, _, ys in self.series for y in ys]
        y0, y1 = (0.0 if self.kind == "bar" and not self.ly else min(ys_all)), max(ys_all)
        y1 = y1 if y1 > y0 else y0 + 1
        py = lambda v: T + ph - (fy(v) - y0) / (y1 - y0) * ph
        if self.kind == "bar":
            cats = self.series[0][1]
            gw = pw / len(cats); bw = gw * 0.8 / len(self.series)
            for si, (name, _, ys) in enumerate(self.series):
                for ci, y in enumerate(ys):
                    out.append(f'<rect class="bar" x="{L + ci * gw + gw * 0.1 + si * bw:.1f}" y="{py(y):.1f}" width="{bw:.1f}" height="{T + ph - py(y):.1f}" fill="{self.PALETTE[si % 6]}"><title>{html.escape(str(name))}: {y:.4g}</title></rect>')
            for ci, c in enumerate(cats):
                out.append(f'<text x="{L + (ci + 0.5) * gw:.1f}" y="{T + ph + 14}" text-anchor="middle">{html.escape(str(c))}</text>')
        else:
            xs_all = [fx(x) for _, xs, _ in self.series for x in xs]
            x0, x1 = min(xs_all), max(xs_all)
            x1 = x1 if x1 > x0 else x0 + 1
            px = lambda v: L + (fx(v) - x0) / (x1 - x0) * pw
            for si, (name, xs, ys) in enumerate(self.series):
                pts = " ".join(f"{px(x):.1f},{py(y):.1f}" for x, y in zip(xs, ys))
                out.append(f'<polyline class="series" fill="none" stroke="{self.PALETTE[si % 6]}" stroke-width="2" points="{pts}"/>')
            for x in (min((x for _, xs, _ in self.series for x in xs)), max((x for _, xs, _ in self.series for x in xs))):
                out.append(f'<text x="{px(x):.1f}" y="{T + ph + 14}" text-anchor="middle">{x:g}</text>')
            for x, y, text in self.notes:
                out.append(f'<text class="note" x="{px(x):.1f}" y="{py(y) - 4:.1f}" fill="#c00">{html.escape(text)}</text>')
        for frac in (0, 0.5, 1):
            val = y0 + frac * (y1 - y0)
            out.append(f'<text x="{L - 4}" y="{T + ph - frac * ph + 4:.1f}" text-anchor="end">{(10 ** val if self.ly else val):.3g}</text>')
        for si, (name, _, _) in enumerate(self.series):
            out.append(f'<text x="{L + 8}" y="{T + 14 + 13 * si}" fill="{self.PALETTE[si % 6]}">{html.escape(str(name))}</text>')
        out += [f'<text x="{L + pw / 2}" y="{self.h - 6}" text-anchor="middle">{html.escape(self.xl)}</text>', f'<text x="12" y="{T + ph / 2}" text-anchor="middle" transform="rotate(-90 12 {T + ph / 2})">{html.escape(self.yl)}</text>', "</svg>"]
        return "\n".join(out)


class HtmlReportGenerator:
    def __init__(self, title: str = "Benchmark report", theme: str = "light"): self.title, self.theme, self.sections = title, theme, []

    def add_results(self, heading: str, results: Sequence[BenchResult], analyzer: BenchmarkAnalyzer | None = None):
        head = ["benchmark", "size", "median", "mean", "std", "GFLOP/s", "GB/s"] + (["bound", "efficiency"] if analyzer else [])
        rows = []
        for r in results:
            row = [r.name, r.size, f"{r.median * 1e3:.4g} ms", f"{r.mean * 1e3:.4g} ms", f"{r.std * 1e3:.3g} ms", f"{r.gflops():.4g}" if r.flops else "-", f"{r.gbps():.4g}" if r.bytes else "-"]
            if analyzer:
                a = analyzer.analyze(r)
                row += [a.get("bottleneck", "-"), f"{a['efficiency']:.0%}" if "efficiency" in a else "-"]
            rows.append(row)
        table = "<table><tr>" + "".join(f"<th>{h}</th>" for h in head) + "</tr>" + "".join("<tr>" + "".join(f"<td>{html.escape(str(c))}</td>" for c in row) + "</tr>" for row in rows) + "</table>"
        self.sections.append(f"<h2>{html.escape(heading)}</h2>{table}"); return self

    def add_chart(self, chart: Chart): self.sections.append(chart.to_svg()); return self
    def add_text(self, heading: str, text: str): self.sections.append(f"<h2>{html.escape(heading)}</h2><pre>{html.escape(text)}</pre>"); return self

    def add_system(self, info: dict | None = None):
        info = info or system_info()
        self.sections.append("<h2>System</h2><ul>" + "".join(f"<li><b>{html.escape(k)}</b>: {html.escape(str(v))}</li>" for k, v in info.items()) + "</ul>"); return self

    def render(self) -> str:
        bg, fg = ("#111", "#eee") if self.theme == "dark" else ("#fff", "#111")
        return (f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(self.title)}</title><style>body{{background:{bg};color:{fg};font-family:sans-serif;margin:2em}}"
                f"table{{border-collapse:collapse}}td,th{{border:1px solid #888;padding:3px 8px}}</style></head><body><h1>{html.escape(self.title)}</h1>" + "\n".join(self.sections) + "</body></html>")

    def save(self, path): Path(path).write_text(self.render()); return path


class PerformanceDashboard:
    """History of runs (one JSON line per run) rendered as one page: a trend chart per metric with regressions marked."""

    def __init__(self, path): self.path = Path(path)

    def record(self, run_id: str, metrics: dict[str, float], timestamp: float | None = None):
        with self.path.open("a") as f:
            f.write(json.dumps({"run": run_id, "t": timestamp if timestamp is not None else time.time(), "metrics": metrics}) + "\n")

    def history(self) -> dict[str, list]:
        out: dict[str, list] = {}
        if self.path.exists():
            for line in self.path.read_text().splitlines():
                d = json.loads(line)
                for k, v in d["metrics"].items():
                    out.setdefault(k, []).append((d["run"], v))
        return out

    def render(self, title: str = "Performance dashboard") -> str:
        rep, det = HtmlReportGenerator(title), AdvancedRegressionDetector()
        summary = []
        for name, pts in self.history().items():
            vals = [v for _, v in pts]
            ch = Chart(name, x_label="run", y_label=name).add_series(name, range(len(vals)), vals)
            a = det.analyze(vals)
            if a.get("status") in ("regression", "improvement"):
                ch.annotate(a["change_point"], vals[a["change_point"]], f"{a['kind']} {a['shift']:+.0%}")
            summary.append(f"{name}: {a['status']}")
            rep.add_chart(ch)
        rep.sections.insert(0, "<ul>" + "".join(f"<li>{html.escape(s)}</li>" for s in summary) + "</ul>")
        return rep.render()


# ================================================================================================ library comparisons
class ComparisonRunner:
    """Times the same operation in several libraries on identical data (NumPy on the host, stock PyTorch, this package) and
    checks that they agree."""

    def __init__(self, iterations: int = 5, warmup: int = 2): self.it, self.wu, self.impls = iterations, warmup, {}
    def register(self, library: str, op: str, fn: Callable, convert: Callable = lambda t: t): self.impls.setdefault(op, {})[library] = (fn, convert)

    def with_defaults(self):
        import numpy as np
        for op, (nf, tf) in {"matmul": (np.matmul, torch.matmul), "add": (np.add, torch.add), "exp": (np.exp, torch.exp), "sum": (lambda a: np.sum(a), lambda a: torch.sum(a))}.items():
            self.register("numpy", op, nf, lambda t: t.numpy()); self.register("torch", op, tf)
        return self

    def run(self, op: str, inputs: Sequence[torch.Tensor], baseline: str = "torch") -> dict:
        rows, outs = {}, {}
        for lib, (fn, conv) in self.impls[op].items():
            args = [conv(i) for i in inputs]
            for _ in range(self.wu):
                fn(*args)
            ts = []
            for _ in range(self.it):
                t0 = time.perf_counter(); o = fn(*args); ts.append(time.perf_counter() - t0)
            outs[lib] = torch.as_tensor(o).double()
            rows[lib] = {"median": statistics.median(ts), "times": ts}
        for lib in rows:
            rows[lib]["speedup_vs_baseline"] = rows[baseline]["median"] / rows[lib]["median"]
            rows[lib]["max_diff_vs_baseline"] = float((outs[lib] - outs[baseline]).abs().max())
        return rows


# ================================================================================================ precision, quantisation, pruning
def precision_benchmark(fn: Callable, inputs: Sequence[torch.Tensor], dtypes=(torch.float32, torch.bfloat16, torch.float16), iterations: int = 5) -> dict:
    """Error against float64 and time for each compute dtype."""
    ref = fn(*[i.double() for i in inputs])
    out = {}
    for dt in dtypes:
        args = [i.to(dt) for i in inputs]
        fn(*args)
        t = statistics.median(Timer(inputs[0].device.type).measure(lambda: fn(*args)) for _ in range(iterations))
        r = fn(*args).double()
        out[str(dt).replace("torch.", "")] = {"time": t, "rel_error": float((r - ref).norm() / ref.norm()), "max_abs_error": float((r - ref).abs().max()), "overflow": int((~torch.isfinite(r)).sum())}
    return out


def quantization_benchmark(w: torch.Tensor, x: torch.Tensor, bits=(8, 4), per_channel: bool = True) -> dict:
    """Symmetric weight quantisation: bytes, compression, weight SQNR and output error of ``x @ w.T``."""
    ref, out = x @ w.t(), {}
    for b in bits:
        qmax = 2 ** (b - 1) - 1
        scale = (w.abs().amax(1, keepdim=True) if per_channel else w.abs().max()) / qmax
        q = (w / scale).round().clamp(-qmax - 1, qmax)
        dq = q * scale
        out[f"int{b}"] = {"bytes": w.numel() * b / 8 + scale.numel() * 4, "compression": w.numel() * w.element_size() / (w.numel() * b / 8 + scale.numel() * 4),
                          "sqnr_db": float(10 * torch.log10(w.pow(2).sum() / (w - dq).pow(2).sum())), "output_rel_error": float((x @ dq.t() - ref).norm() / ref.norm())}
    return out


def pruning_benchmark(w: torch.Tensor, x: torch.Tensor, sparsities=(0.5, 0.75, 0.9), method: str = "magnitude") -> dict:
    ref, out = x @ w.t(), {}
    for s in sparsities:
        if method == "magnitude":
            th = w.abs().flatten().kthvalue(max(1, int(s * w.numel()))).values
            mask = w.abs() > th
        elif method == "2:4":
            g = w.reshape(-1, 4)
            mask = torch.zeros_like(g, dtype=torch.bool).scatter_(1, g.abs().topk(2, 1).indices, True).reshape(w.shape)
        else:
            mask = torch.rand_like(w) >= s
        out[s] = {"achieved_sparsity": float(1 - mask.float().mean()), "output_rel_error": float((x @ (w * mask).t() - ref).norm() / ref.norm()), "dense_flops": 2 * x.shape[0] * w.numel(), "sparse_flops": 2 * x.shape[0] * int(mask.sum())}
    return out


# ================================================================================================ edge deployment
@dataclass
class EdgeProfile:
    name: str = "generic-edge"
    memory_limit_mb: float = 512.0
    power_watts: float = 5.0
    battery_wh: float = 15.0
    target_latency_ms: float = 50.0


def edge_inference_benchmark(model: torch.nn.Module, example: torch.Tensor, profile: EdgeProfile | None = None, iterations: int = 10, inferences_per_hour: float = 3600.0) -> dict:
    """Batch-1 latency, model and activation footprint against the device's memory limit, energy per inference and the
    battery life it implies at the given duty cycle."""
    profile = profile or EdgeProfile()
    model.eval()
    sizes = []
    hooks = [m.register_forward_hook(lambda m, i, o: sizes.append(o.numel() * o.element_size()) if isinstance(o, torch.Tensor) else None) for m in model.modules() if not list(m.children())]
    with torch.no_grad():
        model(example)
        for h in hooks:
            h.remove()
        ts = [Timer(example.device.type).measure(lambda: model(example)) for _ in range(iterations)]
    lat = statistics.median(ts)
    weights = sum(p.numel() * p.element_size() for p in model.parameters()) + sum(b.numel() * b.element_size() for b in model.buffers())
    peak_act = max(sizes) * 2 if sizes else 0
    energy_j = profile.power_watts * lat
    duty_w = energy_j * inferences_per_hour / 3600.0
    return {"profile": profile.name, "latency_ms": lat * 1e3, "p95_ms": sorted(ts)[int(0.95 * (len(ts) - 1))] * 1e3, "meets_latency": lat * 1e3 <= profile.target_latency_ms, "model_mb": weights / 2 ** 20, "peak_activation_mb": peak_act / 2 ** 20,
            "fits_memory": (weights + peak_act) / 2 ** 20 <= profile.memory_limit_mb, "energy_mj": energy_j * 1e3, "battery_hours": profile.battery_wh / duty_w if duty_w else math.inf, "throughput_per_s": 1 / lat}


# ================================================================================================ hardware probes
def hardware_probes(device: str = "cpu", mb: int = 64, n: int = 512, iterations: int = 5) -> dict:
    """Copy and triad bandwidth and matmul throughput of the device (small defaults so it finishes in a moment on a host)."""
    timer = Timer(device)
    a = torch.ones(mb * (1 << 20) // 4, device=device); b = torch.empty_like(a); c = torch.ones_like(a)
    med = lambda f: statistics.median(timer.measure(f) for _ in range(iterations))
    b.copy_(a)
    t_copy, t_triad = med(lambda: b.copy_(a)), med(lambda: torch.add(a, c, alpha=3.0, out=b))
    x, y = torch.randn(n, n, device=device), torch.randn(n, n, device=device)
    x @ y
    t_mm = med(lambda: x @ y)
    return {"copy_gbps": 2 * a.numel() * 4 / t_copy / 1e9, "triad_gbps": 3 * a.numel() * 4 / t_triad / 1e9, "matmul_gflops": 2 * n ** 3 / t_mm / 1e9, "ridge_flops_per_byte": (2 * n ** 3 / t_mm) / (2 * a.numel() * 4 / t_copy)}
