"""Analysis layers over recorded profile events (``crates/torsh-profiler/src``): workload characterisation
(``workload_characterization.rs``), statistical / learned analysis (``ml_analysis.rs``), streaming statistics, anomaly and
drift detection and online prediction (``online_learning.rs``), allocation forecasting and adaptive pools
(``memory_optimization.rs``), a low-overhead recorder with sampling, interning and a ring buffer (``optimization.rs``),
baseline regression detection (``regression.rs``), templated reports (``reporting.rs``), prioritised event streaming with
rate control (``streaming.rs``), schema-driven export (``custom_export.rs``), external tool registry (``custom_tools.rs``),
flame graphs, profiling decorators (``attributes.rs``) and the profiler that ties them together
(``integrated_profiler.rs``).  Events are :class:`torsh_b200.utils.profiler.ProfileEvent` records or dicts with the same keys."""
from __future__ import annotations

import asyncio
import functools
import gzip
import heapq
import html
import json
import math
import statistics
import time
import zlib
from collections import Counter, defaultdict, deque
from dataclasses import asdict, is_dataclass
from typing import Callable, Iterable, Sequence

import numpy as np


def _ev(e) -> dict:
    return asdict(e) if is_dataclass(e) else dict(e)


# ================================================================================================ workload characterisation
class WorkloadCharacterizer:
    """Classifies a trace: per-event arithmetic intensity against a machine balance point decides compute- or
    memory-bound; category shares give the workload type; gaps between events give idle time; overlap gives parallelism;
    a change in the dominant category over windows marks phase changes."""

    def __init__(self, peak_flops: float = 1.4e15, peak_bandwidth: float = 6.6e12, window: int = 50):
        self.balance, self.peak_flops, self.peak_bw, self.window = peak_flops / peak_bandwidth, peak_flops, peak_bandwidth, window

    def analyze(self, events: Iterable) -> dict:
        ev = sorted((_ev(e) for e in events), key=lambda e: e["start_us"])
        if not ev:
            return {"workload_type": "empty"}
        total = sum(e["duration_us"] for e in ev)
        by_cat: dict[str, float] = defaultdict(float)
        bound = Counter()
        for e in ev:
            by_cat[e.get("category", "op")] += e["duration_us"]
            if e.get("flops") and e.get("bytes"):
                bound["compute" if e["flops"] / e["bytes"] >= self.balance else "memory"] += e["duration_us"]
        shares = {k: v / total for k, v in by_cat.items()}
        comm, io = shares.get("communication", 0) + shares.get("collective", 0), shares.get("io", 0) + shares.get("data", 0)
        kind = ("communication_bound" if comm > 0.4 else "io_bound" if io > 0.4 else
                "compute_bound" if bound["compute"] > bound["memory"] else "memory_bound" if bound["memory"] else "mixed")
        span = max(e["start_us"] + e["duration_us"] for e in ev) - ev[0]["start_us"]
        # busy time = union of intervals; parallelism = summed duration / busy time
        busy, end = 0.0, -math.inf
        for e in ev:
            s, t = e["start_us"], e["start_us"] + e["duration_us"]
            if s > end:
                busy, end = busy + (t - s), t
            elif t > end:
                busy, end = busy + (t - end), t
        phases, prev = [], None
        for i in range(0, len(ev), self.window):
            w = ev[i:i + self.window]
            dom = Counter()
            for e in w:
                dom[e.get("category", "op")] += e["duration_us"]
            top = dom.most_common(1)[0][0]
            if top != prev:
                phases.append({"at_event": i, "start_us": w[0]["start_us"], "dominant": top})
                prev = top
        hot = Counter()
        for e in ev:
            hot[e["name"]] += e["duration_us"]
        achieved = [(e["flops"] / (e["duration_us"] * 1e-6)) / self.peak_flops for e in ev if e.get("flops") and e["duration_us"] > 0]
        recs = []
        if kind == "memory_bound":
            recs.append("fuse element-wise operations into their producers; keep tensors resident across kernels")
        if kind == "communication_bound":
            recs.append("overlap collectives with compute on a side stream or fuse them into the producing kernel")
        if span > 0 and busy / span < 0.7:
            recs.append(f"{1 - busy / span:.0%} of the span is idle: capture the launch-bound region in a CUDA graph")
        return {"workload_type": kind, "category_shares": shares, "bound_time_us": dict(bound), "parallelism": total / busy if busy else 0.0,
                "idle_fraction": 1 - busy / span if span else 0.0, "phases": phases, "hotspots": hot.most_common(5),
                "mean_compute_efficiency": float(np.mean(achieved)) if achieved else None, "recommendations": recs}

    @staticmethod
    def critical_path(tasks: dict[str, float], deps: dict[str, Sequence[str]]) -> tuple[float, list[str]]:
        """Longest path through a task DAG given durations and ``task -> prerequisites``."""
        order, seen = [], set()
        def visit(t):
            if t in seen:
                return
            seen.add(t)
            for d in deps.get(t, ()):
                visit(d)
            order.append(t)
        for t in tasks:
            visit(t)
        finish, via = {}, {}
        for t in order:
            best = max(deps.get(t, ()), key=lambda d: finish[d], default=None)
            finish[t], via[t] = tasks[t] + (finish[best] if best else 0.0), best
        end = max(finish, key=finish.get)
        path = []
        while end is not None:
            path.append(end)
            end = via[end]
        return max(finish.values()), path[::-1]


# ================================================================================================ statistical / learned analysis
class MLAnalyzer:
    def extract_features(self, events: Iterable) -> tuple[list[str], np.ndarray]:
        """One row per operation name: count, mean / std / p95 duration, total share, mean flops and bytes."""
        groups: dict[str, list] = defaultdict(list)
        for e in map(_ev, events):
            groups[e["name"]].append(e)
        total = sum(e["duration_us"] for g in groups.values() for e in g) or 1.0
        names, rows = sorted(groups), []
        for n in names:
            d = np.array([e["duration_us"] for e in groups[n]])
            rows.append([len(d), d.mean(), d.std(), np.percentile(d, 95), d.sum() / total, np.mean([e.get("flops", 0) for e in groups[n]]), np.mean([e.get("bytes", 0) for e in groups[n]])])
        return names, np.array(rows)

    @staticmethod
    def detect_anomalies(values: Sequence[float], method: str = "mad", threshold: float = 3.5) -> list[int]:
        v = np.asarray(values, dtype=float)
        if method == "zscore":
            return np.nonzero(np.abs(v - v.mean()) > threshold * max(v.std(), 1e-12))[0].tolist()
        if method == "iqr":
            q1, q3 = np.percentile(v, [25, 75])
            return np.nonzero((v < q1 - 1.5 * (q3 - q1)) | (v > q3 + 1.5 * (q3 - q1)))[0].tolist()
        med = np.median(v)
        mad = np.median(np.abs(v - med)) or 1e-12
        return np.nonzero(0.6745 * np.abs(v - med) / mad > threshold)[0].tolist()

    @staticmethod
    def cluster_operations(features: np.ndarray, k: int = 3, iters: int = 50, seed: int = 0) -> np.ndarray:
        """k-means on standardised log-features."""
        x = np.log1p(np.abs(features))
        x = (x - x.mean(0)) / np.maximum(x.std(0), 1e-12)
        rng = np.random.default_rng(seed)
        c = x[rng.choice(len(x), min(k, len(x)), replace=False)]
        for _ in range(iters):
            lab = ((x[:, None] - c[None]) ** 2).sum(-1).argmin(1)
            new = np.stack([x[lab == j].mean(0) if (lab == j).any() else c[j] for j in range(len(c))])
            if np.allclose(new, c):
                break
            c = new
        return lab

    @staticmethod
    def fit_duration_model(flops: Sequence[float], bytes_: Sequence[float], durations_us: Sequence[float], ridge: float = 1e-9) -> dict:
        """Least squares ``t = a * flops + b * bytes + c``: ``1 / a`` and ``1 / b`` estimate achieved FLOP/s and byte/s,
        ``c`` the launch overhead."""
        x = np.stack([np.asarray(flops, float), np.asarray(bytes_, float), np.ones(len(flops))], 1)
        scale = np.maximum(np.abs(x).max(0), 1e-30)
        xs = x / scale
        coef = np.linalg.solve(xs.T @ xs + ridge * np.eye(3), xs.T @ (np.asarray(durations_us, float) * 1e-6)) / scale
        pred = x @ coef
        y = np.asarray(durations_us, float) * 1e-6
        return {"flops_per_s": 1 / coef[0] if coef[0] > 0 else math.inf, "bytes_per_s": 1 / coef[1] if coef[1] > 0 else math.inf, "overhead_s": float(coef[2]),
                "r2": float(1 - ((y - pred) ** 2).sum() / max(((y - y.mean()) ** 2).sum(), 1e-30)), "predict": lambda f, b: float(coef[0] * f + coef[1] * b + coef[2])}


# ================================================================================================ online statistics
class OnlineStats:
    """Welford mean / variance with min and max."""

    def __init__(self): self.n, self.mean, self.m2, self.min, self.max = 0, 0.0, 0.0, math.inf, -math.inf

    def update(self, x: float):
        self.n += 1
        d = x - self.mean
        self.mean += d / self.n
        self.m2 += d * (x - self.mean)
        self.min, self.max = min(self.min, x), max(self.max, x)

    @property
    def variance(self): return self.m2 / (self.n - 1) if self.n > 1 else 0.0
    @property
    def std(self): return math.sqrt(self.variance)


class EWMA:
    def __init__(self, alpha: float = 0.1): self.alpha, self.value, self.var = alpha, None, 0.0

    def update(self, x: float) -> float:
        if self.value is None:
            self.value = x
        else:
            d = x - self.value
            self.value += self.alpha * d
            self.var = (1 - self.alpha) * (self.var + self.alpha * d * d)
        return self.value


class OnlineAnomalyDetector:
    """Flags a value that is more than ``threshold`` running standard deviations from the running mean (after
    ``warmup`` values); anomalous values do not update the statistics, so a burst cannot hide itself."""

    def __init__(self, threshold: float = 4.0, warmup: int = 20):
        self.stats, self.threshold, self.warmup, self.events = OnlineStats(), threshold, warmup, []

    def update(self, x: float) -> bool:
        s = self.stats
        if s.n >= self.warmup and abs(x - s.mean) > self.threshold * max(s.std, 1e-12):
            self.events.append({"index": s.n + len(self.events), "value": x, "kind": "spike" if x > s.mean else "drop", "zscore": (x - s.mean) / max(s.std, 1e-12)})
            return True
        s.update(x)
        return False


class DriftDetector:
    """Compares the mean of the latest ``window`` values with the preceding ``window`` (Welch statistic)."""

    def __init__(self, window: int = 50, threshold: float = 4.0): self.window, self.threshold, self.buf = window, threshold, deque(maxlen=2 * window)

    def update(self, x: float) -> bool:
        self.buf.append(x)
        if len(self.buf) < 2 * self.window:
            return False
        a, b = np.array(list(self.buf)[:self.window]), np.array(list(self.buf)[self.window:])
        t = abs(a.mean() - b.mean()) / math.sqrt(a.var(ddof=1) / len(a) + b.var(ddof=1) / len(b) + 1e-30)
        if t > self.threshold:
            self.buf.clear()
            return True
        return False


class StreamingKMeans:
    """MacQueen updates: the nearest centroid moves by ``1 / count`` toward each point; the first ``k`` points seed it."""

    def __init__(self, k: int): self.k, self.centroids, self.counts = k, [], []

    def update(self, x) -> int:
        x = np.asarray(x, float)
        if len(self.centroids) < self.k:
            self.centroids.append(x.copy()); self.counts.append(1)
            return len(self.centroids) - 1
        j = int(np.argmin([((c - x) ** 2).sum() for c in self.centroids]))
        self.counts[j] += 1
        self.centroids[j] += (x - self.centroids[j]) / self.counts[j]
        return j


class OnlinePredictor:
    """Recursive least squares with forgetting for ``y ~ w . [x, 1]`` (predicts the next duration from features)."""

    def __init__(self, dim: int, forgetting: float = 0.99, delta: float = 1e3):
        self.w, self.p, self.lam, self.n, self.abs_err = np.zeros(dim + 1), np.eye(dim + 1) * delta, forgetting, 0, EWMA(0.05)

    def predict(self, x) -> float: return float(self.w @ np.append(np.asarray(x, float), 1.0))

    def update(self, x, y: float) -> float:
        z = np.append(np.asarray(x, float), 1.0)
        err = y - self.w @ z
        k = self.p @ z / (self.lam + z @ self.p @ z)
        self.w += k * err
        self.p = (self.p - np.outer(k, z @ self.p)) / self.lam
        self.n += 1
        self.abs_err.update(abs(err))
        return float(err)


# ================================================================================================ memory forecasting
class MemoryUsagePredictor:
    """Linear trend plus the largest recent residual over a window of ``(time, bytes)`` samples: forecasts usage at a
    horizon and the time left until a limit."""

    def __init__(self, window: int = 64): self.samples = deque(maxlen=window)
    def record(self, t: float, used: float): self.samples.append((t, used))

    def _fit(self):
        t, u = np.array([s[0] for s in self.samples]), np.array([s[1] for s in self.samples])
        slope, icpt = np.polyfit(t, u, 1) if len(t) > 1 and np.ptp(t) > 0 else (0.0, u[-1])
        return slope, icpt, float(np.max(u - (slope * t + icpt))) if len(t) > 1 else 0.0

    def predict(self, t: float) -> float:
        slope, icpt, resid = self._fit()
        return slope * t + icpt + resid

    def time_to_limit(self, limit: float) -> float | None:
        slope, icpt, resid = self._fit()
        if slope <= 0:
            return None
        return max(0.0, (limit - resid - icpt) / slope - self.samples[-1][0])

    def leak_suspected(self, min_slope: float = 1.0, min_r2: float = 0.9) -> bool:
        t, u = np.array([s[0] for s in self.samples]), np.array([s[1] for s in self.samples])
        if len(t) < 8:
            return False
        slope, icpt = np.polyfit(t, u, 1)
        r2 = 1 - ((u - (slope * t + icpt)) ** 2).sum() / max(((u - u.mean()) ** 2).sum(), 1e-30)
        return bool(slope > min_slope and r2 > min_r2)


class AdaptivePoolManager:
    """Size-class pools whose capacity follows demand: each class keeps as many free blocks as the recent peak of
    simultaneously live blocks of that class (times ``headroom``); ``trim`` releases the excess."""

    def __init__(self, headroom: float = 1.25, min_class: int = 256):
        self.headroom, self.min_class = headroom, min_class
        self.free: dict[int, int] = defaultdict(int)
        self.live: dict[int, int] = defaultdict(int)
        self.peak: dict[int, int] = defaultdict(int)
        self.hits = self.misses = 0

    def size_class(self, n: int) -> int: return max(self.min_class, 1 << (max(n, 1) - 1).bit_length())

    def allocate(self, n: int) -> int:
        c = self.size_class(n)
        if self.free[c]:
            self.free[c] -= 1
            self.hits += 1
        else:
            self.misses += 1
        self.live[c] += 1
        self.peak[c] = max(self.peak[c], self.live[c])
        return c

    def release(self, n: int):
        c = self.size_class(n)
        self.live[c] -= 1
        self.free[c] += 1

    def trim(self) -> int:
        freed = 0
        for c in list(self.free):
            keep = max(0, int(math.ceil(self.peak[c] * self.headroom)) - self.live[c])
            if self.free[c] > keep:
                freed += (self.free[c] - keep) * c
                self.free[c] = keep
            self.peak[c] = self.live[c]
        return freed

    def stats(self): return {"hit_rate": self.hits / max(self.hits + self.misses, 1), "cached_bytes": sum(c * n for c, n in self.free.items()), "live_bytes": sum(c * n for c, n in self.live.items())}


# ================================================================================================ low-overhead recorder
class StringInterner:
    def __init__(self): self.ids, self.names = {}, []
    def intern(self, s: str) -> int:
        i = self.ids.get(s)
        if i is None:
            i = self.ids[s] = len(self.names)
            self.names.append(s)
        return i
    def resolve(self, i: int) -> str: return self.names[i]


class OptimizedProfiler:
    """Records ``(name id, start, duration)`` triples into a fixed ring buffer, sampling one event in ``sample_every`` per
    name (counts stay exact), and measures its own cost per record."""

    def __init__(self, capacity: int = 65536, sample_every: int = 1, clock=time.perf_counter):
        self.buf = np.zeros((capacity, 3)); self.capacity, self.head, self.total = capacity, 0, 0
        self.sample_every, self.clock, self.names, self.counts, self.overhead = sample_every, clock, StringInterner(), Counter(), OnlineStats()

    def record(self, name: str, start: float, duration: float):
        t0 = self.clock()
        i = self.names.intern(name)
        self.counts[i] += 1
        if (self.counts[i] - 1) % self.sample_every == 0:
            self.buf[self.head % self.capacity] = (i, start, duration)
            self.head += 1
        self.total += 1
        self.overhead.update(self.clock() - t0)

    def events(self) -> list[dict]:
        n = min(self.head, self.capacity)
        rows = self.buf[:n] if self.head <= self.capacity else np.roll(self.buf, -(self.head % self.capacity), axis=0)
        return [{"name": self.names.resolve(int(r[0])), "start_us": r[1], "duration_us": r[2], "category": "op"} for r in rows]

    def estimated_totals(self) -> dict[str, float]:
        """Per-name total time: mean of the sampled durations times the exact count."""
        acc: dict[int, list] = defaultdict(list)
        for r in self.buf[:min(self.head, self.capacity)]:
            acc[int(r[0])].append(r[2])
        return {self.names.resolve(i): float(np.mean(v)) * self.counts[i] for i, v in acc.items()}

    def stats(self): return {"recorded": self.total, "stored": min(self.head, self.capacity), "dropped": max(0, self.head - self.capacity), "names": len(self.names.names),
                             "overhead_per_record_s": self.overhead.mean}


# ================================================================================================ regression detection
class RegressionDetector:
    """Baselines per metric (mean, std, n) with Welch's t statistic and a relative-change gate; severity by the size of the
    slowdown (``minor`` >= 5 %, ``major`` >= 20 %, ``critical`` >= 50 % by default)."""

    def __init__(self, min_relative: float = 0.05, t_threshold: float = 3.0, levels=((0.5, "critical"), (0.2, "major"), (0.05, "minor")), higher_is_better: bool = False):
        self.baselines, self.min_rel, self.t, self.levels, self.hib = {}, min_relative, t_threshold, levels, higher_is_better

    def set_baseline(self, metric: str, samples: Sequence[float]):
        self.baselines[metric] = {"mean": statistics.fmean(samples), "std": statistics.stdev(samples) if len(samples) > 1 else 0.0, "n": len(samples)}

    def save(self, path): open(path, "w").write(json.dumps(self.baselines))
    def load(self, path): self.baselines = json.loads(open(path).read())

    def check(self, metric: str, samples: Sequence[float]) -> dict:
        b = self.baselines[metric]
        m, s, n = statistics.fmean(samples), (statistics.stdev(samples) if len(samples) > 1 else 0.0), len(samples)
        rel = (m - b["mean"]) / abs(b["mean"]) if b["mean"] else 0.0
        worse = -rel if self.hib else rel
        t = abs(m - b["mean"]) / math.sqrt(b["std"] ** 2 / b["n"] + s ** 2 / n + 1e-30)
        significant = t > self.t and abs(rel) >= self.min_rel
        sev = next((name for thr, name in self.levels if worse >= thr), None) if significant and worse > 0 else None
        return {"metric": metric, "baseline": b["mean"], "current": m, "relative_change": rel, "t": t, "regression": sev is not None, "severity": sev,
                "improvement": bool(significant and worse < 0)}


# ================================================================================================ reports
class TemplateEngine:
    """``{{ name }}`` substitution (HTML-escaped unless ``{{{ name }}}``), ``{% for x in xs %} ... {% endfor %}`` loops over
    lists of dicts, dotted lookups."""

    import re as _re
    _FOR = _re.compile(r"{%\s*for (\w+) in ([\w.]+)\s*%}(.*?){%\s*endfor\s*%}", _re.S)
    _RAW, _VAR = _re.compile(r"{{{\s*([\w.]+)\s*}}}"), _re.compile(r"{{\s*([\w.]+)\s*}}")

    @staticmethod
    def _get(ctx, path):
        cur = ctx
        for p in path.split("."):
            cur = cur[p] if isinstance(cur, dict) else getattr(cur, p)
        return cur

    def render(self, template: str, ctx: dict) -> str:
        def loop(m):
            return "".join(self.render(m.group(3), {**ctx, m.group(1): item}) for item in self._get(ctx, m.group(2)))
        out = self._FOR.sub(loop, template)
        out = self._RAW.sub(lambda m: str(self._get(ctx, m.group(1))), out)
        return self._VAR.sub(lambda m: html.escape(str(self._get(ctx, m.group(1)))), out)


class ReportGenerator:
    HTML = ("<html><head><title>{{ title }}</title></head><body><h1>{{ title }}</h1><p>{{ summary.events }} events, {{ summary.total_ms }} ms total</p>"
            "<table><tr><th>operation</th><th>calls</th><th>total ms</th><th>share</th></tr>{% for r in rows %}<tr><td>{{ r.name }}</td><td>{{ r.calls }}</td>"
            "<td>{{ r.total_ms }}</td><td>{{ r.share }}</td></tr>{% endfor %}</table><ul>{% for f in findings %}<li>{{ f.text }}</li>{% endfor %}</ul></body></html>")
    MD = "# {{{ title }}}\n\n{{{ summary.events }}} events, {{{ summary.total_ms }}} ms total\n\n| operation | calls | total ms | share |\n|---|---|---|---|\n{% for r in rows %}| {{{ r.name }}} | {{{ r.calls }}} | {{{ r.total_ms }}} | {{{ r.share }}} |\n{% endfor %}\n{% for f in findings %}- {{{ f.text }}}\n{% endfor %}"

    def build(self, events: Iterable, title: str = "Profile report", top: int = 10, since_us: float | None = None, category: str | None = None) -> dict:
        ev = [e for e in map(_ev, events) if (since_us is None or e["start_us"] >= since_us) and (category is None or e.get("category") == category)]
        total = sum(e["duration_us"] for e in ev) or 1.0
        agg: dict[str, list] = defaultdict(list)
        for e in ev:
            agg[e["name"]].append(e["duration_us"])
        rows = sorted(({"name": n, "calls": len(d), "total_ms": round(sum(d) / 1e3, 3), "share": f"{sum(d) / total:.1%}", "_t": sum(d)} for n, d in agg.items()), key=lambda r: -r["_t"])[:top]
        findings = [{"text": f"{r['name']} takes {r['share']} of the time"} for r in rows if r["_t"] / total > 0.3]
        findings += [{"text": f"{n}: slowest call is {max(d) / statistics.median(d):.1f}x its median"} for n, d in agg.items() if len(d) >= 5 and max(d) > 5 * statistics.median(d)]
        return {"title": title, "summary": {"events": len(ev), "total_ms": round(total / 1e3, 3)}, "rows": rows, "findings": findings}

    def render(self, report: dict, fmt: str = "html") -> str:
        if fmt == "json":
            return json.dumps({k: ([{a: b for a, b in r.items() if a != "_t"} for r in v] if k == "rows" else v) for k, v in report.items()})
        return TemplateEngine().render(self.HTML if fmt == "html" else self.MD, report)


# ================================================================================================ streaming
class EventStreamer:
    """Outgoing event queue for a live viewer: bounded, drops the lowest priority first when full, batches events into
    compressed frames, and adapts the send rate to the measured throughput of ``send(frame: bytes) -> seconds``."""

    LEVELS = [{"name": "full", "keep": 1.0, "batch": 256}, {"name": "reduced", "keep": 0.5, "batch": 128}, {"name": "minimal", "keep": 0.1, "batch": 32}]

    def __init__(self, send: Callable[[bytes], float], capacity: int = 4096, compression: str = "zlib", target_latency: float = 0.05):
        self.send, self.capacity, self.compression, self.target = send, capacity, compression, target_latency
        self.heap: list = []
        self.seq, self.level, self.dropped, self.sent_events, self.bytes_raw, self.bytes_sent = 0, 0, 0, 0, 0, 0
        self.latency = EWMA(0.3)

    def push(self, event: dict, priority: int = 1):
        self.seq += 1
        lvl = self.LEVELS[self.level]
        if priority < 2 and lvl["keep"] < 1.0 and (self.seq * 2654435761 % 1000) / 1000 >= lvl["keep"]:
            self.dropped += 1
            return
        heapq.heappush(self.heap, (priority, self.seq, event))
        if len(self.heap) > self.capacity:
            heapq.heappop(self.heap)                                          # lowest priority, oldest
            self.dropped += 1

    def _encode(self, events) -> bytes:
        raw = json.dumps(events, separators=(",", ":")).encode()
        self.bytes_raw += len(raw)
        return {"zlib": lambda b: zlib.compress(b, 6), "gzip": lambda b: gzip.compress(b, 6), "none": lambda b: b}[self.compression](raw)

    def flush(self) -> int:
        frames = 0
        while self.heap:
            n = min(self.LEVELS[self.level]["batch"], len(self.heap))
            batch = [e for _, _, e in heapq.nlargest(n, self.heap)]
            keep = heapq.nsmallest(len(self.heap) - n, self.heap)
            self.heap = keep
            heapq.heapify(self.heap)
            frame = self._encode(batch)
            lat = self.latency.update(self.send(frame))
            self.bytes_sent += len(frame); self.sent_events += len(batch); frames += 1
            if lat > self.target and self.level < len(self.LEVELS) - 1:
                self.level += 1
            elif lat < 0.25 * self.target and self.level > 0:
                self.level -= 1
        return frames

    def stats(self): return {"sent": self.sent_events, "dropped": self.dropped, "quality": self.LEVELS[self.level]["name"], "compression_ratio": self.bytes_sent / max(self.bytes_raw, 1)}


# ================================================================================================ custom export / tools
class CustomExporter:
    """Column schema ``[{"header", "field", "format"}]`` with formats ``us`` / ``ms`` / ``s`` for durations, ``bytes`` /
    ``kib`` / ``mib`` for sizes, ``%.3f``-style number formats or ``str``; writes CSV, TSV or aligned text."""

    @staticmethod
    def _fmt(v, f):
        if v is None:
            return ""
        if f in ("us", "ms", "s"):
            return f"{v / {'us': 1, 'ms': 1e3, 's': 1e6}[f]:.3f}"
        if f in ("bytes", "kib", "mib"):
            return f"{v / {'bytes': 1, 'kib': 1024, 'mib': 1 << 20}[f]:.2f}" if f != "bytes" else str(int(v))
        if isinstance(f, str) and f.startswith("%"):
            return f % v
        return str(v)

    def export(self, events: Iterable, schema: Sequence[dict], kind: str = "csv") -> str:
        rows = [[self._fmt(_ev(e).get(c["field"]), c.get("format", "str")) for c in schema] for e in events]
        head = [c["header"] for c in schema]
        if kind in ("csv", "tsv"):
            sep = "," if kind == "csv" else "\t"
            q = lambda s: '"' + s.replace('"', '""') + '"' if (sep in s or '"' in s or "\n" in s) else s
            return "\n".join(sep.join(q(v) for v in r) for r in [head] + rows) + "\n"
        w = [max(len(r[i]) for r in [head] + rows) for i in range(len(head))]
        return "\n".join("  ".join(v.ljust(w[i]) for i, v in enumerate(r)).rstrip() for r in [head] + rows) + "\n"


class CustomToolRegistry:
    """Named analysis callbacks ``fn(events, **config) -> result`` with per-tool call counts and time."""

    def __init__(self): self.tools, self.stats = {}, {}
    def register(self, name, fn, **config): self.tools[name] = (fn, config); self.stats[name] = {"calls": 0, "seconds": 0.0, "errors": 0}
    def unregister(self, name): self.tools.pop(name, None)
    def list_tools(self): return sorted(self.tools)

    def run(self, name, events):
        fn, cfg = self.tools[name]
        t0 = time.perf_counter()
        try:
            return fn(events, **cfg)
        except Exception:
            self.stats[name]["errors"] += 1
            raise
        finally:
            self.stats[name]["calls"] += 1
            self.stats[name]["seconds"] += time.perf_counter() - t0

    def run_all(self, events): return {n: self.run(n, events) for n in self.list_tools()}


# ================================================================================================ flame graphs
def build_stacks(events: Iterable) -> dict[str, float]:
    """Folded stacks ``root;child;leaf -> self time`` from nested intervals per thread (an event whose interval lies inside
    another's is its child)."""
    out: dict[str, float] = defaultdict(float)
    by_thread: dict = defaultdict(list)
    for e in map(_ev, events):
        by_thread[e.get("thread_id", 0)].append(e)
    for evs in by_thread.values():
        evs.sort(key=lambda e: (e["start_us"], -e["duration_us"]))
        stack: list = []
        def close(upto):
            while stack and stack[-1][1] <= upto:
                name, end, self_t, path = stack.pop()
                out[path] += max(self_t, 0.0)
        for e in evs:
            close(e["start_us"])
            if stack:
                stack[-1][2] -= e["duration_us"]
            path = (stack[-1][3] + ";" if stack else "") + e["name"]
            stack.append([e["name"], e["start_us"] + e["duration_us"], e["duration_us"], path])
        close(math.inf)
    return dict(out)


def folded_text(stacks: dict[str, float]) -> str: return "".join(f"{k} {int(round(v))}\n" for k, v in sorted(stacks.items()))


def speedscope_json(stacks: dict[str, float], name: str = "profile") -> str:
    """The ``sampled`` profile form of the speedscope file format."""
    frames, index, samples, weights = [], {}, [], []
    for path, w in sorted(stacks.items()):
        ids = []
        for f in path.split(";"):
            if f not in index:
                index[f] = len(frames)
                frames.append({"name": f})
            ids.append(index[f])
        samples.append(ids); weights.append(w)
    return json.dumps({"$schema": "https://www.speedscope.app/file-format-schema.json", "shared": {"frames": frames},
                       "profiles": [{"type": "sampled", "name": name, "unit": "microseconds", "startValue": 0, "endValue": sum(weights), "samples": samples, "weights": weights}]})


# ================================================================================================ decorators
class AttributeRegistry:
    """``@registry.profile(category=...)`` wraps sync and async functions, ``@registry.profile_if(predicate)`` only when the
    predicate holds at call time; records go to ``sink(event dict)``."""

    def __init__(self, sink: Callable[[dict], None] | None = None, clock=time.perf_counter):
        self.events, self.clock = [], clock
        self.sink = sink or self.events.append

    def _emit(self, name, category, t0, extra): self.sink({"name": name, "category": category, "start_us": t0 * 1e6, "duration_us": (self.clock() - t0) * 1e6, **extra})

    def profile(self, name: str | None = None, category: str = "function", condition: Callable[..., bool] | None = None, **extra):
        def deco(fn):
            label = name or fn.__qualname__
            if asyncio.iscoroutinefunction(fn):
                @functools.wraps(fn)
                async def aw(*a, **kw):
                    if condition and not condition(*a, **kw):
                        return await fn(*a, **kw)
                    t0 = self.clock()
                    try:
                        return await fn(*a, **kw)
                    finally:
                        self._emit(label, category, t0, extra)
                return aw
            @functools.wraps(fn)
            def w(*a, **kw):
                if condition and not condition(*a, **kw):
                    return fn(*a, **kw)
                t0 = self.clock()
                try:
                    return fn(*a, **kw)
                finally:
                    self._emit(label, category, t0, extra)
            return w
        return deco

    def profile_if(self, condition, **kw): return self.profile(condition=condition, **kw)


# ================================================================================================ integrated profiler
class IntegratedProfiler:
    """Feeds every recorded duration to the online detectors and predictors, keeps trends, and assembles one report with
    workload characterisation, anomalies, drift points, regressions against baselines and recommendations."""

    def __init__(self, characterizer: WorkloadCharacterizer | None = None, regression: RegressionDetector | None = None):
        self.events: list[dict] = []
        self.detectors: dict[str, OnlineAnomalyDetector] = defaultdict(OnlineAnomalyDetector)
        self.drift: dict[str, DriftDetector] = defaultdict(lambda: DriftDetector(30, 5.0))
        self.trend: dict[str, EWMA] = defaultdict(lambda: EWMA(0.1))
        self.drift_points: list = []
        self.characterizer, self.regression, self.state = characterizer or WorkloadCharacterizer(), regression, "running"

    def record(self, event):
        e = _ev(event)
        if self.state != "running":
            return
        self.events.append(e)
        n, d = e["name"], e["duration_us"]
        self.detectors[n].update(d)
        self.trend[n].update(d)
        if self.drift[n].update(d):
            self.drift_points.append({"name": n, "at_event": len(self.events) - 1})

    def pause(self): self.state = "paused"
    def resume(self): self.state = "running"

    def report(self) -> dict:
        anomalies = {n: d.events for n, d in self.detectors.items() if d.events}
        regs = []
        if self.regression:
            by = defaultdict(list)
            for e in self.events:
                by[e["name"]].append(e["duration_us"])
            regs = [r for n, v in by.items() if n in self.regression.baselines and (r := self.regression.check(n, v))["regression"]]
        work = self.characterizer.analyze(self.events)
        recs = list(work.get("recommendations", []))
        recs += [f"{n}: {len(a)} outlier calls, check for contention or recompilation" for n, a in anomalies.items()]
        recs += [f"{r['metric']} is {r['relative_change']:.0%} slower than its baseline ({r['severity']})" for r in regs]
        return {"events": len(self.events), "workload": work, "anomalies": anomalies, "drift": self.drift_points, "regressions": regs,
                "trends": {n: t.value for n, t in self.trend.items()}, "recommendations": recs}
