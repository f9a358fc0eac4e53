"""Metrics and monitoring of a distributed job (``crates/torsh-distributed/src/metrics.rs:33-760``,
``distributed_monitoring.rs:18-960``): a time-series collector for system / communication / training metrics with JSON
and Prometheus-text export, and a monitor that checks alert thresholds (step-time regression, communication share,
memory, stragglers across ranks) and aggregates per-rank summaries on rank 0 through a store."""
from __future__ import annotations

import json
import statistics
import time
from collections import defaultdict, deque
from dataclasses import dataclass, field


class MetricsCollector:
    def __init__(self, history: int = 1000):
        self.series: dict[str, deque] = defaultdict(lambda: deque(maxlen=history))
        self.counters: dict[str, float] = defaultdict(float)

    def record(self, name: str, value: float, t: float | None = None) -> None:
        self.series[name].append((time.time() if t is None else t, float(value)))

    def incr(self, name: str, by: float = 1.0) -> None:
        self.counters[name] += by

    def record_step(self, step_ms: float, tokens: int = 0, comm_ms: float = 0.0, loss: float | None = None) -> None:
        self.record("training/step_ms", step_ms)
        if tokens:
            self.record("training/tokens_per_s", tokens / (step_ms / 1e3))
        self.record("communication/share", comm_ms / step_ms if step_ms else 0.0)
        if loss is not None:
            self.record("training/loss", loss)
        self.incr("training/steps")

    def record_system(self) -> None:
        try:
            import psutil
            self.record("system/cpu_percent", psutil.cpu_percent(None))
            self.record("system/host_mem_gb", psutil.virtual_memory().used / 2**30)
        except ImportError:
            pass
        try:
            import torch
            if torch.cuda.is_available():
                self.record("system/gpu_mem_gb", torch.cuda.memory_allocated() / 2**30)
                self.record("system/gpu_mem_reserved_gb", torch.cuda.memory_reserved() / 2**30)
        except ImportError:
            pass

    def summary(self, name: str) -> dict:
        v = [x for _, x in self.series.get(name, ())]
        if not v:
            return {"count": 0}
        s = sorted(v)
        return {"count": len(v), "mean": statistics.fmean(v), "min": s[0], "max": s[-1], "last": v[-1],
                "p50": s[len(s) // 2], "p95": s[min(len(s) - 1, int(0.95 * len(s)))]}

    def export_json(self) -> str:
        return json.dumps({"series": {k: list(v) for k, v in self.series.items()}, "counters": dict(self.counters)})

    def export_prometheus(self, prefix: str = "torsh") -> str:
        clean = lambda n: f"{prefix}_{n}".replace("/", "_").replace("-", "_").replace(".", "_")
        lines = []
        for k, v in sorted(self.series.items()):
            if v:
                lines += [f"# TYPE {clean(k)} gauge", f"{clean(k)} {v[-1][1]}"]
        for k, c in sorted(self.counters.items()):
            lines += [f"# TYPE {clean(k)}_total counter", f"{clean(k)}_total {c}"]
        return "\n".join(lines) + "\n"


@dataclass
class AlertThresholds:
    step_time_regression: float = 1.5      # last step vs median of the window
    max_comm_share: float = 0.5
    max_gpu_mem_gb: float | None = None
    straggler_ratio: float = 1.3           # slowest rank vs median rank


@dataclass
class Alert:
    kind: str
    message: str
    value: float
    t: float = field(default_factory=time.time)


class DistributedMonitor:
    def __init__(self, collector: MetricsCollector | None = None, thresholds: AlertThresholds | None = None, rank: int = 0,
                 world_size: int = 1, store=None):
        self.c, self.th = collector or MetricsCollector(), thresholds or AlertThresholds()
        self.rank, self.world, self.store = rank, world_size, store
        self.alerts: list[Alert] = []

    def check(self) -> list[Alert]:
        new = []
        steps = [v for _, v in self.c.series.get("training/step_ms", ())]
        if len(steps) >= 5:
            med = statistics.median(steps[:-1])
            if steps[-1] > self.th.step_time_regression * med:
                new.append(Alert("step_time", f"step took {steps[-1]:.1f} ms vs median {med:.1f} ms", steps[-1] / med))
        share = self.c.series.get("communication/share")
        if share and share[-1][1] > self.th.max_comm_share:
            new.append(Alert("comm_share", f"communication is {share[-1][1]:.0%} of the step", share[-1][1]))
        mem = self.c.series.get("system/gpu_mem_gb")
        if self.th.max_gpu_mem_gb and mem and mem[-1][1] > self.th.max_gpu_mem_gb:
            new.append(Alert("memory", f"{mem[-1][1]:.1f} GB allocated", mem[-1][1]))
        self.alerts += new
        return new

    def publish(self) -> None:
        """Write this rank's summary to the store (``monitor/<rank>``)."""
        if self.store is not None:
            self.store.set(f"monitor/{self.rank}", json.dumps(self.c.summary("training/step_ms")).encode())

    def aggregate(self) -> dict:
        """Rank 0: read every rank's summary, flag stragglers."""
        per_rank = {}
        for r in range(self.world):
            raw = self.store.get(f"monitor/{r}") if self.store is not None else None
            if raw:
                per_rank[r] = json.loads(raw)
        means = {r: s["mean"] for r, s in per_rank.items() if s.get("count")}
        out = {"ranks": per_rank, "stragglers": []}
        if len(means) >= 2:
            med = statistics.median(means.values())
            out["stragglers"] = [r for r, m in means.items() if m > self.th.straggler_ratio * med]
            for r in out["stragglers"]:
                self.alerts.append(Alert("straggler", f"rank {r} averages {means[r]:.1f} ms vs median {med:.1f} ms", means[r] / med))
        return out
