"""Metrics and monitoring of a distributed job (``crates/torsh-distributed/src/metrics.rs:33-760``,
``distributed_monitoring.rs:18-960``): a time-series collector for system / communication / training metrics with JSON
and Prometheus-text export, and a monitor that checks alert thresholds (step-time regression, communication share,
memory, stragglers across ranks) and aggregates per-rank summaries on rank 0 through a store."""
from __future__ import annotations

import enum
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


# ---------------------------------------------------------------------------------------------------------------------
# Bottleneck detection (``crates/torsh-distributed/src/bottleneck_detection.rs:16-717``: types, severity, remediation)
class BottleneckType(enum.Enum):
    COMMUNICATION = "communication"
    COMPUTE = "compute"
    MEMORY = "memory"
    DATA_LOADING = "data_loading"
    LOAD_IMBALANCE = "load_imbalance"
    HOST_LAUNCH = "host_launch"
    POWER_CAP = "power_cap"


class Severity(enum.IntEnum):
    LOW = 1
    MEDIUM = 2
    HIGH = 3
    CRITICAL = 4


@dataclass
class Bottleneck:
    kind: BottleneckType
    severity: Severity
    evidence: str
    remediation: list[str]
    ranks: list[int] = field(default_factory=list)


@dataclass
class StepSample:
    """What one rank measured for one step (milliseconds unless stated)."""
    rank: int
    step_ms: float
    compute_ms: float = 0.0
    exposed_comm_ms: float = 0.0            # communication time that was NOT hidden behind compute
    data_wait_ms: float = 0.0               # time the step waited for its batch
    device_idle_ms: float = 0.0             # gaps between kernels (host could not launch fast enough)
    mem_used_frac: float = 0.0
    sm_mhz: float | None = None
    sm_max_mhz: float | None = None


class BottleneckDetector:
    """Turns a window of per-rank step samples into a ranked list of bottlenecks with remediation hints."""

    def __init__(self, window: int = 50, comm_frac: float = 0.15, data_frac: float = 0.05, idle_frac: float = 0.05,
                 mem_frac: float = 0.92, imbalance: float = 0.10, clock_frac: float = 0.90):
        self.window, self.samples = window, []
        self.t = dict(comm=comm_frac, data=data_frac, idle=idle_frac, mem=mem_frac, imb=imbalance, clk=clock_frac)

    def record(self, s: StepSample):
        self.samples.append(s)
        del self.samples[:-self.window * 64]

    @staticmethod
    def _sev(x: float, lo: float) -> Severity:
        r = x / lo
        return Severity.CRITICAL if r >= 4 else Severity.HIGH if r >= 2.5 else Severity.MEDIUM if r >= 1.5 else Severity.LOW

    def analyze(self) -> list[Bottleneck]:
        if not self.samples:
            return []
        by_rank: dict[int, list[StepSample]] = {}
        for s in self.samples:
            by_rank.setdefault(s.rank, []).append(s)
        mean = lambda xs: sum(xs) / max(len(xs), 1)
        step = {r: mean([s.step_ms for s in v[-self.window:]]) for r, v in by_rank.items()}
        tot = mean(list(step.values())) or 1e-9
        frac = lambda attr: mean([mean([getattr(s, attr) for s in v[-self.window:]]) for v in by_rank.values()]) / tot
        out: list[Bottleneck] = []
        c = frac("exposed_comm_ms")
        if c > self.t["comm"]:
            out.append(Bottleneck(BottleneckType.COMMUNICATION, self._sev(c, self.t["comm"]),
                                  f"{c:.0%} of the step is exposed communication",
                                  ["use the fused compute + collective kernels (all-gather→GEMM, GEMM→reduce-scatter)",
                                   "raise the gradient bucket size so fewer launches pay the barrier latency",
                                   "check that NVLS is enabled beyond two ranks"]))
        d = frac("data_wait_ms")
        if d > self.t["data"]:
            out.append(Bottleneck(BottleneckType.DATA_LOADING, self._sev(d, self.t["data"]),
                                  f"{d:.0%} of the step waits for input batches",
                                  ["prefetch batches on a copy stream from pinned memory", "add loader workers"]))
        i = frac("device_idle_ms")
        if i > self.t["idle"]:
            out.append(Bottleneck(BottleneckType.HOST_LAUNCH, self._sev(i, self.t["idle"]),
                                  f"the device idles {i:.0%} of the step between kernels",
                                  ["capture the step in a CUDA graph", "use step_async so the host runs one step ahead"]))
        m = max(mean([s.mem_used_frac for s in v[-self.window:]]) for v in by_rank.values())
        if m > self.t["mem"]:
            out.append(Bottleneck(BottleneckType.MEMORY, self._sev(m, self.t["mem"]) if m < 0.99 else Severity.CRITICAL,
                                  f"device memory is {m:.0%} full",
                                  ["shard optimizer state and parameters (FSDP)", "checkpoint activations", "lower the micro-batch"]))
        if len(step) > 1:
            slow = max(step, key=step.get)
            spread = (step[slow] - min(step.values())) / tot
            if spread > self.t["imb"]:
                out.append(Bottleneck(BottleneckType.LOAD_IMBALANCE, self._sev(spread, self.t["imb"]),
                                      f"rank {slow} is {spread:.0%} of a step slower than the fastest rank",
                                      ["rebalance pipeline stages or expert capacity", "check that rank's clocks and neighbours"],
                                      ranks=[slow]))
        clk = [(s.sm_mhz / s.sm_max_mhz, s.rank) for s in self.samples[-self.window:] if s.sm_mhz and s.sm_max_mhz]
        if clk and mean([c for c, _ in clk]) < self.t["clk"]:
            out.append(Bottleneck(BottleneckType.POWER_CAP, Severity.LOW,
                                  f"SM clocks average {mean([c for c, _ in clk]):.0%} of maximum",
                                  ["expected under the board power cap during dense GEMMs; compare time x MHz, not time"],
                                  ranks=sorted({r for _, r in clk})))
        if not out and frac("compute_ms") > 0.8:
            out.append(Bottleneck(BottleneckType.COMPUTE, Severity.LOW, "the step is compute-bound",
                                  ["profile the top kernels against the tensor-core and HBM rooflines"]))
        return sorted(out, key=lambda b: -int(b.severity))
