"""Exporters and dashboards for profiler data: Grafana dashboard JSON, CloudWatch metric payloads, a streaming JSONL
sink, CSV / Markdown / JSON tables, a self-contained HTML report, a CI regression gate (JUnit XML + Markdown), Kubernetes
pod metadata, and a read-only power / temperature / clock monitor over NVML.

Nothing here talks to a network by itself: publishers build the payload their service expects and hand it to a ``sink``
callable (default: keep it in memory / write a file), so the same code runs in an air-gapped job and, with a sink that
posts the payload, against the real service. The reference has one module per target
(crates/torsh-profiler/src/{grafana,cloudwatch,streaming,custom_export,reporting,ci_cd,kubernetes,power,thermal}.rs).
"""
from __future__ import annotations

import csv
import html
import io
import json
import os
import threading
import time
from dataclasses import asdict, dataclass, field

from .profiler import ProfileEvent


# ---------------------------------------------------------------------------------------------------- Grafana
@dataclass
class GridPos:
    x: int = 0
    y: int = 0
    w: int = 12
    h: int = 8


class GrafanaDashboardGenerator:
    """Builds a Grafana dashboard document (schema version 36) whose panels query a Prometheus data source: the text
    this package's ``Profiler.prometheus_text`` / ``parallel.monitoring`` expose (grafana.rs:11-360)."""

    def __init__(self, title: str, datasource: str = "Prometheus"):
        self.doc = {"id": None, "uid": None, "title": title, "tags": [], "timezone": "browser", "schemaVersion": 36, "version": 1,
                    "refresh": "5s", "time": {"from": "now-15m", "to": "now"}, "panels": [], "templating": {"list": []}}
        self.datasource = datasource
        self._next_id = 1

    def with_uid(self, uid: str):
        self.doc["uid"] = uid
        return self

    def with_tags(self, tags):
        self.doc["tags"] = list(tags)
        return self

    def with_time_range(self, frm: str, to: str):
        self.doc["time"] = {"from": frm, "to": to}
        return self

    def with_refresh(self, refresh: str):
        self.doc["refresh"] = refresh
        return self

    def _panel(self, kind: str, title: str, queries, pos: GridPos, unit: str | None = None, **extra):
        targets = [{"expr": q, "refId": chr(ord("A") + i), "legendFormat": ""} for i, q in enumerate([queries] if isinstance(queries, str) else queries)]
        p = {"id": self._next_id, "type": kind, "title": title, "datasource": self.datasource, "targets": targets,
             "gridPos": asdict(pos), "fieldConfig": {"defaults": {"unit": unit or "short"}, "overrides": []}}
        p.update(extra)
        self._next_id += 1
        self.doc["panels"].append(p)
        return self

    def add_graph_panel(self, title, queries, pos: GridPos, unit=None):
        return self._panel("timeseries", title, queries, pos, unit)

    def add_heatmap_panel(self, title, query, pos: GridPos):
        return self._panel("heatmap", title, query, pos)

    def add_gauge_panel(self, title, query, pos: GridPos, lo=0.0, hi=100.0, thresholds=((None, "green"), (70.0, "yellow"), (90.0, "red")), unit=None):
        steps = [{"value": v, "color": c} for v, c in thresholds]
        self._panel("gauge", title, query, pos, unit)
        d = self.doc["panels"][-1]["fieldConfig"]["defaults"]
        d.update({"min": lo, "max": hi, "thresholds": {"mode": "absolute", "steps": steps}})
        return self

    def add_stat_panel(self, title, query, pos: GridPos, unit=None):
        return self._panel("stat", title, query, pos, unit)

    def add_variable(self, name: str, query: str, label: str | None = None, multi: bool = False):
        self.doc["templating"]["list"].append({"name": name, "label": label or name, "type": "query", "query": query,
                                               "datasource": self.datasource, "multi": multi, "includeAll": multi, "refresh": 1})
        return self

    def build(self) -> dict:
        return self.doc

    def export_json(self) -> str:
        return json.dumps(self.doc, indent=2)

    def export_to_file(self, path) -> None:
        with open(path, "w") as f:
            f.write(self.export_json())


class DashboardTemplates:
    """Ready-made dashboards over the metric names this package exports (prefix ``torsh``)."""

    @staticmethod
    def profiling(prefix: str = "torsh") -> GrafanaDashboardGenerator:
        g = GrafanaDashboardGenerator("torsh_b200 profiling").with_uid("torsh-profiling").with_tags(["torsh", "profiling"])
        g.add_variable("scope", f"label_values({prefix}_scope_duration_us_sum, scope)", multi=True)
        g.add_graph_panel("Scope time per second", f'rate({prefix}_scope_duration_us_sum{{scope=~"$scope"}}[1m])', GridPos(0, 0, 12, 8), "µs")
        g.add_graph_panel("Scope calls per second", f'rate({prefix}_scope_calls_total{{scope=~"$scope"}}[1m])', GridPos(12, 0, 12, 8), "ops")
        g.add_stat_panel("Tokens per second", f"{prefix}_tokens_per_second", GridPos(0, 8, 6, 4))
        g.add_stat_panel("Step time", f"{prefix}_step_ms", GridPos(6, 8, 6, 4), "ms")
        g.add_heatmap_panel("Kernel duration distribution", f"{prefix}_kernel_duration_us_bucket", GridPos(12, 8, 12, 8))
        return g

    @staticmethod
    def memory(prefix: str = "torsh") -> GrafanaDashboardGenerator:
        g = GrafanaDashboardGenerator("torsh_b200 memory").with_uid("torsh-memory").with_tags(["torsh", "memory"])
        g.add_graph_panel("Device memory", [f"{prefix}_memory_allocated_bytes", f"{prefix}_memory_reserved_bytes"], GridPos(0, 0, 16, 8), "bytes")
        g.add_gauge_panel("HBM in use", f"100 * {prefix}_memory_allocated_bytes / {prefix}_memory_total_bytes", GridPos(16, 0, 8, 8), unit="percent")
        g.add_stat_panel("Peak allocated", f"{prefix}_memory_peak_bytes", GridPos(0, 8, 8, 4), "bytes")
        g.add_stat_panel("Allocator cache hits", f"rate({prefix}_pool_hits_total[1m])", GridPos(8, 8, 8, 4), "ops")
        return g

    @staticmethod
    def performance(prefix: str = "torsh") -> GrafanaDashboardGenerator:
        g = GrafanaDashboardGenerator("torsh_b200 performance").with_uid("torsh-performance").with_tags(["torsh", "performance"])
        g.add_graph_panel("Throughput", f"{prefix}_tokens_per_second", GridPos(0, 0, 12, 8))
        g.add_graph_panel("Collective bus bandwidth", f"{prefix}_collective_bus_gbs", GridPos(12, 0, 12, 8), "GBs")
        g.add_gauge_panel("SM clock", f"{prefix}_sm_clock_mhz", GridPos(0, 8, 6, 6), lo=0, hi=1965,
                          thresholds=((None, "red"), (1300.0, "yellow"), (1700.0, "green")))
        g.add_gauge_panel("Power", f"{prefix}_power_watts", GridPos(6, 8, 6, 6), lo=0, hi=1000,
                          thresholds=((None, "green"), (900.0, "yellow"), (990.0, "red")), unit="watt")
        g.add_graph_panel("Straggler skew", f"max({prefix}_step_ms) - min({prefix}_step_ms)", GridPos(12, 8, 12, 6), "ms")
        return g


# ---------------------------------------------------------------------------------------------------- CloudWatch
CLOUDWATCH_UNITS = {"Seconds", "Microseconds", "Milliseconds", "Bytes", "Kilobytes", "Megabytes", "Gigabytes", "Percent", "Count",
                    "Bytes/Second", "Count/Second", "None"}


@dataclass
class MetricDatum:
    name: str
    value: float | None = None
    unit: str = "None"
    timestamp: float = 0.0
    dimensions: dict = field(default_factory=dict)
    statistics: dict | None = None          # {"SampleCount", "Sum", "Minimum", "Maximum"}

    def to_api(self) -> dict:
        d = {"MetricName": self.name, "Unit": self.unit,
             "Timestamp": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime(self.timestamp)),
             "Dimensions": [{"Name": k, "Value": str(v)} for k, v in sorted(self.dimensions.items())]}
        if self.statistics is not None:
            d["StatisticValues"] = dict(self.statistics)
        else:
            d["Value"] = float(self.value)
        return d


class CloudWatchPublisher:
    """Buffers metric data and emits ``PutMetricData`` request bodies (at most 1000 data per request, the service's
    limit) to ``sink(namespace, region, body_dict)``. With ``aggregate=True`` repeated names within one flush are folded
    into statistic sets (cloudwatch.rs:12-330)."""

    MAX_PER_REQUEST = 1000

    def __init__(self, namespace: str, region: str = "us-east-1", buffer_size: int = 20, aggregate: bool = False, sink=None):
        self.namespace, self.region, self.buffer_size, self.aggregate = namespace, region, buffer_size, aggregate
        self.default_dimensions: dict = {}
        self.buffer: list[MetricDatum] = []
        self.sent: list[dict] = []
        self.sink = sink if sink is not None else (lambda ns, region, body: self.sent.append(body))

    def add_dimension(self, name: str, value) -> "CloudWatchPublisher":
        self.default_dimensions[name] = value
        return self

    def put_metric(self, name: str, value: float, unit: str = "None", dimensions: dict | None = None):
        if unit not in CLOUDWATCH_UNITS:
            raise ValueError(f"unknown CloudWatch unit {unit!r}")
        self.buffer.append(MetricDatum(name, float(value), unit, time.time(), {**self.default_dimensions, **(dimensions or {})}))
        if len(self.buffer) >= self.buffer_size:
            self.flush()

    def put_metric_statistics(self, name: str, values, unit: str = "None", dimensions: dict | None = None):
        values = [float(v) for v in values]
        if not values:
            return
        stats = {"SampleCount": float(len(values)), "Sum": sum(values), "Minimum": min(values), "Maximum": max(values)}
        self.buffer.append(MetricDatum(name, None, unit, time.time(), {**self.default_dimensions, **(dimensions or {})}, stats))

    def publish_from_events(self, events: list[ProfileEvent]):
        """One duration statistic set per scope name, plus FLOP and byte totals where the scopes declared them."""
        by_name: dict[str, list[ProfileEvent]] = {}
        for e in events:
            by_name.setdefault(e.name, []).append(e)
        for name, evs in by_name.items():
            dims = {"Scope": name, "Category": evs[0].category}
            self.put_metric_statistics("ScopeDuration", [(e.device_us if e.device_us is not None else e.duration_us) for e in evs],
                                       "Microseconds", dims)
            flops, nbytes = sum(e.flops for e in evs), sum(e.bytes for e in evs)
            if flops:
                self.put_metric("ScopeFlops", flops, "Count", dims)
            if nbytes:
                self.put_metric("ScopeBytes", nbytes, "Bytes", dims)

    def _aggregated(self) -> list[MetricDatum]:
        if not self.aggregate:
            return self.buffer
        out: dict = {}
        for d in self.buffer:
            key = (d.name, d.unit, tuple(sorted(d.dimensions.items())))
            vals = out.setdefault(key, [])
            if d.statistics is not None:
                vals.append(d.statistics)
            else:
                vals.append({"SampleCount": 1.0, "Sum": d.value, "Minimum": d.value, "Maximum": d.value})
        res = []
        for (name, unit, dims), stats in out.items():
            agg = {"SampleCount": sum(s["SampleCount"] for s in stats), "Sum": sum(s["Sum"] for s in stats),
                   "Minimum": min(s["Minimum"] for s in stats), "Maximum": max(s["Maximum"] for s in stats)}
            res.append(MetricDatum(name, None, unit, time.time(), dict(dims), agg))
        return res

    def export_json(self) -> str:
        return json.dumps({"Namespace": self.namespace, "MetricData": [d.to_api() for d in self._aggregated()]}, indent=2)

    def flush(self) -> int:
        data = self._aggregated()
        n = 0
        for i in range(0, len(data), self.MAX_PER_REQUEST):
            chunk = data[i:i + self.MAX_PER_REQUEST]
            self.sink(self.namespace, self.region, {"Namespace": self.namespace, "MetricData": [d.to_api() for d in chunk]})
            n += len(chunk)
        self.buffer = []
        return n


# ---------------------------------------------------------------------------------------------------- streaming / tables
class StreamingExporter:
    """Appends one JSON object per event to a file (or any ``write``-able) as events arrive, with a bounded in-memory
    queue and back-pressure by dropping the oldest entries (streaming.rs)."""

    def __init__(self, target, max_queue: int = 4096, flush_every: int = 64):
        self._own = isinstance(target, (str, os.PathLike))
        self._f = open(target, "a") if self._own else target
        self.max_queue, self.flush_every = max_queue, flush_every
        self._q: list[str] = []
        self.dropped = 0
        self.written = 0
        self._lock = threading.Lock()

    def emit(self, event) -> None:
        rec = asdict(event) if hasattr(event, "__dataclass_fields__") else dict(event)
        with self._lock:
            if len(self._q) >= self.max_queue:
                self._q.pop(0)
                self.dropped += 1
            self._q.append(json.dumps(rec, default=str))
            if len(self._q) >= self.flush_every:
                self._flush_locked()

    def _flush_locked(self):
        if self._q:
            self._f.write("\n".join(self._q) + "\n")
            self._f.flush()
            self.written += len(self._q)
            self._q = []

    def flush(self):
        with self._lock:
            self._flush_locked()

    def close(self):
        self.flush()
        if self._own:
            self._f.close()


def summarize_events(events: list[ProfileEvent]) -> list[dict]:
    """Per-scope rows sorted by total time: calls, total / mean / max µs, share of the whole, FLOP/s and bytes/s."""
    rows: dict[str, dict] = {}
    for e in events:
        d = e.device_us if e.device_us is not None else e.duration_us
        r = rows.setdefault(e.name, {"name": e.name, "category": e.category, "calls": 0, "total_us": 0.0, "max_us": 0.0, "flops": 0.0, "bytes": 0.0})
        r["calls"] += 1
        r["total_us"] += d
        r["max_us"] = max(r["max_us"], d)
        r["flops"] += e.flops
        r["bytes"] += e.bytes
    total = sum(r["total_us"] for r in rows.values()) or 1.0
    out = sorted(rows.values(), key=lambda r: -r["total_us"])
    for r in out:
        r["mean_us"] = r["total_us"] / r["calls"]
        r["share"] = r["total_us"] / total
        r["tflops"] = r["flops"] / r["total_us"] / 1e6 if r["total_us"] else 0.0
        r["gbs"] = r["bytes"] / r["total_us"] / 1e3 if r["total_us"] else 0.0
    return out


def export_table(events: list[ProfileEvent], fmt: str = "markdown") -> str:
    """``fmt``: "csv", "markdown" or "json" (custom_export.rs)."""
    rows = summarize_events(events)
    cols = ["name", "category", "calls", "total_us", "mean_us", "max_us", "share", "tflops", "gbs"]
    if fmt == "json":
        return json.dumps(rows, indent=2)
    if fmt == "csv":
        buf = io.StringIO()
        w = csv.DictWriter(buf, fieldnames=cols, extrasaction="ignore")
        w.writeheader()
        w.writerows(rows)
        return buf.getvalue()
    if fmt == "markdown":
        def cell(r, c):
            v = r[c]
            return f"{v:.1%}" if c == "share" else (f"{v:.1f}" if isinstance(v, float) else str(v))
        lines = ["| " + " | ".join(cols) + " |", "|" + "---|" * len(cols)]
        lines += ["| " + " | ".join(cell(r, c) for c in cols) + " |" for r in rows]
        return "\n".join(lines)
    raise ValueError(f"unknown format {fmt!r}")


def html_report(events: list[ProfileEvent], title: str = "torsh_b200 profile", extra: dict | None = None) -> str:
    """A self-contained HTML page (no scripts or remote assets): summary table with inline share bars (reporting.rs,
    dashboard/)."""
    rows = summarize_events(events)
    head = "".join(f"<th>{c}</th>" for c in ("scope", "category", "calls", "total ms", "mean µs", "max µs", "share", "TFLOP/s", "GB/s"))
    body = []
    for r in rows:
        bar = f'<div style="background:#4a90d9;height:10px;width:{r["share"] * 100:.1f}%"></div>'
        body.append("<tr>" + "".join(f"<td>{c}</td>" for c in (
            html.escape(r["name"]), html.escape(r["category"]), r["calls"], f'{r["total_us"] / 1e3:.3f}', f'{r["mean_us"]:.1f}',
            f'{r["max_us"]:.1f}', f'{r["share"]:.1%}{bar}', f'{r["tflops"]:.1f}', f'{r["gbs"]:.0f}')) + "</tr>")
    meta = "".join(f"<li><b>{html.escape(str(k))}</b>: {html.escape(str(v))}</li>" for k, v in (extra or {}).items())
    return (f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(title)}</title>"
            "<style>body{font-family:sans-serif}table{border-collapse:collapse}td,th{border:1px solid #ccc;padding:4px 8px;text-align:right}"
            "td:first-child{text-align:left}</style></head><body>"
            f"<h1>{html.escape(title)}</h1><ul>{meta}</ul><table><tr>{head}</tr>{''.join(body)}</table></body></html>")


# ---------------------------------------------------------------------------------------------------- CI gate
def ci_regression_report(current: dict[str, float], baseline: dict[str, float], tolerance: float = 0.05, lower_is_better: bool = True):
    """Compares named measurements with a stored baseline. Returns ``(ok, junit_xml, markdown)``: one test case per
    metric, failing when it regressed by more than ``tolerance`` (ci_cd.rs)."""
    cases, md, ok = [], ["| metric | baseline | current | change | status |", "|---|---|---|---|---|"], True
    for name in sorted(current):
        cur, base = current[name], baseline.get(name)
        if base is None or base == 0:
            status, change = "new", 0.0
        else:
            change = (cur - base) / abs(base)
            worse = change > tolerance if lower_is_better else change < -tolerance
            status = "regressed" if worse else "ok"
            ok &= not worse
        md.append(f"| {name} | {'' if base is None else f'{base:.4g}'} | {cur:.4g} | {change:+.1%} | {status} |")
        inner = f'<failure message="{html.escape(name)} changed by {change:+.1%} (tolerance {tolerance:.0%})"/>' if status == "regressed" else ""
        cases.append(f'<testcase classname="perf" name="{html.escape(name)}" time="0">{inner}</testcase>')
    fails = sum("<failure" in c for c in cases)
    xml = f'<?xml version="1.0"?><testsuite name="torsh_b200.perf" tests="{len(cases)}" failures="{fails}">{"".join(cases)}</testsuite>'
    return ok, xml, "\n".join(md)


# ---------------------------------------------------------------------------------------------------- Kubernetes
def kubernetes_metadata(env: dict | None = None) -> dict:
    """Labels that identify the pod a job runs in, from the downward-API / standard variables (kubernetes.rs)."""
    e = os.environ if env is None else env
    keys = {"pod": ("POD_NAME", "HOSTNAME"), "namespace": ("POD_NAMESPACE",), "node": ("NODE_NAME",), "job": ("JOB_NAME",),
            "container": ("CONTAINER_NAME",), "service_host": ("KUBERNETES_SERVICE_HOST",)}
    out = {}
    for label, names in keys.items():
        for n in names:
            if e.get(n):
                out[label] = e[n]
                break
    out["in_cluster"] = "service_host" in out
    return out


# ---------------------------------------------------------------------------------------------------- power / thermal
class PowerThermalMonitor:
    """Samples power draw, temperature, SM clock and the active throttle reasons of one GPU on a background thread.
    READ-ONLY: it never sets clocks, power limits or any other device state. ``nvml`` is the ``pynvml`` module or an
    object with the same functions (tests pass a fake); without NVML the monitor records nothing (power.rs, thermal.rs)."""

    def __init__(self, device_index: int = 0, interval_s: float = 0.2, nvml=None):
        self.index, self.interval_s = device_index, interval_s
        self.samples: list[dict] = []
        self._stop = threading.Event()
        self._thread = None
        if nvml is None:
            try:
                import pynvml as nvml          # provided by nvidia-ml-py
            except Exception:
                nvml = None
        self.nvml = nvml

    def sample_once(self) -> dict | None:
        n = self.nvml
        if n is None:
            return None
        try:
            h = n.nvmlDeviceGetHandleByIndex(self.index)
            s = {"t": time.time(), "power_w": n.nvmlDeviceGetPowerUsage(h) / 1000.0,
                 "temp_c": float(n.nvmlDeviceGetTemperature(h, getattr(n, "NVML_TEMPERATURE_GPU", 0))),
                 "sm_mhz": float(n.nvmlDeviceGetClockInfo(h, getattr(n, "NVML_CLOCK_SM", 1))),
                 "throttle_reasons": int(n.nvmlDeviceGetCurrentClocksThrottleReasons(h))}
        except Exception:
            return None
        self.samples.append(s)
        return s

    def start(self):
        if self.nvml is None or self._thread is not None:
            return self
        try:
            self.nvml.nvmlInit()
        except Exception:
            self.nvml = None
            return self
        self._stop.clear()

        def loop():
            while not self._stop.is_set():
                self.sample_once()
                self._stop.wait(self.interval_s)
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2.0)
            self._thread = None
        return self.summary()

    def summary(self) -> dict:
        if not self.samples:
            return {"samples": 0}
        p = [s["power_w"] for s in self.samples]
        t = [s["temp_c"] for s in self.samples]
        c = sorted(s["sm_mhz"] for s in self.samples)
        dt = self.samples[-1]["t"] - self.samples[0]["t"]
        reasons = 0
        for s in self.samples:
            reasons |= s["throttle_reasons"]
        return {"samples": len(self.samples), "power_w_mean": sum(p) / len(p), "power_w_max": max(p), "temp_c_max": max(t),
                "sm_mhz_median": c[len(c) // 2], "energy_j": sum(p) / len(p) * dt, "throttle_reason_bits": reasons}
