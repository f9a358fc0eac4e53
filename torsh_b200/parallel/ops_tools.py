"""Operations tooling for distributed training (``crates/torsh-distributed/src``): energy and carbon accounting with
carbon-aware scheduling (``green_computing.rs``), compression chosen from measured link speed
(``network_aware_compression.rs``), per-rank memory balancing and pressure handling
(``distributed_memory_optimization.rs``), collective-sequence and divergence debugging (``debugging.rs``), NCCL algorithm /
protocol / bucket selection from a latency-bandwidth model (``nccl_optimization.rs``), bus-bandwidth arithmetic and
model fitting for benchmark sweeps (``enhanced_benchmarks.rs``), analytics over per-rank step records with an HTML
dashboard and text timelines (``advanced_monitoring.rs``, ``training_analytics_dashboard.rs``, ``visualization.rs``).

Nothing here changes a GPU's settings: power caps and clocks appear only as numbers in reports."""
from __future__ import annotations

import hashlib
import html
import math
import statistics
import time
from collections import Counter, defaultdict
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch

from .compression import Compressor, Int8BlockQuantization, PackedSignSGD, TopK


# ================================================================================================ green computing
CARBON_INTENSITY = {"eu-north": 30.0, "ca-quebec": 35.0, "eu-west": 250.0, "us-west": 210.0, "us-east": 380.0, "asia-east": 540.0, "default": 450.0}   # gCO2e per kWh, yearly averages


class EnergyTracker:
    """Integrates sampled power (watts per device; the sampler is injected — NVML's ``nvmlDeviceGetPowerUsage`` on a
    machine that has it) into energy, and reports carbon for a region and work per joule."""

    def __init__(self, sampler: Callable[[], Sequence[float]], region: str = "default", pue: float = 1.2, clock=time.monotonic):
        self.sampler, self.region, self.pue, self.clock = sampler, region, pue, clock
        self.joules, self.samples, self._last, self.work = 0.0, [], None, 0.0

    def sample(self):
        now, watts = self.clock(), sum(self.sampler())
        if self._last is not None:
            self.joules += 0.5 * (watts + self._last[1]) * (now - self._last[0])          # trapezoid
        self._last = (now, watts); self.samples.append((now, watts))
        return watts

    def add_work(self, units: float): self.work += units
    def kwh(self) -> float: return self.joules * self.pue / 3.6e6
    def carbon_grams(self) -> float: return self.kwh() * CARBON_INTENSITY.get(self.region, CARBON_INTENSITY["default"])

    def report(self) -> dict:
        w = [s[1] for s in self.samples]
        return {"device_joules": self.joules, "facility_kwh": self.kwh(), "carbon_g": self.carbon_grams(), "mean_watts": statistics.fmean(w) if w else 0.0, "peak_watts": max(w, default=0.0),
                "work_per_joule": self.work / self.joules if self.joules else 0.0, "region": self.region, "equivalent_km_driven": self.carbon_grams() / 120.0}


def carbon_aware_schedule(forecast: Sequence[float], duration: int, deadline: int | None = None, splittable: bool = False) -> dict:
    """Start slot (or, for a job that can pause, the set of slots) minimising the summed forecast carbon intensity over
    ``duration`` slots, finishing by ``deadline``."""
    horizon = min(len(forecast), deadline if deadline is not None else len(forecast))
    if duration > horizon:
        raise ValueError("the job does not fit before the deadline")
    now = sum(forecast[:duration])
    if splittable:
        slots = sorted(sorted(range(horizon), key=lambda i: forecast[i])[:duration])
        cost = sum(forecast[i] for i in slots)
        return {"slots": slots, "intensity_sum": cost, "saving": 1 - cost / now}
    start = min(range(horizon - duration + 1), key=lambda s: sum(forecast[s:s + duration]))
    cost = sum(forecast[start:start + duration])
    return {"start": start, "slots": list(range(start, start + duration)), "intensity_sum": cost, "saving": 1 - cost / now}


def efficiency_advice(throughput_at_power: dict[float, float]) -> dict:
    """Given measured throughput at several power levels (from runs an operator made), the level with the most work per
    joule and what it costs in speed against the fastest level.  Advice only: nothing is applied."""
    eff = {p: t / p for p, t in throughput_at_power.items()}
    best, fastest = max(eff, key=eff.get), max(throughput_at_power, key=throughput_at_power.get)
    return {"most_efficient_watts": best, "work_per_joule": eff[best], "slowdown_vs_fastest": 1 - throughput_at_power[best] / throughput_at_power[fastest], "energy_saving_vs_fastest": 1 - eff[fastest] / eff[best]}


# ================================================================================================ network-aware compression
@dataclass
class LinkEstimate:
    bandwidth: float = 50e9           # bytes / s
    latency: float = 5e-6             # s
    alpha: float = 0.3                # smoothing of new observations

    def observe(self, nbytes: int, seconds: float):
        if nbytes > 1 << 16:
            bw = nbytes / max(seconds - self.latency, 1e-9)
            self.bandwidth = (1 - self.alpha) * self.bandwidth + self.alpha * bw
        else:
            self.latency = (1 - self.alpha) * self.latency + self.alpha * seconds
    def transfer_time(self, nbytes: float) -> float: return self.latency + nbytes / self.bandwidth


class NetworkAwareCompressor:
    """Chooses per tensor among no compression, int8 blocks, top-k and packed signs: the candidate with the lowest estimated
    ``compress + transfer + decompress`` time wins, subject to an error budget (relative L2 error of the round trip).  The link
    estimate follows observed transfers, so the choice moves as the network does."""

    def __init__(self, link: LinkEstimate | None = None, max_error: float = 0.5, compress_throughput: float = 20e9):
        self.link, self.max_error, self.ctp = link or LinkEstimate(), max_error, compress_throughput
        self.candidates: dict[str, Compressor | None] = {"none": None, "int8": Int8BlockQuantization(), "topk_1%": TopK(0.01), "topk_10%": TopK(0.1), "sign": PackedSignSGD()}
        self.choices = Counter()

    def _payload_bytes(self, name: str, n: int, es: int) -> float:
        return {"none": n * es, "int8": n + 4 * math.ceil(n / 1024), "topk_1%": 0.01 * n * (4 + es), "topk_10%": 0.1 * n * (4 + es), "sign": n / 8 + 4}[name]

    def estimate(self, g: torch.Tensor) -> dict:
        n, es = g.numel(), g.element_size()
        return {name: self.link.transfer_time(self._payload_bytes(name, n, es)) + (0.0 if c is None else 2 * n * es / self.ctp) for name, c in self.candidates.items()}

    def error(self, name: str, g: torch.Tensor) -> float:
        c = self.candidates[name]
        if c is None:
            return 0.0
        r = c.decompress(c.compress(g), g.shape, g.dtype, g.device)
        return float((r.float() - g.float()).norm() / g.float().norm().clamp_min(1e-30))

    def choose(self, g: torch.Tensor) -> str:
        for name, _ in sorted(self.estimate(g).items(), key=lambda kv: kv[1]):
            if self.error(name, g) <= self.max_error:
                self.choices[name] += 1
                return name
        return "none"

    def compress(self, g: torch.Tensor):
        name = self.choose(g)
        c = self.candidates[name]
        return name, (g if c is None else c.compress(g))

    def decompress(self, name: str, payload, shape, dtype=torch.float32, device=None):
        c = self.candidates[name]
        return payload if c is None else c.decompress(payload, shape, dtype, device)


# ================================================================================================ memory across ranks
def balance_shards(sizes: Sequence[int], capacities: Sequence[float]) -> dict:
    """Assigns shards to ranks so that the fullest rank (as a fraction of its capacity) is as empty as possible: largest
    shard first, to the rank whose fill fraction would be smallest."""
    load, assign = [0.0] * len(capacities), {}
    for i in sorted(range(len(sizes)), key=lambda i: -sizes[i]):
        r = min(range(len(capacities)), key=lambda r: (load[r] + sizes[i]) / capacities[r])
        load[r] += sizes[i]; assign[i] = r
    fill = [l / c for l, c in zip(load, capacities)]
    return {"assignment": assign, "load": load, "fill": fill, "imbalance": max(fill) / (sum(fill) / len(fill)) if sum(fill) else 1.0}


class DistributedMemoryOptimizer:
    """Looks at each rank's memory (used, capacity, split into parameters / gradients / optimizer state / activations) and
    proposes the cheapest action that brings every rank under ``target`` utilisation."""
    ACTIONS = (("activation_checkpointing", "activations", 0.7, 0.33), ("shard_optimizer_state", "optimizer", None, 0.0), ("shard_gradients", "gradients", None, 0.0), ("offload_optimizer_state", "optimizer", 1.0, 0.15),
               ("shard_parameters", "parameters", None, 0.10), ("offload_parameters", "parameters", 1.0, 0.40))   # (name, component, fraction saved (None: (w-1)/w), step-time cost)

    def __init__(self, world_size: int, target: float = 0.9): self.world, self.target = world_size, target

    def pressure(self, ranks: Sequence[dict]) -> list[dict]:
        return [{"rank": i, "utilisation": sum(r["components"].values()) / r["capacity"], "level": "critical" if sum(r["components"].values()) / r["capacity"] > 0.97 else "high" if sum(r["components"].values()) / r["capacity"] > self.target else "ok"} for i, r in enumerate(ranks)]

    def plan(self, ranks: Sequence[dict]) -> dict:
        comps = [dict(r["components"]) for r in ranks]
        util = lambda: max(sum(c.values()) / r["capacity"] for c, r in zip(comps, ranks))
        chosen, cost = [], 0.0
        for name, comp, frac, c in self.ACTIONS:
            if util() <= self.target:
                break
            frac = (self.world - 1) / self.world if frac is None else frac
            if frac <= 0 or all(cm.get(comp, 0) == 0 for cm in comps):
                continue
            for cm in comps:
                cm[comp] = cm.get(comp, 0) * (1 - frac)
            chosen.append(name); cost += c
        return {"actions": chosen, "estimated_slowdown": cost, "utilisation_after": util(), "feasible": util() <= self.target}


# ================================================================================================ debugging
class CollectiveRecorder:
    """Per-rank log of collective calls (operation, element count, dtype, group); logs from all ranks are compared to find the
    first call at which they disagree — the usual cause of a hang."""

    def __init__(self, rank: int): self.rank, self.calls = rank, []
    def record(self, op: str, numel: int, dtype: str = "float32", group: str = "world"): self.calls.append((op, numel, dtype, group))

    @staticmethod
    def first_mismatch(logs: dict[int, list]) -> dict | None:
        n = max(len(l) for l in logs.values())
        for i in range(n):
            seen = {r: (l[i] if i < len(l) else None) for r, l in logs.items()}
            if len(set(seen.values())) > 1:
                major = Counter(seen.values()).most_common(1)[0][0]
                odd = sorted(r for r, c in seen.items() if c != major)
                return {"index": i, "expected": major, "ranks": odd, "got": {r: seen[r] for r in odd},
                        "diagnosis": "rank(s) stopped issuing collectives" if all(seen[r] is None for r in odd) else "different operation or size: the ranks will wait for each other forever"}
        return None


def tensor_fingerprint(t: torch.Tensor) -> str: return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()[:16]


def find_divergence(per_rank_state: dict[int, dict[str, torch.Tensor]], atol: float = 0.0) -> list[dict]:
    """Parameters that should be replicated but differ between ranks, with the largest difference and the ranks that
    disagree with rank 0."""
    ranks = sorted(per_rank_state)
    ref, out = per_rank_state[ranks[0]], []
    for name, t in ref.items():
        bad = {}
        for r in ranks[1:]:
            d = float((per_rank_state[r][name].double() - t.double()).abs().max())
            if d > atol:
                bad[r] = d
        if bad:
            out.append({"name": name, "ranks": sorted(bad), "max_abs_diff": max(bad.values())})
    return sorted(out, key=lambda e: -e["max_abs_diff"])


def diagnose_hang(heartbeats: dict[int, dict], now: float, timeout: float = 30.0) -> dict:
    """From each rank's last heartbeat ``{"time", "step", "phase"}``: which ranks are silent, which are behind, and on what the
    others are waiting."""
    silent = sorted(r for r, h in heartbeats.items() if now - h["time"] > timeout)
    front = max(h["step"] for h in heartbeats.values())
    behind = sorted(r for r, h in heartbeats.items() if h["step"] < front)
    waiting = Counter(h["phase"] for r, h in heartbeats.items() if r not in silent and h["step"] == front)
    culprit = silent or behind
    return {"silent": silent, "behind": behind, "front_step": front, "waiting_on": waiting.most_common(1)[0][0] if waiting else None,
            "suspect": culprit[0] if culprit else None, "summary": (f"rank {culprit[0]} " + ("sends no heartbeat" if silent else f"is at step {heartbeats[culprit[0]]['step']} of {front}")) if culprit else "no rank stands out"}


# ================================================================================================ NCCL choices from a latency-bandwidth model
@dataclass
class FabricModel:
    """Per-GPU link bandwidth (bytes / s, one direction), base latency per hop and per-launch overhead; the defaults are a
    B200 on NVLink 5 through NVSwitch (770 GB/s measured peer copy)."""
    bandwidth: float = 770e9
    hop_latency: float = 1.5e-6
    launch: float = 6e-6
    nvls: bool = True

    def allreduce_time(self, nbytes: float, n: int, algo: str) -> float:
        if n == 1:
            return 0.0
        if algo == "ring":
            return self.launch + 2 * (n - 1) * self.hop_latency + 2 * (n - 1) / n * nbytes / self.bandwidth
        if algo == "tree":
            return self.launch + 2 * math.ceil(math.log2(n)) * self.hop_latency + 2 * nbytes / self.bandwidth * (1.0 if n > 2 else 0.5)
        if algo == "nvls":                                                      # reduce in the switch: each GPU sends and receives its data once
            return self.launch + 2 * self.hop_latency + (n + 1) / n * nbytes / self.bandwidth if self.nvls else math.inf
        raise ValueError(algo)

    def best_allreduce(self, nbytes: float, n: int) -> tuple[str, float]:
        t = {a: self.allreduce_time(nbytes, n, a) for a in ("ring", "tree", "nvls")}
        a = min(t, key=t.get)
        return a, t[a]


def nccl_environment(message_bytes: int, world: int, fabric: FabricModel | None = None, fault_tolerant_test: bool = False) -> dict:
    """Environment for NCCL matched to the dominant message size.  Returned, never exported: the caller decides.  A
    fault-tolerance test keeps NVLS off so that a rank that leaves never holds switch multicast memory."""
    fabric = fabric or FabricModel()
    algo, _ = fabric.best_allreduce(message_bytes, world)
    env = {"NCCL_ALGO": {"ring": "Ring", "tree": "Tree", "nvls": "NVLS"}[algo], "NCCL_PROTO": "LL" if message_bytes <= 64 << 10 else "LL128" if message_bytes <= 4 << 20 else "Simple",
           "NCCL_NVLS_ENABLE": "1" if algo == "nvls" else "0", "NCCL_MIN_NCHANNELS": str(4 if message_bytes < 1 << 20 else 16), "NCCL_BUFFSIZE": str(max(4 << 20, min(64 << 20, message_bytes // 8)))}
    if fault_tolerant_test:
        env.update(NCCL_NVLS_ENABLE="0", NCCL_ALGO="Ring" if algo == "nvls" else env["NCCL_ALGO"])
    return env


def optimal_bucket_bytes(total_bytes: float, world: int, backward_seconds: float, fabric: FabricModel | None = None, candidates=(1 << 20, 4 << 20, 16 << 20, 25 << 20, 64 << 20, 256 << 20),
                         interference: float = 0.15) -> dict:
    """Gradient bucket size for overlapped data parallelism: buckets become ready uniformly during backward; the exposed time
    is what remains of the communication queue when backward ends, and overlapped communication still costs the compute
    ``interference`` of its duration (the SMs and memory bandwidth it takes).  Small buckets pay launch latency many times,
    one huge bucket cannot overlap."""
    fabric = fabric or FabricModel()
    rows = {}
    for b in candidates:
        nb = max(1, math.ceil(total_bytes / b))
        t_bucket = fabric.best_allreduce(total_bytes / nb, world)[1]
        free = 0.0
        for i in range(nb):
            ready = backward_seconds * (i + 1) / nb
            free = max(free, ready) + t_bucket
        rows[b] = {"buckets": nb, "exposed": free - backward_seconds, "comm_total": nb * t_bucket, "cost": free - backward_seconds + interference * nb * t_bucket}
    best = min(rows, key=lambda b: (round(rows[b]["cost"], 9), -b))
    return {"bucket_bytes": best, "table": rows}


# ================================================================================================ benchmark arithmetic
_BUS_FACTOR = {"all_reduce": lambda n: 2 * (n - 1) / n, "all_gather": lambda n: (n - 1) / n, "reduce_scatter": lambda n: (n - 1) / n, "broadcast": lambda n: 1.0, "reduce": lambda n: 1.0, "all_to_all": lambda n: (n - 1) / n}


def bus_bandwidth(collective: str, nbytes: float, seconds: float, world: int) -> dict:
    """Algorithm bandwidth (payload / time) and bus bandwidth (what each link carried), comparable across rank counts."""
    alg = nbytes / seconds
    return {"algbw": alg, "busbw": alg * _BUS_FACTOR[collective](world)}


def fit_alpha_beta(sizes: Sequence[float], seconds: Sequence[float]) -> dict:
    """Least-squares ``t = alpha + size / beta``: launch-plus-latency and asymptotic bandwidth of a sweep; ``half_size`` is the
    message at which half of the asymptotic bandwidth is reached."""
    import numpy as np
    A = np.stack([np.ones(len(sizes)), np.asarray(sizes, float)], 1)
    (alpha, inv_beta), *_ = np.linalg.lstsq(A, np.asarray(seconds, float), rcond=None)
    return {"alpha": float(alpha), "beta": float(1 / inv_beta), "half_size": float(alpha / inv_beta)}


# ================================================================================================ analytics and views
@dataclass
class StepRecord:
    rank: int
    step: int
    compute: float
    communication: float
    data: float = 0.0
    idle: float = 0.0
    samples: int = 0
    loss: float | None = None

    @property
    def total(self): return self.compute + self.communication + self.data + self.idle


class TrainingAnalytics:
    def __init__(self): self.records: list[StepRecord] = []
    def add(self, rec: StepRecord): self.records.append(rec)

    def per_rank(self) -> dict[int, dict]:
        by = defaultdict(list)
        for r in self.records:
            by[r.rank].append(r)
        return {k: {"mean_step": statistics.fmean(x.total for x in v), "compute": statistics.fmean(x.compute for x in v), "communication": statistics.fmean(x.communication for x in v), "data": statistics.fmean(x.data for x in v),
                    "idle": statistics.fmean(x.idle for x in v), "steps": len(v)} for k, v in sorted(by.items())}

    def stragglers(self, threshold: float = 1.15) -> list[dict]:
        pr = self.per_rank()
        med = statistics.median(v["compute"] + v["data"] for v in pr.values())
        return [{"rank": k, "slowdown": (v["compute"] + v["data"]) / med, "cause": "data loading" if v["data"] > 0.3 * (v["compute"] + v["data"]) else "compute"} for k, v in pr.items() if (v["compute"] + v["data"]) / med > threshold]

    def summary(self) -> dict:
        pr = self.per_rank()
        steps = defaultdict(list)
        for r in self.records:
            steps[r.step].append(r)
        step_time = statistics.fmean(max(x.total for x in v) for v in steps.values())
        samples = statistics.fmean(sum(x.samples for x in v) for v in steps.values())
        comm = statistics.fmean(v["communication"] for v in pr.values())
        comp = statistics.fmean(v["compute"] for v in pr.values())
        losses = [(s, statistics.fmean(x.loss for x in v if x.loss is not None)) for s, v in sorted(steps.items()) if any(x.loss is not None for x in v)]
        return {"ranks": len(pr), "step_time": step_time, "throughput": samples / step_time if step_time else 0.0, "communication_fraction": comm / (comm + comp) if comm + comp else 0.0,
                "load_imbalance": max(v["compute"] for v in pr.values()) / comp if comp else 1.0, "stragglers": self.stragglers(), "loss_curve": losses}

    def timeline(self, step: int, width: int = 60) -> str:
        """One text row per rank for one step: ``#`` compute, ``~`` communication, ``d`` data, ``.`` idle, scaled to the
        slowest rank."""
        recs = sorted((r for r in self.records if r.step == step), key=lambda r: r.rank)
        longest = max(r.total for r in recs)
        rows = []
        for r in recs:
            seg = [("d", r.data), ("#", r.compute), ("~", r.communication), (".", r.idle)]
            bar = "".join(ch * int(round(v / longest * width)) for ch, v in seg)
            rows.append(f"rank {r.rank:>3} |{bar:<{width}}| {r.total * 1e3:.1f} ms")
        return "\n".join(rows)

    def dashboard_html(self, title: str = "Distributed training") -> str:
        from ..utils.bench_suite import Chart
        s, pr = self.summary(), self.per_rank()
        ranks = list(pr)
        bars = Chart("time per step by rank", kind="bar", y_label="seconds")
        for comp in ("compute", "communication", "data", "idle"):
            bars.add_series(comp, ranks, [pr[r][comp] for r in ranks])
        parts = [f"<h1>{html.escape(title)}</h1>", f"<p>{s['ranks']} ranks, {s['step_time'] * 1e3:.1f} ms per step, {s['throughput']:.1f} samples/s, communication {s['communication_fraction']:.0%} of busy time, load imbalance {s['load_imbalance']:.2f}</p>", bars.to_svg()]
        if s["loss_curve"]:
            parts.append(Chart("loss", x_label="step", y_label="loss").add_series("loss", [p[0] for p in s["loss_curve"]], [p[1] for p in s["loss_curve"]]).to_svg())
        if s["stragglers"]:
            parts.append("<h2>Stragglers</h2><table><tr><th>rank</th><th>slowdown</th><th>cause</th></tr>" + "".join(f"<tr><td>{x['rank']}</td><td>{x['slowdown']:.2f}x</td><td>{x['cause']}</td></tr>" for x in s["stragglers"]) + "</table>")
        return "<!doctype html><html><head><meta charset='utf-8'><title>" + html.escape(title) + "</title></head><body>" + "\n".join(parts) + "</body></html>"


def topology_dot(world: int, gpus_per_node: int = 8, groups: dict[str, Sequence[Sequence[int]]] | None = None) -> str:
    """Graphviz view of the job: one cluster per node, NVSwitch inside, the inter-node fabric between them, and coloured edges
    for the members of each named process group (``{"tp": [[0, 1], [2, 3]], ...}``)."""
    L = ["graph job {", "  node [shape=box];"]
    nodes = math.ceil(world / gpus_per_node)
    for n in range(nodes):
        L.append(f"  subgraph cluster_{n} {{ label=\"node {n}\"; sw{n} [label=\"NVSwitch\", shape=ellipse];")
        for r in range(n * gpus_per_node, min(world, (n + 1) * gpus_per_node)):
            L.append(f"    r{r} [label=\"rank {r}\"]; r{r} -- sw{n};")
        L.append("  }")
    if nodes > 1:
        L.append("  fabric [label=\"inter-node fabric\", shape=ellipse];")
        L += [f"  sw{n} -- fabric;" for n in range(nodes)]
    colours = ["red", "blue", "darkgreen", "orange", "purple"]
    for gi, (name, members) in enumerate((groups or {}).items()):
        for grp in members:
            for a, b in zip(grp, grp[1:]):
                L.append(f"  r{a} -- r{b} [color={colours[gi % 5]}, label=\"{name}\", constraint=false];")
    L.append("}")
    return "\n".join(L) + "\n"
