"""Services around gradient computation (``crates/torsh-autograd/src``): federated learning with robust aggregation,
secure aggregation, personalisation and client selection (``federated_learning/``), communication-efficient updates
(``communication_efficient/``), gradient garbage collection (``garbage_collection.rs``), capacity planning
(``capacity_planning.rs``), operation cost analysis and record / replay (``operation_cost_analysis.rs``,
``operation_replay.rs``), health diagnostics (``health_diagnostics.rs``), progress reporting (``progress_reporting.rs``),
a breakpoint debugger over module execution (``interactive_debugger.rs``), VJP chain optimisation
(``vjp_optimization.rs``), differentiable quantum circuits with a VQE loop (``quantum_autograd.rs``), complex-valued
(Wirtinger) helpers (``complex_ops.rs``), edge-case handling and automatic recovery (``edge_case_handling.rs``,
``automatic_error_recovery.rs``)."""
from __future__ import annotations

import copy
import gc
import math
import time
import weakref
from collections import Counter, defaultdict, deque
from typing import Callable, Sequence

import torch
from torch import nn


# ================================================================================================ federated learning
def _flat(state: dict) -> torch.Tensor: return torch.cat([v.reshape(-1).double() for v in state.values()])


def _unflat(vec: torch.Tensor, like: dict) -> dict:
    out, i = {}, 0
    for k, v in like.items():
        out[k] = vec[i:i + v.numel()].reshape(v.shape).to(v.dtype); i += v.numel()
    return out


def aggregate_updates(updates: Sequence[torch.Tensor], weights=None, method: str = "fedavg", f: int = 0, trim: float = 0.1) -> torch.Tensor:
    """Robust aggregation of flat client updates: ``fedavg`` (weighted mean), ``median``, ``trimmed_mean``, ``krum`` /
    ``multi_krum`` (updates closest to their ``n - f - 2`` nearest neighbours), ``norm_clipping`` (clip to the median norm),
    ``geometric_median`` (Weiszfeld iterations)."""
    u = torch.stack([x.double() for x in updates])
    n = len(u)
    w = torch.ones(n, dtype=torch.float64) if weights is None else torch.as_tensor(weights, dtype=torch.float64)
    w = w / w.sum()
    if method == "fedavg":
        return (w[:, None] * u).sum(0)
    if method == "median":
        return u.median(0).values
    if method == "trimmed_mean":
        k = int(trim * n)
        return u.sort(0).values[k:n - k].mean(0)
    if method in ("krum", "multi_krum"):
        d = torch.cdist(u, u) ** 2
        score = d.sort(1).values[:, 1:max(n - f - 1, 2)].sum(1)
        if method == "krum":
            return u[score.argmin()]
        return u[score.argsort()[:max(n - f, 1)]].mean(0)
    if method == "norm_clipping":
        norms = u.norm(dim=1)
        clip = norms.median()
        return (w[:, None] * u * (clip / norms.clamp(min=1e-12)).clamp(max=1)[:, None]).sum(0)
    if method == "geometric_median":
        z = u.mean(0)
        for _ in range(100):
            d = (u - z).norm(dim=1).clamp(min=1e-10)
            z_new = (u / d[:, None]).sum(0) / (1 / d).sum()
            if (z_new - z).norm() < 1e-10:
                break
            z = z_new
        return z
    raise ValueError(f"unknown aggregation {method!r}")


def secure_aggregate(updates: Sequence[torch.Tensor], seed: int = 0, dropped: Sequence[int] = ()) -> tuple[torch.Tensor, list[torch.Tensor]]:
    """Pairwise-mask secure aggregation: clients ``i < j`` share a mask that ``i`` adds and ``j`` subtracts, so the server
    sees only masked vectors whose sum equals the true sum.  Masks of ``dropped`` clients are reconstructed (from the
    shared seeds) and removed.  Returns ``(sum of the surviving updates, masked vectors the server received)``."""
    n, dim = len(updates), updates[0].numel()
    pair = lambda i, j: torch.randn(dim, generator=torch.Generator().manual_seed(seed * 1_000_003 + i * 1009 + j), dtype=torch.float64)
    masked = []
    for i, u in enumerate(updates):
        m = u.double().clone()
        for j in range(n):
            if j != i:
                m += pair(min(i, j), max(i, j)) * (1 if i < j else -1)
        masked.append(m)
    alive = [i for i in range(n) if i not in dropped]
    total = sum(masked[i] for i in alive)
    for d in dropped:                                                        # the dropped client's pair masks no longer cancel
        for i in alive:
            total -= pair(min(i, d), max(i, d)) * (1 if i < d else -1)
    return total, masked


class FederatedServer:
    """Round loop: select clients, send the global model, collect local updates (``local_train(model, client) -> samples``),
    aggregate, apply with a server learning rate; supports FedProx (proximal term added through ``proximal_mu`` passed to the
    client), server momentum (FedAvgM) and differential privacy (clip + Gaussian noise on every update)."""

    def __init__(self, model: nn.Module, aggregation: str = "fedavg", server_lr: float = 1.0, momentum: float = 0.0, byzantine: int = 0,
                 dp_clip: float | None = None, dp_noise: float = 0.0, seed: int = 0):
        self.model, self.aggregation, self.lr, self.mom, self.f, self.clip, self.noise = model, aggregation, server_lr, momentum, byzantine, dp_clip, dp_noise
        self.gen, self.velocity, self.history = torch.Generator().manual_seed(seed), None, []

    def select(self, clients: Sequence, k: int, strategy: str = "random", scores: dict | None = None) -> list:
        if strategy == "random":
            return [clients[i] for i in torch.randperm(len(clients), generator=self.gen)[:k].tolist()]
        if strategy == "round_robin":
            start = len(self.history) * k
            return [clients[(start + i) % len(clients)] for i in range(k)]
        w = torch.tensor([max(scores.get(c, 0.0), 1e-12) for c in clients], dtype=torch.float64)       # "importance": by loss / data size / utility
        return [clients[i] for i in torch.multinomial(w, k, False, generator=self.gen).tolist()]

    def round(self, clients: Sequence, local_train: Callable[[nn.Module, object], int]) -> dict:
        base = {k: v.detach().clone() for k, v in self.model.state_dict().items() if v.is_floating_point()}
        g0 = _flat(base)
        ups, ns = [], []
        for c in clients:
            local = copy.deepcopy(self.model)
            n = local_train(local, c)
            d = _flat({k: v for k, v in local.state_dict().items() if k in base}) - g0
            if self.clip is not None:
                d = d * min(1.0, self.clip / max(float(d.norm()), 1e-12))
                d = d + self.noise * self.clip * torch.randn(d.shape, generator=self.gen, dtype=torch.float64)
            ups.append(d); ns.append(n)
        agg = aggregate_updates(ups, ns, self.aggregation, self.f)
        if self.mom:
            self.velocity = agg if self.velocity is None else self.mom * self.velocity + agg
            agg = self.velocity
        new = _unflat(g0 + self.lr * agg, base)
        self.model.load_state_dict({**self.model.state_dict(), **new})
        rec = {"clients": len(clients), "update_norm": float(agg.norm()), "client_norms": [float(u.norm()) for u in ups],
               "divergence": float(torch.stack([(u - agg).norm() for u in ups]).mean())}
        self.history.append(rec)
        return rec


def fedprox_penalty(local: nn.Module, global_state: dict, mu: float) -> torch.Tensor:
    return 0.5 * mu * sum(((p - global_state[n]) ** 2).sum() for n, p in local.named_parameters())


def personalize(global_model: nn.Module, client_data, train: Callable[[nn.Module, object], None], shared_prefixes: Sequence[str] = ()) -> nn.Module:
    """Local fine-tuning of a copy of the global model; parameters under ``shared_prefixes`` stay frozen (FedPer: shared body,
    personal head)."""
    m = copy.deepcopy(global_model)
    for n, p in m.named_parameters():
        p.requires_grad_(not any(n.startswith(s) for s in shared_prefixes))
    train(m, client_data)
    return m


# ================================================================================================ communication-efficient updates
class LocalSGDController:
    """Decides when replicas synchronise: every ``period`` steps, with the period adapted to the measured divergence
    between replicas (halve when it exceeds ``high``, double when under ``low``), inside ``[min_period, max_period]``."""

    def __init__(self, period: int = 8, low: float = 0.01, high: float = 0.1, min_period: int = 1, max_period: int = 64):
        self.period, self.low, self.high, self.min, self.max, self.step_count, self.syncs = period, low, high, min_period, max_period, 0, 0

    def should_sync(self) -> bool:
        self.step_count += 1
        return self.step_count % self.period == 0

    def after_sync(self, relative_divergence: float):
        self.syncs += 1
        if relative_divergence > self.high:
            self.period = max(self.min, self.period // 2)
        elif relative_divergence < self.low:
            self.period = min(self.max, self.period * 2)


def encode_update(delta: torch.Tensor, method: str = "topk", ratio: float = 0.01, bits: int = 8, generator=None) -> dict:
    """``topk`` (indices + values), ``randk`` (unbiased: values scaled by ``1 / ratio``), ``sign`` (1 bit + mean magnitude),
    ``quantize`` (stochastic uniform quantisation to ``bits``); ``decode_update`` restores a dense tensor."""
    flat = delta.reshape(-1)
    n = flat.numel()
    if method in ("topk", "randk"):
        k = max(1, int(ratio * n))
        idx = flat.abs().topk(k).indices if method == "topk" else torch.randperm(n, generator=generator)[:k]
        vals = flat[idx] * (n / k if method == "randk" else 1.0)
        return {"method": method, "shape": delta.shape, "indices": idx.to(torch.int32), "values": vals, "bytes": k * (4 + flat.element_size())}
    if method == "sign":
        return {"method": method, "shape": delta.shape, "sign": flat >= 0, "scale": flat.abs().mean(), "bytes": math.ceil(n / 8) + 4}
    lo, hi = flat.min(), flat.max()
    levels = 2 ** bits - 1
    x = (flat - lo) / (hi - lo).clamp(min=1e-30) * levels
    q = torch.floor(x + torch.rand(x.shape, generator=generator)).clamp(0, levels).to(torch.uint8 if bits <= 8 else torch.int32)
    return {"method": "quantize", "shape": delta.shape, "q": q, "lo": lo, "hi": hi, "levels": levels, "bytes": math.ceil(n * bits / 8) + 8}


def decode_update(msg: dict) -> torch.Tensor:
    n = math.prod(msg["shape"])
    if msg["method"] in ("topk", "randk"):
        return torch.zeros(n, dtype=msg["values"].dtype).index_put_((msg["indices"].long(),), msg["values"]).reshape(msg["shape"])
    if msg["method"] == "sign":
        return (torch.where(msg["sign"], 1.0, -1.0) * msg["scale"]).reshape(msg["shape"])
    return (msg["q"].float() / msg["levels"] * (msg["hi"] - msg["lo"]) + msg["lo"]).reshape(msg["shape"])


# ================================================================================================ gradient garbage collection
class GradientGarbageCollector:
    """Tracks tensors (weakly) with a generation counter: a tensor that survives a collection moves to an older generation,
    young generations are scanned more often; ``collect`` drops ``.grad`` of tracked tensors that were not touched for
    ``max_idle`` ticks and forgets dead references."""

    def __init__(self, max_idle: int = 3, generations: int = 3, thresholds=(1, 4, 16)):
        self.max_idle, self.n_gen, self.thresholds, self.tick_count = max_idle, generations, thresholds, 0
        self.refs: dict[int, dict] = {}
        self.stats = {"collections": 0, "freed_grads": 0, "freed_bytes": 0, "dead_refs": 0}

    def track(self, t: torch.Tensor): self.refs[id(t)] = {"ref": weakref.ref(t), "gen": 0, "last": self.tick_count}

    def touch(self, t: torch.Tensor):
        if id(t) in self.refs:
            self.refs[id(t)]["last"] = self.tick_count

    def tick(self): self.tick_count += 1

    def collect(self, force: bool = False) -> dict:
        freed, bytes_, dead = 0, 0, 0
        for key, r in list(self.refs.items()):
            if not force and self.tick_count % self.thresholds[min(r["gen"], len(self.thresholds) - 1)]:
                continue
            t = r["ref"]()
            if t is None:
                del self.refs[key]; dead += 1
                continue
            if t.grad is not None and (force or self.tick_count - r["last"] >= self.max_idle):
                bytes_ += t.grad.numel() * t.grad.element_size()
                t.grad = None
                freed += 1
            r["gen"] = min(r["gen"] + 1, self.n_gen - 1)
        self.stats["collections"] += 1; self.stats["freed_grads"] += freed; self.stats["freed_bytes"] += bytes_; self.stats["dead_refs"] += dead
        return {"freed_grads": freed, "freed_bytes": bytes_, "dead_refs": dead, "tracked": len(self.refs)}


# ================================================================================================ capacity planning / cost analysis
class CapacityPlanner:
    """Linear and seasonal (weekly) trend over daily peak usage; forecasts the horizon, the day capacity is exhausted, and
    recommends scaling with an urgency level."""

    def __init__(self, capacity: float, headroom: float = 0.2): self.capacity, self.headroom, self.days = capacity, headroom, []
    def record_day(self, peak_usage: float): self.days.append(float(peak_usage))

    def forecast(self, horizon: int = 30) -> dict:
        y = torch.tensor(self.days, dtype=torch.float64)
        t = torch.arange(len(y), dtype=torch.float64)
        X = torch.stack([t, torch.ones_like(t)], 1)
        slope, icpt = torch.linalg.lstsq(X, y[:, None]).solution[:, 0].tolist()
        resid = y - (slope * t + icpt)
        season = torch.stack([resid[d::7].mean() if len(resid[d::7]) else torch.tensor(0.0, dtype=torch.float64) for d in range(7)]) if len(y) >= 14 else torch.zeros(7, dtype=torch.float64)
        fut = torch.arange(len(y), len(y) + horizon, dtype=torch.float64)
        pred = slope * fut + icpt + season[(fut.long() % 7)]
        limit = self.capacity * (1 - self.headroom)
        over = (pred > limit).nonzero()
        days_left = int(over[0]) if len(over) else None
        urgency = "none" if days_left is None else "critical" if days_left <= 3 else "high" if days_left <= 7 else "medium" if days_left <= 14 else "low"
        need = float(pred.max()) / (1 - self.headroom)
        return {"trend_per_day": slope, "direction": "growing" if slope > 1e-9 else "shrinking" if slope < -1e-9 else "flat", "forecast": pred, "days_until_exhausted": days_left,
                "urgency": urgency, "action": "scale_up" if days_left is not None else ("scale_down" if need < 0.5 * self.capacity else "hold"), "recommended_capacity": max(need, 0.0)}


class OperationCostAnalyzer:
    """Aggregates recorded operation costs (time, memory, FLOPs) per operation type and suggests where optimisation pays:
    the largest time share, low arithmetic intensity, many tiny calls."""

    def __init__(self): self.entries = []
    def record(self, op: str, seconds: float, bytes_: float = 0.0, flops: float = 0.0, phase: str = "forward"): self.entries.append({"op": op, "s": seconds, "bytes": bytes_, "flops": flops, "phase": phase})

    def aggregate(self) -> dict:
        out = defaultdict(lambda: {"calls": 0, "seconds": 0.0, "bytes": 0.0, "flops": 0.0})
        for e in self.entries:
            a = out[e["op"]]
            a["calls"] += 1; a["seconds"] += e["s"]; a["bytes"] += e["bytes"]; a["flops"] += e["flops"]
        total = sum(a["seconds"] for a in out.values()) or 1.0
        for a in out.values():
            a["share"], a["mean_seconds"], a["intensity"] = a["seconds"] / total, a["seconds"] / a["calls"], a["flops"] / a["bytes"] if a["bytes"] else None
        return dict(out)

    def phase_breakdown(self): c = Counter(); [c.update({e["phase"]: e["s"]}) for e in self.entries]; return dict(c)

    def suggestions(self, balance: float = 200.0, tiny: float = 20e-6) -> list[dict]:
        out = []
        for op, a in sorted(self.aggregate().items(), key=lambda kv: -kv[1]["share"]):
            if a["share"] > 0.3:
                out.append({"op": op, "priority": "high", "kind": "hotspot", "text": f"{op} takes {a['share']:.0%} of the time"})
            if a["intensity"] is not None and a["intensity"] < balance and a["share"] > 0.05:
                out.append({"op": op, "priority": "medium", "kind": "memory_bound", "text": f"{op} does {a['intensity']:.1f} FLOP/byte: fuse it with its neighbours"})
            if a["calls"] >= 50 and a["mean_seconds"] < tiny:
                out.append({"op": op, "priority": "medium", "kind": "launch_bound", "text": f"{op}: {a['calls']} calls of {a['mean_seconds'] * 1e6:.1f} us: batch them or capture a CUDA graph"})
        return out


# ================================================================================================ record / replay
class OperationRecorder:
    """Records calls ``(name, fn, inputs, output)`` of a computation so it can be replayed later, on the same inputs (for
    determinism checks and timing comparison) or on substituted ones."""

    def __init__(self): self.session = []

    def call(self, name: str, fn: Callable, *args):
        t0 = time.perf_counter()
        out = fn(*args)
        self.session.append({"name": name, "fn": fn, "args": [a.detach().clone() if isinstance(a, torch.Tensor) else a for a in args],
                             "output": out.detach().clone() if isinstance(out, torch.Tensor) else out, "seconds": time.perf_counter() - t0})
        return out


class OperationReplayer:
    def __init__(self, session: list): self.session = session

    def replay(self, atol: float = 0.0, substitute: dict[int, list] | None = None) -> dict:
        mismatches, timings = [], []
        for i, rec in enumerate(self.session):
            args = (substitute or {}).get(i, rec["args"])
            t0 = time.perf_counter()
            out = rec["fn"](*args)
            timings.append((rec["seconds"], time.perf_counter() - t0))
            if i not in (substitute or {}) and isinstance(out, torch.Tensor) and not torch.allclose(out, rec["output"], atol=atol, rtol=0, equal_nan=True):
                mismatches.append({"index": i, "name": rec["name"], "max_abs_diff": float((out - rec["output"]).abs().max())})
        return {"operations": len(self.session), "mismatches": mismatches, "deterministic": not mismatches, "recorded_seconds": sum(a for a, _ in timings), "replayed_seconds": sum(b for _, b in timings)}


# ================================================================================================ health / progress / debugger
class HealthDiagnostics:
    """Checks gradients (finite, not vanishing / exploding, present), the graph (parameters without gradient, unused
    parameters), memory (growth across recent steps) and step time (slowdown against its own median)."""

    def __init__(self, vanish: float = 1e-8, explode: float = 1e3): self.vanish, self.explode, self.mem, self.times = vanish, explode, deque(maxlen=50), deque(maxlen=50)

    def record_step(self, seconds: float, memory_bytes: float): self.times.append(seconds); self.mem.append(memory_bytes)

    def check(self, model: nn.Module) -> dict:
        issues = []
        for n, p in model.named_parameters():
            if not p.requires_grad:
                continue
            if p.grad is None:
                issues.append(("graph", "warning", f"{n} received no gradient (unused or detached)"))
                continue
            g = p.grad
            if not torch.isfinite(g).all():
                issues.append(("gradient", "critical", f"{n} has non-finite gradient"))
                continue
            gn = float(g.norm())
            if gn < self.vanish:
                issues.append(("gradient", "warning", f"{n} gradient norm {gn:.1e} vanishes"))
            elif gn > self.explode:
                issues.append(("gradient", "warning", f"{n} gradient norm {gn:.1e} explodes"))
        if len(self.mem) >= 10 and self.mem[-1] > 1.5 * self.mem[0] and all(b >= a for a, b in zip(list(self.mem)[-10:], list(self.mem)[-9:])):
            issues.append(("memory", "warning", f"memory grew {self.mem[-1] / max(self.mem[0], 1):.1f}x and is still rising"))
        if len(self.times) >= 10:
            med = sorted(self.times)[len(self.times) // 2]
            if self.times[-1] > 2 * med:
                issues.append(("performance", "warning", f"last step took {self.times[-1] / med:.1f}x the median"))
        status = "critical" if any(s == "critical" for _, s, _ in issues) else "degraded" if issues else "healthy"
        return {"status": status, "issues": [{"category": c, "severity": s, "message": m} for c, s, m in issues]}


class ProgressReporter:
    """Step progress with smoothed rate and ETA; ``scope(name, total)`` nests; updates go to ``sink(dict)`` at most every
    ``min_interval`` seconds (always on completion)."""

    def __init__(self, total: int, sink: Callable[[dict], None] | None = None, min_interval: float = 0.0, clock=time.perf_counter):
        self.total, self.done, self.sink, self.min_interval, self.clock = total, 0, sink or (lambda d: None), min_interval, clock
        self.t0 = self.last_emit = clock()
        self.rate, self.updates, self.children = None, [], []

    def update(self, n: int = 1, **info):
        now = self.clock()
        inst = n / max(now - getattr(self, "_last_t", self.t0), 1e-12)
        self._last_t = now
        self.rate = inst if self.rate is None else 0.7 * self.rate + 0.3 * inst
        self.done += n
        if now - self.last_emit >= self.min_interval or self.done >= self.total:
            u = {"done": self.done, "total": self.total, "fraction": self.done / self.total, "rate": self.rate, "eta_s": (self.total - self.done) / max(self.rate, 1e-12), "elapsed_s": now - self.t0, **info}
            self.updates.append(u); self.sink(u); self.last_emit = now

    def scope(self, name: str, total: int) -> "ProgressReporter":
        child = ProgressReporter(total, lambda d: self.sink({"scope": name, **d}), self.min_interval, self.clock)
        self.children.append((name, child))
        return child

    def statistics(self): return {"steps": self.done, "elapsed_s": self.clock() - self.t0, "mean_rate": self.done / max(self.clock() - self.t0, 1e-12), "updates": len(self.updates)}


class InteractiveDebugger:
    """Breakpoints on module execution: by module name, by a condition on the output (``nan``, ``inf``, ``norm_above``,
    custom callable), or on the gradient flowing back.  When one fires, the scripted ``commands`` are executed against the
    paused context (``print``, ``stats``, ``watch <name>``, ``continue``, ``abort``), so a session is reproducible in tests."""

    def __init__(self, model: nn.Module, commands: Sequence[str] = ("stats", "continue")):
        self.model, self.commands, self.breakpoints, self.watch, self.log, self.hits, self.handles = model, list(commands), [], {}, [], [], []

    def add_breakpoint(self, module: str | None = None, condition: str | Callable | None = None, threshold: float = 0.0, on: str = "forward"):
        self.breakpoints.append({"module": module, "condition": condition, "threshold": threshold, "on": on})

    def _fires(self, bp, name, t):
        if bp["module"] is not None and bp["module"] != name:
            return False
        c = bp["condition"]
        if c is None:
            return True
        if callable(c):
            return bool(c(t))
        return {"nan": lambda: bool(torch.isnan(t).any()), "inf": lambda: bool(torch.isinf(t).any()), "norm_above": lambda: float(t.detach().norm()) > bp["threshold"]}[c]()

    def _pause(self, kind, name, t):
        self.hits.append({"kind": kind, "module": name})
        for cmd in self.commands:
            if cmd == "stats":
                t = t.detach()
                self.log.append({"module": name, "kind": kind, "mean": float(t.float().mean()), "std": float(t.float().std()) if t.numel() > 1 else 0.0, "norm": float(t.float().norm()),
                                 "nan": int(torch.isnan(t).sum()), "shape": tuple(t.shape)})
            elif cmd == "print":
                self.log.append({"module": name, "kind": kind, "tensor": t.detach().clone()})
            elif cmd.startswith("watch "):
                self.watch.setdefault(cmd.split(" ", 1)[1], None)
            elif cmd == "abort":
                raise RuntimeError(f"aborted at breakpoint in {name} ({kind})")
            elif cmd == "continue":
                break

    def attach(self):
        for name, m in self.model.named_modules():
            if not name:
                continue
            def fwd(mod, inp, out, name=name):
                if name in self.watch and isinstance(out, torch.Tensor):
                    self.watch[name] = out.detach().clone()
                if isinstance(out, torch.Tensor):
                    for bp in self.breakpoints:
                        if bp["on"] == "forward" and self._fires(bp, name, out):
                            self._pause("forward", name, out)
            def bwd(mod, gin, gout, name=name):
                if gout and gout[0] is not None:
                    for bp in self.breakpoints:
                        if bp["on"] == "backward" and self._fires(bp, name, gout[0]):
                            self._pause("backward", name, gout[0])
            self.handles += [m.register_forward_hook(fwd), m.register_full_backward_hook(bwd)]
        return self

    def detach(self):
        for h in self.handles:
            h.remove()
        self.handles.clear()


# ================================================================================================ VJP chains
class VjpOptimizer:
    """A chain of linear maps ``y = A_k ... A_2 A_1 x``: the pullback ``v^T A_k ... A_1`` is cheapest evaluated from the
    output side, and sub-chains of matrices can be pre-multiplied when that lowers the total cost for repeated use
    (matrix-chain ordering by dynamic programming); element-wise (diagonal) maps fuse into their neighbours."""

    def __init__(self): self.ops = []
    def add_matrix(self, a: torch.Tensor): self.ops.append(("matrix", a)); return self
    def add_diagonal(self, d: torch.Tensor): self.ops.append(("diag", d)); return self

    def fuse(self) -> "VjpOptimizer":
        out = VjpOptimizer()
        for kind, t in self.ops:
            if kind == "diag" and out.ops and out.ops[-1][0] == "diag":
                out.ops[-1] = ("diag", out.ops[-1][1] * t)
            elif kind == "diag" and out.ops and out.ops[-1][0] == "matrix":
                out.ops[-1] = ("matrix", t[:, None] * out.ops[-1][1])
            else:
                out.ops.append((kind, t))
        return out

    def vjp(self, v: torch.Tensor) -> torch.Tensor:
        for kind, t in reversed(self.ops):
            v = v @ t if kind == "matrix" else v * t
        return v

    def jvp(self, x: torch.Tensor) -> torch.Tensor:
        for kind, t in self.ops:
            x = t @ x if kind == "matrix" else t * x
        return x

    @staticmethod
    def chain_order(dims: Sequence[int]) -> tuple[int, str]:
        """Optimal parenthesisation of ``A_1 (d0 x d1) ... A_n``; returns ``(scalar multiplications, expression)``."""
        n = len(dims) - 1
        cost = [[0] * n for _ in range(n)]
        split = [[0] * n for _ in range(n)]
        for length in range(2, n + 1):
            for i in range(n - length + 1):
                j = i + length - 1
                cost[i][j], split[i][j] = min((cost[i][k] + cost[k + 1][j] + dims[i] * dims[k + 1] * dims[j + 1], k) for k in range(i, j))
        def expr(i, j): return f"A{i + 1}" if i == j else f"({expr(i, split[i][j])} {expr(split[i][j] + 1, j)})"
        return cost[0][n - 1], expr(0, n - 1)

    def costs(self, batch: int = 1) -> dict:
        mats = [t for k, t in self.ops if k == "matrix"]
        per_vjp = sum(t.numel() for t in mats) * batch
        dims = [mats[0].shape[1]] + [t.shape[0] for t in mats]
        full, _ = self.chain_order(dims[::-1]) if len(mats) > 1 else (0, "")
        return {"vjp_flops": 2 * per_vjp, "materialize_flops": 2 * full, "materialized_vjp_flops": 2 * dims[0] * dims[-1] * batch,
                "break_even_batch": math.ceil(full / max(sum(t.numel() for t in mats) - dims[0] * dims[-1], 1)) if sum(t.numel() for t in mats) > dims[0] * dims[-1] else None}


# ================================================================================================ quantum circuits
class QuantumCircuit:
    """State-vector simulator of ``n`` qubits with parameterised rotations as differentiable tensor ops (autograd gives the
    exact gradient; ``parameter_shift`` gives the hardware-style estimate).  Qubit 0 is the most significant bit."""

    def __init__(self, n_qubits: int): self.n, self.gates = n_qubits, []
    def rx(self, q, p): self.gates.append(("rx", q, p)); return self
    def ry(self, q, p): self.gates.append(("ry", q, p)); return self
    def rz(self, q, p): self.gates.append(("rz", q, p)); return self
    def h(self, q): self.gates.append(("h", q, None)); return self
    def x(self, q): self.gates.append(("x", q, None)); return self
    def cnot(self, c, t): self.gates.append(("cnot", c, t)); return self

    @staticmethod
    def _matrix(kind, theta):
        c = torch.complex128
        if kind == "h":
            return torch.tensor([[1, 1], [1, -1]], dtype=c) / math.sqrt(2)
        if kind == "x":
            return torch.tensor([[0, 1], [1, 0]], dtype=c)
        co, si = torch.cos(theta / 2).to(c), torch.sin(theta / 2).to(c)
        if kind == "rx":
            return torch.stack([torch.stack([co, -1j * si]), torch.stack([-1j * si, co])])
        if kind == "ry":
            return torch.stack([torch.stack([co, -si]), torch.stack([si, co])])
        return torch.stack([torch.stack([torch.exp(-0.5j * theta.to(c)), torch.zeros((), dtype=c)]), torch.stack([torch.zeros((), dtype=c), torch.exp(0.5j * theta.to(c))])])

    def run(self, params: torch.Tensor) -> torch.Tensor:
        state = torch.zeros(2 ** self.n, dtype=torch.complex128)
        state[0] = 1
        state = state.reshape([2] * self.n)
        for kind, a, b in self.gates:
            if kind == "cnot":
                idx = [slice(None)] * self.n
                idx[a] = 1
                sub = state[tuple(idx)]
                tdim = b if b < a else b - 1
                state = torch.stack([state.select(a, 0), sub.flip(tdim)], a)
            else:
                theta = params[b].double() if b is not None else None
                state = torch.movedim(torch.tensordot(self._matrix(kind, theta), state, dims=([1], [a])), 0, a)
        return state.reshape(-1)

    def expectation(self, params: torch.Tensor, observable: torch.Tensor) -> torch.Tensor:
        s = self.run(params)
        return (s.conj() @ (observable.to(torch.complex128) @ s)).real

    def parameter_shift(self, params: torch.Tensor, observable: torch.Tensor) -> torch.Tensor:
        g = torch.zeros_like(params, dtype=torch.float64)
        for i in range(len(params)):
            e = torch.zeros_like(params); e[i] = math.pi / 2
            g[i] = 0.5 * (self.expectation(params + e, observable) - self.expectation(params - e, observable))
        return g


def pauli_string(ops: str) -> torch.Tensor:
    """Kronecker product of single-qubit Paulis, e.g. ``"ZZ"`` or ``"XI"``."""
    m = {"I": torch.eye(2, dtype=torch.complex128), "X": torch.tensor([[0, 1], [1, 0]], dtype=torch.complex128), "Y": torch.tensor([[0, -1j], [1j, 0]], dtype=torch.complex128),
         "Z": torch.tensor([[1, 0], [0, -1]], dtype=torch.complex128)}
    out = m[ops[0]]
    for o in ops[1:]:
        out = torch.kron(out, m[o])
    return out


def vqe(circuit: QuantumCircuit, hamiltonian: torch.Tensor, n_params: int, steps: int = 200, lr: float = 0.1, seed: int = 0) -> dict:
    """Variational quantum eigensolver: minimise the energy expectation over circuit parameters with Adam."""
    p = torch.nn.Parameter(0.1 * torch.randn(n_params, generator=torch.Generator().manual_seed(seed), dtype=torch.float64))
    opt = torch.optim.Adam([p], lr)
    hist = []
    for _ in range(steps):
        e = circuit.expectation(p, hamiltonian)
        opt.zero_grad(); e.backward(); opt.step()
        hist.append(float(e.detach()))
    return {"energy": hist[-1], "params": p.detach(), "history": hist, "exact": float(torch.linalg.eigvalsh(hamiltonian)[0])}


# ================================================================================================ complex helpers
def wirtinger_grad(f: Callable[[torch.Tensor], torch.Tensor], z: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(df/dz, df/dz*)`` of a real- or complex-valued scalar function by differentiating with respect to real and
    imaginary parts: ``d/dz = (d/dx - i d/dy) / 2``, ``d/dz* = (d/dx + i d/dy) / 2``."""
    x, y = z.real.clone().requires_grad_(True), z.imag.clone().requires_grad_(True)
    out = f(torch.complex(x, y))
    parts = []
    for comp in ((out.real, out.imag) if out.is_complex() else (out, None)):
        if comp is None:
            parts.append((torch.zeros_like(x), torch.zeros_like(y)))
        else:
            gx, gy = torch.autograd.grad(comp, (x, y), retain_graph=True, allow_unused=True)
            parts.append((gx if gx is not None else torch.zeros_like(x), gy if gy is not None else torch.zeros_like(y)))
    (ux, uy), (vx, vy) = parts
    fx, fy = torch.complex(ux, vx), torch.complex(uy, vy)
    return (fx - 1j * fy) / 2, (fx + 1j * fy) / 2


def is_holomorphic(f, z: torch.Tensor, atol: float = 1e-8) -> bool: return bool(wirtinger_grad(f, z)[1].abs().max() < atol)


# ================================================================================================ edge cases / recovery
class EdgeCaseHandler:
    """Normalises awkward inputs before an operation: empty tensors, zero-dimensional scalars, NaN / Inf values,
    sub-normal magnitudes and extreme values, with a strategy per case (``error``, ``skip``, ``replace``, ``clamp``) and counts."""

    def __init__(self, nan: str = "replace", inf: str = "clamp", empty: str = "skip", denormal: str = "replace", limit: float = 1e30, fill: float = 0.0):
        self.policy, self.limit, self.fill, self.stats = {"nan": nan, "inf": inf, "empty": empty, "denormal": denormal}, limit, fill, Counter()

    def handle(self, t: torch.Tensor) -> tuple[torch.Tensor | None, list[str]]:
        found = []
        if t.numel() == 0:
            self.stats["empty"] += 1
            if self.policy["empty"] == "error":
                raise ValueError("empty tensor")
            return (None if self.policy["empty"] == "skip" else t), ["empty"]
        if t.dim() == 0:
            found.append("scalar"); self.stats["scalar"] += 1
            t = t.reshape(1)
        if t.is_floating_point():
            for name, mask in (("nan", torch.isnan(t)), ("inf", torch.isinf(t))):
                if mask.any():
                    found.append(name); self.stats[name] += int(mask.sum())
                    if self.policy[name] == "error":
                        raise FloatingPointError(f"{int(mask.sum())} {name} values")
                    if self.policy[name] == "replace":
                        t = torch.where(mask, torch.full_like(t, self.fill), t)
                    elif self.policy[name] == "clamp":
                        t = torch.nan_to_num(t, nan=float("nan"), posinf=self.limit, neginf=-self.limit) if name == "inf" else t
            tiny = (t != 0) & (t.abs() < torch.finfo(t.dtype).tiny)
            if tiny.any():
                found.append("denormal"); self.stats["denormal"] += int(tiny.sum())
                if self.policy["denormal"] == "replace":
                    t = torch.where(tiny, torch.zeros_like(t), t)
            big = t.abs() > self.limit
            if big.any():
                found.append("extreme"); self.stats["extreme"] += int(big.sum())
                t = t.clamp(-self.limit, self.limit)
        return t, found


class AutomaticErrorRecovery:
    """Runs a step with a ladder of corrective actions for transient failures: on out-of-memory halve the batch (``shrink``
    callback) and empty caches; on non-finite loss lower the learning rate and restore the last good state; on other
    ``retry_on`` errors back off and retry.  Gives up after ``max_attempts`` and re-raises."""

    def __init__(self, save_state: Callable[[], object], load_state: Callable[[object], None], shrink: Callable[[], None] | None = None,
                 lower_lr: Callable[[], None] | None = None, max_attempts: int = 4, retry_on=(RuntimeError,), sleep=time.sleep):
        self.save, self.load, self.shrink, self.lower_lr, self.max_attempts, self.retry_on, self.sleep = save_state, load_state, shrink, lower_lr, max_attempts, retry_on, sleep
        self.good, self.attempts = save_state(), []

    def run(self, step: Callable[[], float]) -> float:
        last = None
        for attempt in range(self.max_attempts):
            try:
                loss = step()
                if not math.isfinite(loss):
                    raise FloatingPointError(f"non-finite loss {loss}")
                self.good = self.save()
                return loss
            except FloatingPointError as e:
                last, action = e, "restore_and_lower_lr"
                self.load(self.good)
                if self.lower_lr:
                    self.lower_lr()
            except self.retry_on as e:
                last = e
                if "out of memory" in str(e).lower():
                    action = "shrink_batch"
                    gc.collect()
                    if torch.cuda.is_available():
                        torch.cuda.empty_cache()
                    if self.shrink:
                        self.shrink()
                else:
                    action = "backoff_retry"
                    self.sleep(0.01 * 2 ** attempt)
            self.attempts.append({"attempt": attempt, "error": type(last).__name__, "action": action})
        raise last
