"""Autograd runtime services (``crates/torsh-autograd/src``): anomaly alerts with channels and cool-down
(``anomaly_alerts.rs``), error-rate windows (``error_rate_monitoring.rs``), audit log (``audit_logging.rs``), gradient
statistics (``metrics_collection.rs``), structured records (``structured_logging.rs``), exception-safe parameter
transactions and resource guards (``exception_safety.rs``, ``raii_resources/``, ``guards.rs``), graceful degradation
(``graceful_degradation.rs``), gradient validation (``gradient_validation.rs``), optimizer-aware gradient scaling
(``gradient_scaling.rs``), backward scheduling (``gradient_scheduler.rs``), gradient path tracing
(``gradient_tracer.rs``, ``gradient_tracing.rs``), operation introspection (``operation_introspection.rs``), buffer reuse
planning (``buffer_optimization.rs``), chunked gradient computation (``intelligent_chunking.rs``,
``parallel_gradient.rs``), automatic tuning (``auto_tuning.rs``), gradient regression baselines
(``regression_testing.rs``), stress graphs (``stress_testing.rs``), pluggable differentiation backends
(``custom_backends.rs``, ``external_ad_integration.rs``), tape / ``value_and_grad`` / ``autograd.grad`` compatibility layers
(``tensorflow_compat.rs``, ``mlx_compat.rs``, ``pytorch_compat.rs``, ``ad_framework_compatibility.rs``), variable
environments (``variable_env.rs``), fused function chains (``function_optimization.rs``) and matrix-product gradients
written as GEMM calls (``blas_integration.rs``)."""
from __future__ import annotations

import contextlib
import hashlib
import json
import math
import time
from collections import Counter, defaultdict, deque
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable, Sequence

import torch


# ================================================================================================ alerts and error rates
@dataclass
class Alert:
    severity: str
    kind: str
    message: str
    step: int
    context: dict = field(default_factory=dict)


class AnomalyAlertManager:
    """Rules over gradient statistics raise alerts; every channel (a callable) receives an alert whose severity reaches the
    channel's minimum; identical alerts are suppressed for ``cooldown`` steps and counted instead."""
    LEVELS = {"info": 0, "warning": 1, "critical": 2}

    def __init__(self, cooldown: int = 10): self.cooldown, self.channels, self.rules, self.history, self.suppressed, self._last = cooldown, [], [], [], Counter(), {}
    def add_channel(self, fn: Callable[[Alert], None], min_severity: str = "info"): self.channels.append((fn, self.LEVELS[min_severity])); return self
    def add_rule(self, kind: str, severity: str, predicate: Callable[[dict], bool], message: str): self.rules.append((kind, severity, predicate, message)); return self

    def with_default_rules(self, explode: float = 1e3, vanish: float = 1e-8):
        self.add_rule("non_finite", "critical", lambda s: s["nan"] + s["inf"] > 0, "non-finite gradient values")
        self.add_rule("exploding", "warning", lambda s: s["norm"] > explode, "gradient norm above the explosion threshold")
        self.add_rule("vanishing", "warning", lambda s: 0 <= s["norm"] < vanish, "gradient norm below the vanishing threshold")
        return self

    def check(self, step: int, stats: dict) -> list[Alert]:
        out = []
        for kind, sev, pred, msg in self.rules:
            if not pred(stats):
                continue
            key = (kind, stats.get("name"))
            if key in self._last and step - self._last[key] < self.cooldown:
                self.suppressed[key] += 1; continue
            self._last[key] = step
            a = Alert(sev, kind, msg, step, dict(stats))
            out.append(a); self.history.append(a)
            for fn, lvl in self.channels:
                if self.LEVELS[sev] >= lvl:
                    fn(a)
        return out


class ErrorRateMonitor:
    """Success / failure outcomes per operation over a sliding window; ``status`` compares the windowed rate with warning and
    critical thresholds, ``trend`` the newer half of the window with the older."""

    def __init__(self, window: int = 100, warn: float = 0.05, critical: float = 0.2): self.window, self.warn, self.critical, self.events, self.kinds = window, warn, critical, defaultdict(lambda: deque(maxlen=window)), defaultdict(Counter)

    def record(self, op: str, ok: bool, kind: str | None = None):
        self.events[op].append(ok)
        if not ok:
            self.kinds[op][kind or "error"] += 1

    def rate(self, op: str) -> float: e = self.events[op]; return 0.0 if not e else 1 - sum(e) / len(e)
    def status(self, op: str) -> str: r = self.rate(op); return "critical" if r >= self.critical else "warning" if r >= self.warn else "healthy"
    def trend(self, op: str) -> str:
        e = list(self.events[op]); h = len(e) // 2
        if h < 5:
            return "unknown"
        old, new = 1 - sum(e[:h]) / h, 1 - sum(e[h:]) / (len(e) - h)
        return "rising" if new > old + 0.05 else "falling" if new < old - 0.05 else "flat"
    def report(self): return {op: {"rate": self.rate(op), "status": self.status(op), "trend": self.trend(op), "kinds": dict(self.kinds[op])} for op in self.events}

    @contextlib.contextmanager
    def watch(self, op: str):
        try:
            yield
        except Exception as e:
            self.record(op, False, type(e).__name__); raise
        else:
            self.record(op, True)


class AutogradAuditLog:
    """Append-only record of who ran which differentiation on what (names, shapes, a digest of the values); each entry
    carries the hash of the previous one so that a later edit is detectable."""

    def __init__(self, path=None): self.entries, self.path = [], Path(path) if path else None

    def record(self, operation: str, actor: str = "system", tensors: dict | None = None, **details):
        prev = self.entries[-1]["hash"] if self.entries else "0" * 64
        body = {"seq": len(self.entries), "time": time.time(), "operation": operation, "actor": actor, "details": details,
                "tensors": {k: {"shape": list(v.shape), "dtype": str(v.dtype), "digest": hashlib.sha256(v.detach().cpu().contiguous().numpy().tobytes()).hexdigest()[:16]} for k, v in (tensors or {}).items()}, "prev": prev}
        body["hash"] = hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()
        self.entries.append(body)
        if self.path:
            with self.path.open("a") as f:
                f.write(json.dumps(body) + "\n")
        return body

    def verify(self) -> bool:
        prev = "0" * 64
        for e in self.entries:
            b = {k: v for k, v in e.items() if k != "hash"}
            if e["prev"] != prev or hashlib.sha256(json.dumps(b, sort_keys=True).encode()).hexdigest() != e["hash"]:
                return False
            prev = e["hash"]
        return True

    def query(self, operation: str | None = None, actor: str | None = None): return [e for e in self.entries if (operation is None or e["operation"] == operation) and (actor is None or e["actor"] == actor)]


class GradientMetricsCollector:
    """Per-parameter gradient statistics each step (norm, mean, extremes, zero fraction, non-finite counts) with running
    histories, a global norm and the update-to-weight ratio when a learning rate is given."""

    def __init__(self, history: int = 1000): self.hist, self.step_no = defaultdict(lambda: deque(maxlen=history)), 0

    @staticmethod
    def stats(name: str, g: torch.Tensor) -> dict:
        f = g.detach().float()
        fin = torch.isfinite(f)
        v = f[fin]
        return {"name": name, "norm": float(v.norm()) if v.numel() else 0.0, "mean": float(v.mean()) if v.numel() else 0.0, "abs_max": float(v.abs().max()) if v.numel() else 0.0, "zero_fraction": float((f == 0).float().mean()),
                "nan": int(torch.isnan(f).sum()), "inf": int(torch.isinf(f).sum()), "numel": g.numel()}

    def collect(self, named_parameters: Iterable, lr: float | None = None) -> dict:
        self.step_no += 1
        rows, sq = {}, 0.0
        for n, p in named_parameters:
            if p.grad is None:
                continue
            s = self.stats(n, p.grad)
            if lr is not None:
                s["update_ratio"] = lr * s["norm"] / max(float(p.detach().float().norm()), 1e-12)
            rows[n] = s; sq += s["norm"] ** 2; self.hist[n].append(s["norm"])
        self.hist["__global__"].append(math.sqrt(sq))
        return {"step": self.step_no, "global_norm": math.sqrt(sq), "parameters": rows}

    def summary(self, name: str = "__global__") -> dict:
        h = list(self.hist[name])
        return {"count": len(h), "mean": sum(h) / len(h), "max": max(h), "min": min(h), "last": h[-1]} if h else {"count": 0}


class StructuredLogger:
    """JSON-lines records with bound context (``bind`` returns a child logger) and level filtering; sinks are callables."""
    LEVELS = ("debug", "info", "warning", "error")

    def __init__(self, sink: Callable[[str], None] | None = None, level: str = "info", context: dict | None = None, clock=time.time): self.records, self.sink, self.level, self.ctx, self.clock = [], sink, level, context or {}, clock
    def bind(self, **ctx): child = StructuredLogger(self.sink, self.level, {**self.ctx, **ctx}, self.clock); child.records = self.records; return child

    def log(self, level: str, event: str, **fields):
        if self.LEVELS.index(level) < self.LEVELS.index(self.level):
            return None
        rec = {"ts": self.clock(), "level": level, "event": event, **self.ctx, **{k: (v.item() if isinstance(v, torch.Tensor) and v.numel() == 1 else list(v.shape) if isinstance(v, torch.Tensor) else v) for k, v in fields.items()}}
        self.records.append(rec)
        if self.sink:
            self.sink(json.dumps(rec, default=str))
        return rec

    def info(self, event, **f): return self.log("info", event, **f)
    def warning(self, event, **f): return self.log("warning", event, **f)
    def error(self, event, **f): return self.log("error", event, **f)
    def debug(self, event, **f): return self.log("debug", event, **f)


# ================================================================================================ exception safety and degradation
class ParameterTransaction:
    """``with ParameterTransaction(params):`` — an exception inside the block restores values and gradients exactly (strong
    guarantee); ``commit_if`` lets the caller veto on a condition (for example a non-finite loss)."""

    def __init__(self, params: Iterable[torch.Tensor], snapshot_grads: bool = True): self.params, self.grads = list(params), snapshot_grads

    def __enter__(self):
        self._vals = [p.detach().clone() for p in self.params]
        self._grads = [None if p.grad is None else p.grad.detach().clone() for p in self.params] if self.grads else None
        self.rolled_back = False
        return self

    def rollback(self):
        with torch.no_grad():
            for i, p in enumerate(self.params):
                p.copy_(self._vals[i])
                if self._grads is not None:
                    p.grad = None if self._grads[i] is None else self._grads[i].clone()
        self.rolled_back = True

    def commit_if(self, ok: bool):
        if not ok:
            self.rollback()
        return ok

    def __exit__(self, et, ev, tb):
        if et is not None:
            self.rollback()
        return False


class ResourceGuard:
    """Releases what it acquired in reverse order on exit, also when a later acquisition or the body raises."""

    def __init__(self): self._stack, self.released = [], []
    def acquire(self, name: str, make: Callable[[], Any], release: Callable[[Any], None]):
        r = make(); self._stack.append((name, r, release)); return r
    def __enter__(self): return self
    def __exit__(self, *exc):
        errors = []
        while self._stack:
            name, r, rel = self._stack.pop()
            try:
                rel(r); self.released.append(name)
            except Exception as e:                                                  # keep releasing the rest
                errors.append((name, e))
        if errors and exc[0] is None:
            raise errors[0][1]
        return False


class GracefulDegradation:
    """Ordered implementations of one operation: the first that works is used; one that raises ``NotImplementedError`` /
    ``RuntimeError`` is demoted for later calls and the decision recorded, with numeric differentiation as the last resort
    for gradients."""

    def __init__(self, name: str): self.name, self.impls, self.disabled, self.events = name, [], set(), []
    def add(self, label: str, fn: Callable, exact: bool = True): self.impls.append((label, fn, exact)); return self

    def __call__(self, *args, **kw):
        last = None
        for label, fn, exact in self.impls:
            if label in self.disabled:
                continue
            try:
                out = fn(*args, **kw)
                if not exact:
                    self.events.append({"op": self.name, "used": label, "note": "approximate fallback"})
                return out
            except (NotImplementedError, RuntimeError) as e:
                self.disabled.add(label); self.events.append({"op": self.name, "disabled": label, "reason": str(e)}); last = e
        raise RuntimeError(f"{self.name}: every implementation failed") from last


def numeric_gradient(fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, eps: float = 1e-4) -> torch.Tensor:
    x = x.detach().double()
    g = torch.zeros_like(x)
    flat, gf = x.view(-1), g.view(-1)
    for i in range(flat.numel()):
        old = float(flat[i])
        flat[i] = old + eps; hi = float(fn(x))
        flat[i] = old - eps; lo = float(fn(x))
        flat[i] = old; gf[i] = (hi - lo) / (2 * eps)
    return g


# ================================================================================================ validation, scaling, scheduling
def validate_gradients(named_parameters: Iterable, check_finite: bool = True, max_norm: float | None = None, require_all: bool = False) -> list[dict]:
    issues = []
    for n, p in named_parameters:
        g = p.grad
        if g is None:
            if require_all and p.requires_grad:
                issues.append({"parameter": n, "kind": "missing", "message": "requires a gradient but has none"})
            continue
        if g.shape != p.shape:
            issues.append({"parameter": n, "kind": "shape", "message": f"gradient {list(g.shape)} vs parameter {list(p.shape)}"})
        if g.dtype != p.dtype:
            issues.append({"parameter": n, "kind": "dtype", "message": f"gradient {g.dtype} vs parameter {p.dtype}"})
        if g.device != p.device:
            issues.append({"parameter": n, "kind": "device", "message": f"gradient on {g.device}, parameter on {p.device}"})
        if check_finite and not torch.isfinite(g).all():
            issues.append({"parameter": n, "kind": "non_finite", "message": f"{int((~torch.isfinite(g)).sum())} non-finite entries"})
        if max_norm is not None and float(g.norm()) > max_norm:
            issues.append({"parameter": n, "kind": "norm", "message": f"norm {float(g.norm()):.3g} above {max_norm:g}"})
    return issues


class OptimizerAwareGradientScaler:
    """Gradient conditioning matched to the optimizer family: plain SGD gets global-norm clipping (its step is proportional to
    the gradient), momentum SGD a tighter clip, adaptive methods only a guard against non-finite or extreme values (their
    step is already normalised), LARS / LAMB style layer-wise trust ratios when asked."""

    def __init__(self, optimizer: torch.optim.Optimizer, clip: float = 1.0, layerwise: bool = False): self.opt, self.clip, self.layerwise = optimizer, clip, layerwise

    def strategy(self) -> str:
        name = type(self.opt).__name__.lower()
        if self.layerwise:
            return "layerwise_trust"
        if name == "sgd":
            return "momentum_clip" if any(g.get("momentum", 0) for g in self.opt.param_groups) else "global_clip"
        return "guard_only" if any(k in name for k in ("adam", "rmsprop", "adagrad", "adadelta", "lamb", "lion")) else "global_clip"

    def apply(self) -> dict:
        params = [p for g in self.opt.param_groups for p in g["params"] if p.grad is not None]
        s = self.strategy()
        total = float(torch.linalg.vector_norm(torch.stack([p.grad.norm() for p in params]))) if params else 0.0
        if s in ("global_clip", "momentum_clip"):
            limit = self.clip * (0.5 if s == "momentum_clip" else 1.0)
            scale = min(1.0, limit / (total + 1e-12))
            for p in params:
                p.grad.mul_(scale)
            return {"strategy": s, "norm": total, "scale": scale}
        if s == "layerwise_trust":
            ratios = []
            for p in params:
                w, g = float(p.detach().norm()), float(p.grad.norm())
                r = w / g if w > 0 and g > 0 else 1.0
                p.grad.mul_(r); ratios.append(r)
            return {"strategy": s, "norm": total, "ratios": ratios}
        bad = sum(int((~torch.isfinite(p.grad)).sum()) for p in params)
        for p in params:
            torch.nan_to_num_(p.grad, nan=0.0, posinf=0.0, neginf=0.0)
        return {"strategy": s, "norm": total, "zeroed": bad}


class GradientScheduler:
    """Orders independent backward tasks: critical path first (longest dependent chain), then largest memory release, under a
    memory budget; returns the order and the peak it implies."""

    def __init__(self): self.tasks = {}
    def add(self, name: str, cost: float, frees: float = 0.0, allocates: float = 0.0, after: Sequence[str] = ()): self.tasks[name] = {"cost": cost, "frees": frees, "alloc": allocates, "after": list(after)}; return self

    def schedule(self, memory_budget: float | None = None, start_memory: float = 0.0) -> dict:
        users = defaultdict(list)
        for n, t in self.tasks.items():
            for d in t["after"]:
                users[d].append(n)
        cp: dict[str, float] = {}
        indeg, queue, seen_n = {n: len(t["after"]) for n, t in self.tasks.items()}, [n for n, t in self.tasks.items() if not t["after"]], 0
        while queue:
            n = queue.pop(); seen_n += 1
            for u in users[n]:
                indeg[u] -= 1
                if indeg[u] == 0:
                    queue.append(u)
        if seen_n < len(self.tasks):
            raise ValueError("dependency cycle")
        def path(n):
            if n not in cp:
                cp[n] = self.tasks[n]["cost"] + max((path(u) for u in users[n]), default=0.0)
            return cp[n]
        for n in self.tasks:
            path(n)
        done, order, mem, peak, t = set(), [], start_memory, start_memory, 0.0
        while len(done) < len(self.tasks):
            ready = [n for n in self.tasks if n not in done and all(d in done for d in self.tasks[n]["after"])]
            if not ready:
                raise ValueError("dependency cycle")
            fits = [n for n in ready if memory_budget is None or mem + self.tasks[n]["alloc"] <= memory_budget] or [min(ready, key=lambda n: self.tasks[n]["alloc"] - self.tasks[n]["frees"])]
            n = max(fits, key=lambda n: (cp[n], self.tasks[n]["frees"] - self.tasks[n]["alloc"]))
            mem += self.tasks[n]["alloc"]; peak = max(peak, mem); mem -= self.tasks[n]["frees"]; t += self.tasks[n]["cost"]
            done.add(n); order.append(n)
        return {"order": order, "peak_memory": peak, "total_cost": t, "critical_path": max(cp.values())}


# ================================================================================================ tracing and introspection
class GradientTracer:
    """Walks the autograd graph under an output: every backward node with its inputs, the leaves reached and, after
    ``backward``, the gradient norm that flowed through each node (captured with node hooks)."""

    def __init__(self, output: torch.Tensor, names: dict | None = None):
        self.output, self.nodes, self.edges, self.flow, self._hooks = output, {}, [], {}, []
        leaf_names = {id(v): k for k, v in (names or {}).items()}
        stack, seen = [output.grad_fn], set()
        while stack:
            fn = stack.pop()
            if fn is None or id(fn) in seen:
                continue
            seen.add(id(fn))
            label = type(fn).__name__
            if hasattr(fn, "variable"):
                label = "leaf:" + leaf_names.get(id(fn.variable), f"{list(fn.variable.shape)}")
            self.nodes[id(fn)] = {"fn": fn, "label": label, "leaf": hasattr(fn, "variable")}
            for nxt, _ in fn.next_functions:
                if nxt is not None:
                    self.edges.append((id(fn), id(nxt))); stack.append(nxt)

    def attach(self):
        for nid, n in self.nodes.items():
            def hook(grad_inputs, grad_outputs, nid=nid):
                g = [x for x in grad_outputs if x is not None]
                self.flow[nid] = float(torch.stack([x.detach().float().norm() for x in g]).norm()) if g else 0.0
            self._hooks.append(n["fn"].register_hook(hook))
        return self

    def detach(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def operations(self) -> Counter: return Counter(n["label"] for n in self.nodes.values() if not n["leaf"])
    def leaves(self) -> list[str]: return sorted(n["label"][5:] for n in self.nodes.values() if n["leaf"])
    def depth(self) -> int:
        children = defaultdict(list)
        for a, b in self.edges:
            children[a].append(b)
        memo = {}
        def d(n):
            if n not in memo:
                memo[n] = 1 + max((d(c) for c in children[n]), default=0)
            return memo[n]
        return d(id(self.output.grad_fn))

    def path_to(self, leaf_name: str) -> list[str]:
        """One chain of backward nodes from the output to the named leaf."""
        children = defaultdict(list)
        for a, b in self.edges:
            children[a].append(b)
        target = next(nid for nid, n in self.nodes.items() if n["label"] == "leaf:" + leaf_name)
        def walk(n, trail):
            trail = trail + [self.nodes[n]["label"]]
            if n == target:
                return trail
            for c in children[n]:
                r = walk(c, trail)
                if r:
                    return r
            return None
        return walk(id(self.output.grad_fn), [])

    def report(self) -> list[dict]: return [{"label": n["label"], "flow": self.flow.get(nid)} for nid, n in self.nodes.items()]

    def bottleneck(self) -> dict | None:
        """Node at which the flowing gradient norm drops the most relative to its parent (where the signal dies)."""
        worst = None
        for a, b in self.edges:
            fa, fb = self.flow.get(a), self.flow.get(b)
            if fa and fb is not None and fa > 0:
                r = fb / fa
                if worst is None or r < worst["ratio"]:
                    worst = {"from": self.nodes[a]["label"], "to": self.nodes[b]["label"], "ratio": r}
        return worst


def introspect_operation(fn: Callable, *inputs: torch.Tensor) -> dict:
    """What an operation does under autograd: output shape / dtype, backward node type, which inputs receive gradients, what it
    saves for backward (count and bytes), and whether it is differentiable twice."""
    saved = []
    def pack(t): saved.append(t.numel() * t.element_size()); return t
    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        out = fn(*inputs)
    info = {"output_shape": tuple(out.shape), "output_dtype": str(out.dtype), "grad_fn": type(out.grad_fn).__name__ if out.grad_fn is not None else None, "saved_tensors": len(saved), "saved_bytes": sum(saved)}
    req = [i for i in inputs if i.requires_grad]
    if out.grad_fn is not None and req:
        gs = torch.autograd.grad(out.sum(), req, create_graph=True, allow_unused=True)
        info["receives_gradient"] = [g is not None for g in gs]
        twice = False
        for g in gs:
            if g is not None and g.requires_grad:
                twice = True
        info["twice_differentiable"] = twice
    else:
        info["receives_gradient"], info["twice_differentiable"] = [], False
    return info


# ================================================================================================ buffers, chunking, tuning
def plan_buffer_reuse(lifetimes: Sequence[tuple[str, int, int, int]], alignment: int = 256) -> dict:
    """Assigns temporaries ``(name, bytes, first_use, last_use)`` to shared buffers: two temporaries may share when their
    lifetimes do not overlap.  Greedy by size (largest first, best-fitting free buffer); returns the assignment and the
    bytes saved against one buffer per temporary."""
    al = lambda b: (b + alignment - 1) // alignment * alignment
    buffers, assign = [], {}
    for name, size, a, b in sorted(lifetimes, key=lambda t: -t[1]):
        size = al(size)
        fit = [i for i, buf in enumerate(buffers) if buf["size"] >= size and all(b < s or a > e for s, e in buf["spans"])]
        if fit:
            i = min(fit, key=lambda i: buffers[i]["size"])
        else:
            buffers.append({"size": size, "spans": []}); i = len(buffers) - 1
        buffers[i]["spans"].append((a, b)); assign[name] = i
    naive = sum(al(t[1]) for t in lifetimes)
    pooled = sum(b["size"] for b in buffers)
    return {"assignment": assign, "buffers": [b["size"] for b in buffers], "bytes": pooled, "naive_bytes": naive, "saved": naive - pooled}


def chunked_gradient(fn: Callable[[torch.Tensor], torch.Tensor], params: Sequence[torch.Tensor], data: torch.Tensor, chunk: int | None = None, memory_budget: int | None = None, bytes_per_sample: int | None = None) -> tuple[torch.Tensor, list]:
    """Gradient of ``sum_i fn(data_i)`` accumulated over chunks of the batch, so the activation memory is that of one chunk.
    The chunk size comes from the budget when given (``budget // bytes_per_sample``)."""
    if chunk is None:
        chunk = max(1, (memory_budget // bytes_per_sample) if memory_budget and bytes_per_sample else len(data))
    grads, total = [torch.zeros_like(p) for p in params], 0.0
    for s in range(0, len(data), chunk):
        y = fn(data[s:s + chunk]).sum()
        for g, d in zip(grads, torch.autograd.grad(y, params)):
            g += d
        total += float(y.detach())
    return torch.tensor(total), grads


class AutoTuner:
    """Measures candidate settings of a knob on the real workload (median of a few runs each), keeps the winner per workload
    key, and re-tunes when the observed time drifts from the tuned time by more than ``drift``."""

    def __init__(self, repeats: int = 3, drift: float = 0.5, clock=time.perf_counter): self.repeats, self.drift, self.clock, self.best, self.trials = repeats, drift, clock, {}, []

    def tune(self, key, candidates: Sequence, run: Callable[[Any], Any]):
        rows = []
        for c in candidates:
            ts = []
            for _ in range(self.repeats):
                t0 = self.clock(); run(c); ts.append(self.clock() - t0)
            rows.append((sorted(ts)[len(ts) // 2], c))
        t, c = min(rows, key=lambda r: r[0])
        self.best[key] = {"choice": c, "time": t}; self.trials.append({"key": key, "rows": rows})
        return c

    def get(self, key, candidates, run):
        return self.best[key]["choice"] if key in self.best else self.tune(key, candidates, run)

    def observe(self, key, seconds: float) -> bool:
        """Returns True when the stored choice should be re-tuned."""
        b = self.best.get(key)
        if b and abs(seconds - b["time"]) > self.drift * b["time"]:
            del self.best[key]; return True
        return False


# ================================================================================================ regression baselines and stress graphs
class GradientRegressionSuite:
    """Stores gradients of named test functions at fixed inputs; a later run is compared with the stored baseline within a
    tolerance (catching silent changes in backward formulas)."""

    def __init__(self, path): self.path, self.cases = Path(path), {}
    def add_case(self, name: str, fn: Callable, inputs: Sequence[torch.Tensor]): self.cases[name] = (fn, [i.detach().clone() for i in inputs]); return self

    def _grads(self, name):
        fn, ins = self.cases[name]
        xs = [i.clone().requires_grad_(True) for i in ins]
        return [g.detach() for g in torch.autograd.grad(fn(*xs).sum(), xs)]

    def record(self): torch.save({n: self._grads(n) for n in self.cases}, self.path)

    def check(self, rtol: float = 1e-5, atol: float = 1e-7) -> dict:
        base = torch.load(self.path)
        out = {}
        for n in self.cases:
            if n not in base:
                out[n] = {"status": "new"}; continue
            cur = self._grads(n)
            err = max(float((a - b).abs().max()) for a, b in zip(cur, base[n]))
            out[n] = {"status": "ok" if all(torch.allclose(a, b, rtol=rtol, atol=atol) for a, b in zip(cur, base[n])) else "regressed", "max_abs_diff": err}
        return out


def stress_graph(kind: str, size: int, width: int = 8) -> dict:
    """Builds and differentiates a large graph: ``deep`` (a chain of ``size`` operations), ``wide`` (``size`` branches summed),
    ``shared`` (one tensor used ``size`` times) or ``diamond`` (repeated fan-out / fan-in).  Returns timings, node count and
    whether the gradient matches its closed form."""
    x = torch.full((width,), 0.5, dtype=torch.float64, requires_grad=True)
    t0 = time.perf_counter()
    if kind == "deep":
        y = x
        for _ in range(size):
            y = y * 1.0001 + 0.0
        expect = torch.full_like(x, 1.0001 ** size)
    elif kind == "wide":
        y = sum(x * float(i) for i in range(size))
        expect = torch.full_like(x, size * (size - 1) / 2)
    elif kind == "shared":
        y = torch.stack([x] * size).sum(0)
        expect = torch.full_like(x, float(size))
    elif kind == "diamond":
        y = x
        for _ in range(size):
            y = y * 0.5 + y * 0.5
        expect = torch.ones_like(x)
    else:
        raise ValueError(kind)
    n, stack, seen = 0, [y.grad_fn], {}
    while stack:                                                                    # counted before backward frees the graph
        f = stack.pop()
        if f is None or id(f) in seen:
            continue
        seen[id(f)] = f; n += 1                                                     # the wrapper is kept alive so that its id stays unique
        stack += [nf for nf, _ in f.next_functions]
    t1 = time.perf_counter()
    g, = torch.autograd.grad(y.sum(), x)
    t2 = time.perf_counter()
    return {"kind": kind, "nodes": n, "forward_s": t1 - t0, "backward_s": t2 - t1, "correct": bool(torch.allclose(g, expect, rtol=1e-9))}


# ================================================================================================ pluggable backends and compatibility layers
class AutogradBackend:
    """Interface of a differentiation engine: ``grad(fn, inputs) -> gradients``."""
    name = "abstract"
    def grad(self, fn: Callable, inputs: Sequence[torch.Tensor]) -> list[torch.Tensor]: raise NotImplementedError


class ReverseModeBackend(AutogradBackend):
    name = "reverse"
    def grad(self, fn, inputs):
        xs = [i.detach().clone().requires_grad_(True) for i in inputs]
        return list(torch.autograd.grad(fn(*xs), xs))


class ForwardModeBackend(AutogradBackend):
    """One forward pass with dual numbers per input element (cheap for few inputs and many outputs)."""
    name = "forward"
    def grad(self, fn, inputs):
        import torch.autograd.forward_ad as fwd
        out = []
        for k, x in enumerate(inputs):
            g = torch.zeros_like(x)
            for i in range(x.numel()):
                tangent = torch.zeros_like(x); tangent.view(-1)[i] = 1
                with fwd.dual_level():
                    args = [fwd.make_dual(x, tangent) if j == k else inp for j, inp in enumerate(inputs)]
                    g.view(-1)[i] = fwd.unpack_dual(fn(*args)).tangent
            out.append(g)
        return out


class FiniteDifferenceBackend(AutogradBackend):
    name = "finite_difference"
    def __init__(self, eps: float = 1e-5): self.eps = eps
    def grad(self, fn, inputs):
        out = []
        for k in range(len(inputs)):
            f = lambda v, k=k: fn(*[v.to(inputs[k].dtype) if j == k else inp for j, inp in enumerate(inputs)])
            out.append(numeric_gradient(f, inputs[k], self.eps).to(inputs[k].dtype))
        return out


class BackendRegistry:
    def __init__(self): self.backends = {b.name: b for b in (ReverseModeBackend(), ForwardModeBackend(), FiniteDifferenceBackend())}
    def register(self, backend: AutogradBackend): self.backends[backend.name] = backend
    def get(self, name: str) -> AutogradBackend: return self.backends[name]
    def cross_check(self, fn, inputs, rtol=1e-3, atol=1e-5) -> dict:
        res = {n: b.grad(fn, inputs) for n, b in self.backends.items()}
        ref = res["reverse"]
        return {n: all(torch.allclose(a.double(), b.double(), rtol=rtol, atol=atol) for a, b in zip(g, ref)) for n, g in res.items()}


class GradientTape:
    """TensorFlow-style tape: operations on watched tensors inside the block are recorded; ``gradient(target, sources)`` after
    it.  A non-persistent tape answers once."""

    def __init__(self, persistent: bool = False): self.persistent, self._watched, self._used = persistent, [], False
    def __enter__(self): return self
    def __exit__(self, *a): return False
    def watch(self, t: torch.Tensor): t.requires_grad_(True); self._watched.append(t); return t

    def gradient(self, target: torch.Tensor, sources):
        if self._used and not self.persistent:
            raise RuntimeError("a non-persistent tape can compute one set of gradients")
        self._used = True
        single = isinstance(sources, torch.Tensor)
        srcs = [sources] if single else list(sources)
        gs = torch.autograd.grad(target.sum() if target.dim() else target, srcs, retain_graph=self.persistent, allow_unused=True)
        return gs[0] if single else list(gs)


def value_and_grad(fn: Callable, argnums: int | Sequence[int] = 0) -> Callable:
    """MLX / JAX style: returns ``f(*args) -> (value, grad)`` with gradients for the selected positional arguments (pytrees of
    tensors — lists, tuples, dicts — are differentiated leaf-wise)."""
    nums = (argnums,) if isinstance(argnums, int) else tuple(argnums)
    def leaves(t): return [t] if isinstance(t, torch.Tensor) else [l for v in (t.values() if isinstance(t, dict) else t) for l in leaves(v)]
    def rebuild(t, it): return next(it) if isinstance(t, torch.Tensor) else {k: rebuild(v, it) for k, v in t.items()} if isinstance(t, dict) else type(t)(rebuild(v, it) for v in t)
    def detach(t): return t.detach().clone().requires_grad_(True) if isinstance(t, torch.Tensor) else {k: detach(v) for k, v in t.items()} if isinstance(t, dict) else type(t)(detach(v) for v in t)
    def wrapped(*args, **kw):
        args = list(args)
        for n in nums:
            args[n] = detach(args[n])
        val = fn(*args, **kw)
        flat = [l for n in nums for l in leaves(args[n])]
        gs = iter(torch.autograd.grad(val, flat, allow_unused=True))
        out = [rebuild(args[n], gs) for n in nums]
        return val.detach(), out[0] if isinstance(argnums, int) else tuple(out)
    return wrapped


class Variable:
    """Legacy PyTorch ``Variable`` spelling: ``.data``, ``.grad``, ``.backward()`` over a tensor."""

    def __init__(self, data: torch.Tensor, requires_grad: bool = False): self.tensor = data.detach().clone().requires_grad_(requires_grad)
    data = property(lambda self: self.tensor.detach())
    grad = property(lambda self: self.tensor.grad)
    def backward(self, gradient=None): self.tensor.backward(gradient)
    def __getattr__(self, k): return getattr(self.tensor, k)


class VariableEnvironment:
    """Named tensors with nested scopes: a lookup walks outward; ``gradients`` differentiates an output with respect to
    every variable visible in the current scope."""

    def __init__(self, parent: "VariableEnvironment | None" = None): self.vars, self.parent = {}, parent
    def define(self, name: str, value: torch.Tensor, requires_grad: bool = True): self.vars[name] = value.detach().clone().requires_grad_(requires_grad); return self.vars[name]
    def lookup(self, name: str) -> torch.Tensor:
        e = self
        while e is not None:
            if name in e.vars:
                return e.vars[name]
            e = e.parent
        raise KeyError(name)
    def child(self): return VariableEnvironment(self)
    def visible(self) -> dict:
        out = dict(self.parent.visible()) if self.parent else {}
        out.update(self.vars); return out
    def gradients(self, output: torch.Tensor) -> dict:
        vis = {k: v for k, v in self.visible().items() if v.requires_grad}
        gs = torch.autograd.grad(output, list(vis.values()), allow_unused=True)
        return {k: g for k, g in zip(vis, gs) if g is not None}


# ================================================================================================ fused chains and GEMM-form gradients
class FusedFunctionChain(torch.autograd.Function):
    """A chain of element-wise functions with known derivatives evaluated as one autograd node: forward saves only the input;
    backward recomputes the intermediates and multiplies the local derivatives (one saved tensor instead of one per link)."""
    TABLE = {"relu": (torch.relu, lambda x, y: (x > 0).to(x.dtype)), "tanh": (torch.tanh, lambda x, y: 1 - y * y), "sigmoid": (torch.sigmoid, lambda x, y: y * (1 - y)), "exp": (torch.exp, lambda x, y: y),
             "square": (torch.square, lambda x, y: 2 * x), "neg": (torch.neg, lambda x, y: -torch.ones_like(x)), "softplus": (torch.nn.functional.softplus, lambda x, y: torch.sigmoid(x))}

    @staticmethod
    def forward(ctx, x, names):
        ctx.names = names
        ctx.save_for_backward(x)
        for n in names:
            x = FusedFunctionChain.TABLE[n][0](x)
        return x

    @staticmethod
    def backward(ctx, grad):
        x, = ctx.saved_tensors
        d = torch.ones_like(x)
        for n in ctx.names:
            f, df = FusedFunctionChain.TABLE[n]
            y = f(x); d = d * df(x, y); x = y
        return grad * d, None


def fused_chain(x: torch.Tensor, *names: str) -> torch.Tensor: return FusedFunctionChain.apply(x, tuple(names))


def matmul_gradients(a: torch.Tensor, b: torch.Tensor, grad_out: torch.Tensor, transpose_a: bool = False, transpose_b: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Gradients of ``op(A) op(B)`` written as the two GEMM calls a BLAS would run (no transposed copies are formed: the
    transposition flags move into the operands' roles)."""
    if not transpose_a and not transpose_b:
        return grad_out @ b.mT, a.mT @ grad_out
    if transpose_a and not transpose_b:
        return b @ grad_out.mT, a @ grad_out
    if not transpose_a and transpose_b:
        return grad_out @ b, grad_out.mT @ a
    return b.mT @ grad_out.mT, grad_out.mT @ a.mT


def solve_gradients(a: torch.Tensor, x: torch.Tensor, grad_x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Gradients of ``X = A^{-1} B``: ``dB = A^{-T} dX`` (one more solve with the same factorisation) and ``dA = -dB X^T`` (one
    GEMM)."""
    gb = torch.linalg.solve(a.mT, grad_x)
    return -gb @ x.mT, gb
