"""Structural utilities for networks and functional code (``crates/torsh-nn/src``, ``crates/torsh-functional/src``):
table-driven activations with error bounds (``activation_lookup.rs``), module combinators (``composition/``,
``container/``), architecture views as Graphviz, text tree and layer table (``visualization.rs``), parameter groups with
freezing, constraints, tying and statistics (``parameter/``), argument conventions (``api_patterns.rs``), functional
profiling and implementation comparison (``profiling/``), threaded chunked execution (``parallel.rs``), a reference-checking
harness with algebraic properties (``numerical_correctness.rs``, ``pytorch_correctness.rs``, ``property_based_tests.rs``,
``testing.rs``) and module diagnostics (``diagnostics/``)."""
from __future__ import annotations

import fnmatch
import functools
import inspect
import math
import statistics
import time
from collections import OrderedDict, defaultdict
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Callable, Iterable, Sequence

import torch
from torch import nn


# ================================================================================================ table-driven activations
class LookupActivation(nn.Module):
    """Activation evaluated from a table with linear interpolation on ``[lo, hi]`` and the function's asymptotes outside (``left``
    / ``right``: ``"zero"``, ``"identity"``, ``"clamp"`` or a constant).  ``max_error()`` measures the table against the exact
    function; the backward pass uses the table's slopes, so forward and backward stay consistent."""

    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], lo: float = -8.0, hi: float = 8.0, size: int = 1024, left="clamp", right="clamp"):
        super().__init__()
        self.fn, self.lo, self.hi, self.left, self.right = fn, lo, hi, left, right
        xs = torch.linspace(lo, hi, size, dtype=torch.float64)
        self.register_buffer("table", fn(xs).float())
        self.step = (hi - lo) / (size - 1)

    @classmethod
    def gelu(cls, **kw): return cls(torch.nn.functional.gelu, left="zero", right="identity", **kw)
    @classmethod
    def sigmoid(cls, **kw): return cls(torch.sigmoid, left=0.0, right=1.0, **kw)
    @classmethod
    def tanh(cls, **kw): return cls(torch.tanh, left=-1.0, right=1.0, **{"lo": -5.0, "hi": 5.0, **kw})
    @classmethod
    def silu(cls, **kw): return cls(torch.nn.functional.silu, left="zero", right="identity", **kw)

    def _edge(self, x, mode, edge_value):
        if mode == "zero":
            return torch.zeros_like(x)
        if mode == "identity":
            return x
        if mode == "clamp":
            return torch.full_like(x, float(edge_value))
        return torch.full_like(x, float(mode))

    def forward(self, x):
        pos = ((x.float() - self.lo) / self.step).clamp(0, len(self.table) - 1)
        i = pos.floor().long().clamp(max=len(self.table) - 2)
        frac = pos - i
        y = torch.lerp(self.table[i], self.table[i + 1], frac)
        y = torch.where(x < self.lo, self._edge(x.float(), self.left, self.table[0]), y)
        y = torch.where(x > self.hi, self._edge(x.float(), self.right, self.table[-1]), y)
        return y.to(x.dtype)

    def max_error(self, samples: int = 100001, span: float = 2.0) -> float:
        xs = torch.linspace(self.lo * span, self.hi * span, samples, dtype=torch.float64)
        return float((self(xs.float()).double() - self.fn(xs)).abs().max())


# ================================================================================================ combinators
class Residual(nn.Module):
    def __init__(self, body: nn.Module, shortcut: nn.Module | None = None, scale: float = 1.0): super().__init__(); self.body, self.shortcut, self.scale = body, shortcut or nn.Identity(), scale
    def forward(self, x): return self.shortcut(x) + self.scale * self.body(x)


class Parallel(nn.Module):
    """Runs every branch on the same input and merges: ``"cat"`` (along ``dim``), ``"sum"``, ``"mean"``, ``"stack"`` or ``"tuple"``."""

    def __init__(self, *branches: nn.Module, merge: str = "cat", dim: int = 1): super().__init__(); self.branches, self.merge, self.dim = nn.ModuleList(branches), merge, dim
    def forward(self, x):
        outs = [b(x) for b in self.branches]
        if self.merge == "cat":
            return torch.cat(outs, self.dim)
        if self.merge == "stack":
            return torch.stack(outs, self.dim)
        if self.merge == "tuple":
            return tuple(outs)
        s = sum(outs)
        return s / len(outs) if self.merge == "mean" else s


class Repeat(nn.Module):
    """``n`` copies of a block built by ``factory(i)``; with ``share=True`` one block applied ``n`` times."""

    def __init__(self, factory: Callable[[int], nn.Module], n: int, share: bool = False):
        super().__init__()
        self.n, self.share = n, share
        self.blocks = nn.ModuleList([factory(0)] if share else [factory(i) for i in range(n)])
    def forward(self, x):
        for i in range(self.n):
            x = self.blocks[0 if self.share else i](x)
        return x


class Conditional(nn.Module):
    """Chooses a branch per call from a predicate on the input (``predicate(x) -> key``)."""

    def __init__(self, predicate: Callable[[torch.Tensor], Any], branches: dict[str, nn.Module]): super().__init__(); self.predicate, self.branches = predicate, nn.ModuleDict(branches)
    def forward(self, x): return self.branches[str(self.predicate(x))](x)


class Lambda(nn.Module):
    def __init__(self, fn: Callable, name: str | None = None): super().__init__(); self.fn, self.name = fn, name or getattr(fn, "__name__", "lambda")
    def forward(self, *a, **k): return self.fn(*a, **k)
    def extra_repr(self): return self.name


class SequentialBuilder:
    """Fluent construction that tracks the feature size: ``SequentialBuilder(784).linear(256).relu().dropout(0.1).linear(10).build()``."""

    def __init__(self, in_features: int): self.features, self.layers = in_features, []
    def linear(self, out: int, bias: bool = True): self.layers.append(nn.Linear(self.features, out, bias)); self.features = out; return self
    def relu(self): self.layers.append(nn.ReLU()); return self
    def gelu(self): self.layers.append(nn.GELU()); return self
    def tanh(self): self.layers.append(nn.Tanh()); return self
    def dropout(self, p: float): self.layers.append(nn.Dropout(p)); return self
    def layer_norm(self): self.layers.append(nn.LayerNorm(self.features)); return self
    def batch_norm(self): self.layers.append(nn.BatchNorm1d(self.features)); return self
    def residual(self, build: Callable[["SequentialBuilder"], "SequentialBuilder"]):
        inner = build(SequentialBuilder(self.features))
        if inner.features != self.features:
            raise ValueError(f"a residual body must keep the feature size ({self.features} -> {inner.features})")
        self.layers.append(Residual(inner.build())); return self
    def add(self, module: nn.Module, out_features: int | None = None): self.layers.append(module); self.features = out_features or self.features; return self
    def build(self) -> nn.Sequential: return nn.Sequential(*self.layers)


# ================================================================================================ architecture views
def _trace_shapes(model: nn.Module, example) -> "OrderedDict[str, dict]":
    rows, hooks = OrderedDict(), []
    for name, m in model.named_modules():
        if name == "":
            continue
        def hook(mod, inp, out, name=name):
            o = out[0] if isinstance(out, (tuple, list)) else out
            i = inp[0] if inp else None
            rows[name] = {"type": type(mod).__name__, "input": tuple(i.shape) if isinstance(i, torch.Tensor) else None, "output": tuple(o.shape) if isinstance(o, torch.Tensor) else None,
                          "params": sum(p.numel() for p in mod.parameters(recurse=False)), "leaf": not list(mod.children())}
        hooks.append(m.register_forward_hook(hook))
    was = model.training
    model.eval()
    with torch.no_grad():
        model(*example) if isinstance(example, (tuple, list)) else model(example)
    model.train(was)
    for h in hooks:
        h.remove()
    return rows


def model_tree(model: nn.Module, example=None, max_depth: int | None = None) -> str:
    """Indented tree of modules with parameter counts (and output shapes when an example input is given)."""
    shapes = _trace_shapes(model, example) if example is not None else {}
    lines = [f"{type(model).__name__} ({sum(p.numel() for p in model.parameters()):,} parameters)"]
    def walk(mod, prefix, path, depth):
        kids = list(mod.named_children())
        for k, (name, child) in enumerate(kids):
            last = k == len(kids) - 1
            full = f"{path}.{name}" if path else name
            n = sum(p.numel() for p in child.parameters())
            shp = shapes.get(full, {}).get("output")
            lines.append(f"{prefix}{'└─ ' if last else '├─ '}{name}: {type(child).__name__}" + (f" {list(shp)}" if shp else "") + (f" [{n:,}]" if n else ""))
            if max_depth is None or depth + 1 < max_depth:
                walk(child, prefix + ("   " if last else "│  "), full, depth + 1)
    walk(model, "", "", 0)
    return "\n".join(lines)


def layer_table(model: nn.Module, example) -> str:
    rows = [(n, r) for n, r in _trace_shapes(model, example).items() if r["leaf"]]
    w = max(len(n) for n, _ in rows)
    head = f"{'layer':<{w}}  {'type':<16} {'output':<20} {'params':>10}"
    body = [f"{n:<{w}}  {r['type']:<16} {str(list(r['output'])) if r['output'] else '-':<20} {r['params']:>10,}" for n, r in rows]
    return "\n".join([head, "-" * len(head), *body, "-" * len(head), f"{'total':<{w}}  {'':<16} {'':<20} {sum(r['params'] for _, r in rows):>10,}"])


def model_to_dot(model: nn.Module, example) -> str:
    """Data-flow graph from a symbolic trace when the model is traceable (true branches and merges), else the chain of leaf
    modules in execution order."""
    shapes = _trace_shapes(model, example)
    L = ["digraph model {", "  rankdir=TB; node [shape=box, fontname=Helvetica];"]
    try:
        gm = torch.fx.symbolic_trace(model)
        mods = dict(gm.named_modules())
        for n in gm.graph.nodes:
            label = n.name
            if n.op == "call_module":
                shp = shapes.get(n.target, {}).get("output")
                label = f"{n.target}\\n{type(mods[n.target]).__name__}" + (f"\\n{list(shp)}" if shp else "")
            elif n.op in ("call_function", "call_method"):
                label = getattr(n.target, "__name__", str(n.target))
            style = ", shape=ellipse" if n.op in ("placeholder", "output") else ", style=dashed" if n.op != "call_module" else ""
            L.append(f'  {n.name} [label="{label}"{style}];')
            L += [f"  {i.name} -> {n.name};" for i in n.all_input_nodes]
    except Exception:                                                              # control flow the tracer cannot follow
        prev = "input"
        L.append('  input [shape=ellipse];')
        for name, r in shapes.items():
            if r["leaf"]:
                nid = name.replace(".", "_")
                L += [f'  {nid} [label="{name}\\n{r["type"]}\\n{list(r["output"]) if r["output"] else ""}"];', f"  {prev} -> {nid};"]
                prev = nid
    L.append("}")
    return "\n".join(L) + "\n"


# ================================================================================================ parameter management
class ParameterManager:
    """Named groups chosen by glob patterns over parameter names, with per-group options for an optimizer, freezing, value
    constraints applied after each step, tying, and statistics."""

    def __init__(self, model: nn.Module): self.model, self.groups, self.constraints = model, OrderedDict(), []

    def select(self, *patterns: str) -> list[tuple[str, nn.Parameter]]: return [(n, p) for n, p in self.model.named_parameters() if any(fnmatch.fnmatch(n, pat) for pat in patterns)]
    def group(self, name: str, *patterns: str, **options): self.groups[name] = (patterns, options); return self

    def optimizer_groups(self, **defaults) -> list[dict]:
        """One dict per group plus a final one with every parameter no pattern claimed; a parameter goes to the first group that
        matches it."""
        taken, out = set(), []
        for gname, (patterns, opts) in self.groups.items():
            ps = [p for n, p in self.select(*patterns) if id(p) not in taken and p.requires_grad]
            taken.update(id(p) for p in ps)
            if ps:
                out.append({"name": gname, "params": ps, **defaults, **opts})
        rest = [p for p in self.model.parameters() if id(p) not in taken and p.requires_grad]
        if rest:
            out.append({"name": "default", "params": rest, **defaults})
        return out

    def freeze(self, *patterns: str) -> int:
        sel = self.select(*patterns)
        for _, p in sel:
            p.requires_grad_(False)
        return len(sel)

    def unfreeze(self, *patterns: str) -> int:
        sel = self.select(*patterns)
        for _, p in sel:
            p.requires_grad_(True)
        return len(sel)

    def constrain(self, kind: str, *patterns: str, value: float = 1.0):
        """``non_negative``, ``unit_norm`` (rows), ``max_norm`` (rows, ``value``), ``clip`` (``[-value, value]``)."""
        self.constraints.append((kind, patterns, value)); return self

    @torch.no_grad()
    def apply_constraints(self):
        for kind, patterns, value in self.constraints:
            for _, p in self.select(*patterns):
                if kind == "non_negative":
                    p.clamp_(min=0)
                elif kind == "clip":
                    p.clamp_(-value, value)
                elif kind in ("unit_norm", "max_norm"):
                    rows = p.view(p.shape[0], -1)
                    n = rows.norm(dim=1, keepdim=True).clamp_min(1e-12)
                    rows.mul_(1 / n if kind == "unit_norm" else (value / n).clamp(max=1.0))
                else:
                    raise ValueError(kind)

    def tie(self, source: str, target: str):
        """Makes ``target`` the same ``Parameter`` object as ``source``."""
        src = dict(self.model.named_parameters())[source]
        mod_path, _, attr = target.rpartition(".")
        mod = self.model.get_submodule(mod_path) if mod_path else self.model
        if getattr(mod, attr).shape != src.shape:
            raise ValueError(f"cannot tie {target} {tuple(getattr(mod, attr).shape)} to {source} {tuple(src.shape)}")
        setattr(mod, attr, src)

    def statistics(self) -> dict:
        rows = {}
        for n, p in self.model.named_parameters():
            d = p.detach().float()
            rows[n] = {"shape": tuple(p.shape), "numel": p.numel(), "mean": float(d.mean()), "std": float(d.std()) if p.numel() > 1 else 0.0, "abs_max": float(d.abs().max()), "zero_fraction": float((d == 0).float().mean()),
                       "trainable": p.requires_grad, "grad_norm": float(p.grad.norm()) if p.grad is not None else None}
        total = sum(r["numel"] for r in rows.values())
        return {"parameters": rows, "total": total, "trainable": sum(r["numel"] for r in rows.values() if r["trainable"]), "frozen": sum(r["numel"] for r in rows.values() if not r["trainable"])}


# ================================================================================================ argument conventions
def validated(**rules):
    """Checks named arguments before the call: ``positive``, ``non_negative``, ``probability``, ``("choice", [...])``, ``("ndim", k)``
    / ``("ndim", (lo, hi))``, ``"floating"``.  Errors name the function and the argument."""
    def deco(fn):
        sig = inspect.signature(fn)
        @functools.wraps(fn)
        def wrapper(*a, **k):
            bound = sig.bind(*a, **k); bound.apply_defaults()
            for arg, rule in rules.items():
                v = bound.arguments[arg]
                kind, param = (rule, None) if isinstance(rule, str) else rule
                bad = None
                if kind == "positive" and not v > 0:
                    bad = "must be positive"
                elif kind == "non_negative" and not v >= 0:
                    bad = "must be non-negative"
                elif kind == "probability" and not 0 <= v <= 1:
                    bad = "must be in [0, 1]"
                elif kind == "choice" and v not in param:
                    bad = f"must be one of {list(param)}"
                elif kind == "ndim" and not ((v.dim() == param) if isinstance(param, int) else (param[0] <= v.dim() <= param[1])):
                    bad = f"must have {param} dimensions, got {v.dim()}"
                elif kind == "floating" and not v.is_floating_point():
                    bad = f"must be a floating-point tensor, got {v.dtype}"
                if bad:
                    raise ValueError(f"{fn.__name__}: argument {arg!r} {bad} (got {v if not isinstance(v, torch.Tensor) else tuple(v.shape)})")
            return fn(*a, **k)
        return wrapper
    return deco


def apply_reduction(values: torch.Tensor, reduction: str = "mean", weights: torch.Tensor | None = None) -> torch.Tensor:
    """The one reduction convention of loss-like functions: ``none``, ``sum``, ``mean`` (weighted mean when weights are given)."""
    if weights is not None:
        values = values * weights
    if reduction == "none":
        return values
    if reduction == "sum":
        return values.sum()
    if reduction == "mean":
        return values.sum() / (weights.sum() if weights is not None else values.numel())
    raise ValueError(f"reduction must be 'none', 'sum' or 'mean', got {reduction!r}")


# ================================================================================================ functional profiling
def profile_function(fn: Callable, *inputs, iterations: int = 10, warmup: int = 2, flops: float | None = None) -> dict:
    """Median time, bytes allocated for outputs, and achieved rates when the operation's FLOPs are supplied; device work is
    timed with events."""
    from ..utils.bench_suite import Timer
    dev = next((i.device.type for i in inputs if isinstance(i, torch.Tensor)), "cpu")
    t = Timer(dev)
    for _ in range(warmup):
        out = fn(*inputs)
    ts = sorted(t.measure(lambda: fn(*inputs)) for _ in range(iterations))
    outs = out if isinstance(out, (tuple, list)) else [out]
    in_b = sum(i.numel() * i.element_size() for i in inputs if isinstance(i, torch.Tensor))
    out_b = sum(o.numel() * o.element_size() for o in outs if isinstance(o, torch.Tensor))
    med = ts[len(ts) // 2]
    return {"median_s": med, "min_s": ts[0], "max_s": ts[-1], "input_bytes": in_b, "output_bytes": out_b, "gbps": (in_b + out_b) / med / 1e9, "gflops": flops / med / 1e9 if flops else None}


def compare_implementations(impls: dict[str, Callable], *inputs, reference: str | None = None, rtol: float = 1e-4, atol: float = 1e-6, **kw) -> dict:
    ref_name = reference or next(iter(impls))
    ref = impls[ref_name](*inputs)
    rows = {}
    for name, f in impls.items():
        p = profile_function(f, *inputs, **kw)
        out = f(*inputs)
        rows[name] = {**p, "matches": bool(torch.allclose(out.double(), ref.double(), rtol=rtol, atol=atol)), "max_abs_diff": float((out.double() - ref.double()).abs().max())}
    base = rows[ref_name]["median_s"]
    for r in rows.values():
        r["speedup"] = base / r["median_s"]
    return {"reference": ref_name, "fastest": min((n for n in rows if rows[n]["matches"]), key=lambda n: rows[n]["median_s"]), "rows": rows}


# ================================================================================================ threaded chunked execution
def parallel_chunks(fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, threads: int = 4, dim: int = 0, min_chunk: int = 1024) -> torch.Tensor:
    """Applies ``fn`` to slices of ``x`` along ``dim`` on a thread pool (tensor kernels release the interpreter lock) and
    concatenates; small inputs run inline.  Each worker uses one intra-op thread so that the pool does not oversubscribe."""
    n = x.shape[dim]
    if threads <= 1 or n < 2 * min_chunk:
        return fn(x)
    parts = x.tensor_split(min(threads, n // min_chunk), dim)
    def work(p):
        return fn(p)
    with ThreadPoolExecutor(len(parts)) as ex:
        return torch.cat(list(ex.map(work, parts)), dim)


def parallel_reduce(fn: Callable[[torch.Tensor], torch.Tensor], combine: Callable, x: torch.Tensor, threads: int = 4, dim: int = 0) -> torch.Tensor:
    parts = x.tensor_split(max(1, min(threads, x.shape[dim])), dim)
    with ThreadPoolExecutor(len(parts)) as ex:
        return functools.reduce(combine, ex.map(fn, parts))


# ================================================================================================ reference-checking harness
DEFAULT_TOLERANCES = {torch.float64: (1e-10, 1e-12), torch.float32: (1e-4, 1e-6), torch.bfloat16: (3e-2, 1e-2), torch.float16: (5e-3, 1e-3)}


def check_against_reference(fn: Callable, reference: Callable, make_inputs: Callable[[torch.dtype, torch.Generator], Sequence[torch.Tensor]], dtypes=(torch.float64, torch.float32, torch.bfloat16), trials: int = 3,
                            tolerances: dict | None = None, check_grad: bool = False, seed: int = 0) -> dict:
    """Runs ``fn`` in each dtype against ``reference`` evaluated in float64 on the same (rounded) inputs.  With ``check_grad`` the
    input gradients of ``sum(output)`` are compared too."""
    tol, report = {**DEFAULT_TOLERANCES, **(tolerances or {})}, {}
    g = torch.Generator().manual_seed(seed)
    for dt in dtypes:
        worst, worst_g, ok = 0.0, 0.0, True
        for _ in range(trials):
            ins = [i.to(dt) if i.is_floating_point() else i for i in make_inputs(dt, g)]
            ref_in = [i.double().requires_grad_(check_grad) if i.is_floating_point() else i for i in ins]
            ref = reference(*ref_in)
            test_in = [i.clone().requires_grad_(check_grad) if i.is_floating_point() else i for i in ins]
            out = fn(*test_in)
            rt, at = tol[dt]
            worst = max(worst, float((out.detach().double() - ref.detach()).abs().max()))
            ok &= bool(torch.allclose(out.double(), ref.detach(), rtol=rt, atol=at, equal_nan=True)) and out.dtype == dt
            if check_grad:
                gr = torch.autograd.grad(ref.sum(), [i for i in ref_in if i.is_floating_point()])
                gt = torch.autograd.grad(out.float().sum(), [i for i in test_in if i.is_floating_point()])
                for a, b in zip(gt, gr):
                    worst_g = max(worst_g, float((a.double() - b).abs().max()))
                    ok &= bool(torch.allclose(a.double(), b, rtol=10 * rt, atol=10 * at))
        report[str(dt).replace("torch.", "")] = {"passed": ok, "max_abs_error": worst, **({"max_grad_error": worst_g} if check_grad else {})}
    report["passed"] = all(v["passed"] for v in report.values())
    return report


def check_properties(fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, properties: Sequence[str], atol: float = 1e-5, dim: int = -1) -> dict:
    """Algebraic properties on a sample: ``idempotent``, ``odd``, ``even``, ``monotone``, ``linear``, ``positive_homogeneous``,
    ``shift_invariant`` (along ``dim``), ``permutation_equivariant`` (along ``dim``), ``bounded01``, ``sums_to_one`` (along ``dim``),
    ``non_negative``."""
    y, out = fn(x), {}
    close = lambda a, b: bool(torch.allclose(a, b, atol=atol, rtol=1e-4))
    for p in properties:
        if p == "idempotent":
            out[p] = close(fn(y), y)
        elif p == "odd":
            out[p] = close(fn(-x), -y)
        elif p == "even":
            out[p] = close(fn(-x), y)
        elif p == "monotone":
            s = x.flatten().sort().values
            out[p] = bool((fn(s).diff() >= -atol).all())
        elif p == "linear":
            z = torch.randn_like(x)
            out[p] = close(fn(2.0 * x + z), 2.0 * y + fn(z))
        elif p == "positive_homogeneous":
            out[p] = close(fn(3.0 * x), 3.0 * y)
        elif p == "shift_invariant":
            out[p] = close(fn(x + 5.0), y)
        elif p == "permutation_equivariant":
            perm = torch.randperm(x.shape[dim])
            out[p] = close(fn(x.index_select(dim, perm)), y.index_select(dim, perm))
        elif p == "bounded01":
            out[p] = bool((y >= -atol).all() and (y <= 1 + atol).all())
        elif p == "sums_to_one":
            out[p] = close(y.sum(dim), torch.ones_like(y.sum(dim)))
        elif p == "non_negative":
            out[p] = bool((y >= -atol).all())
        else:
            raise ValueError(p)
    return out


# ================================================================================================ diagnostics
def diagnose_module(model: nn.Module, example: torch.Tensor, loss_fn: Callable[[torch.Tensor], torch.Tensor] | None = None) -> dict:
    """One forward / backward pass with checks: non-finite activations, dead rectifiers (always zero), saturated sigmoid /
    tanh units, parameters that receive no gradient, and layers whose gradient norm is vanishing or exploding relative to
    the median."""
    acts, hooks, issues = {}, [], []
    for name, m in model.named_modules():
        if not list(m.children()) and name:
            hooks.append(m.register_forward_hook(lambda mod, i, o, name=name: acts.__setitem__(name, (mod, o.detach())) if isinstance(o, torch.Tensor) else None))
    model.zero_grad()
    out = model(example)
    (loss_fn(out) if loss_fn else out.float().pow(2).mean()).backward()
    for h in hooks:
        h.remove()
    for name, (mod, a) in acts.items():
        if not torch.isfinite(a).all():
            issues.append({"layer": name, "kind": "non_finite_activation"})
        if isinstance(mod, (nn.ReLU, nn.ReLU6)) and a.dim() >= 2:
            dead = float((a.transpose(0, 1).flatten(1) == 0).all(1).float().mean())
            if dead > 0.5:
                issues.append({"layer": name, "kind": "dead_units", "fraction": dead})
        if isinstance(mod, (nn.Sigmoid, nn.Tanh)):
            sat = float(((a.abs() > 0.99) if isinstance(mod, nn.Tanh) else ((a < 0.01) | (a > 0.99))).float().mean())
            if sat > 0.5:
                issues.append({"layer": name, "kind": "saturated", "fraction": sat})
    norms = {n: float(p.grad.norm()) for n, p in model.named_parameters() if p.grad is not None and p.dim() > 1}
    for n, p in model.named_parameters():
        if p.requires_grad and (p.grad is None or float(p.grad.abs().sum()) == 0.0):
            issues.append({"parameter": n, "kind": "no_gradient"})
    if norms:
        med = statistics.median(norms.values()) or 1e-30
        for n, v in norms.items():
            if v > 0 and (v / med > 1e3 or v / med < 1e-3):
                issues.append({"parameter": n, "kind": "exploding_gradient" if v > med else "vanishing_gradient", "ratio": v / med})
    return {"issues": issues, "gradient_norms": norms, "healthy": not issues}
