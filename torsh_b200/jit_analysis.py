"""Compiler analyses and research passes (``crates/torsh-jit/src``): interval abstract interpretation
(``abstract_interpretation/``), path-exploring symbolic execution (``symbolic_execution.rs``), partial evaluation
(``partial_evaluation.rs``), generic functions with monomorphisation (``generics.rs``, ``specialization.rs``), code templates
and loop unrolling (``metaprogramming.rs``), an optimisation advisor (``advisor/``), profile-guided optimisation
(``pgo.rs``), loop-nest dependence analysis with interchange and tiling (``polyhedral_optimization.rs``), cost under
uncertain shapes (``probabilistic_compilation.rs``), enumerative synthesis from examples (``program_synthesis.rs``),
guarded speculation with deoptimisation (``speculative_optimization.rs``), gradient-based variant selection
(``differentiable_compilation.rs``), a learned cost model (``neural_compilation.rs``), debug symbols
(``debug_symbols.rs``), hardware tuning tables for the B200 (``hardware_tuning.rs``) and LLVM IR text for fused
element-wise loops (``llvm_backend.rs``)."""
from __future__ import annotations

import inspect
import itertools
import json
import math
import operator
import re
import string
import time
from collections import Counter, defaultdict
from dataclasses import dataclass, field
from typing import Any, Callable, Sequence

import torch
import torch.fx


# ================================================================================================ abstract interpretation
@dataclass(frozen=True)
class Interval:
    lo: float
    hi: float

    @staticmethod
    def of(v): return v if isinstance(v, Interval) else Interval(float(v), float(v))
    def __add__(self, o): o = Interval.of(o); return Interval(self.lo + o.lo, self.hi + o.hi)
    __radd__ = __add__
    def __neg__(self): return Interval(-self.hi, -self.lo)
    def __sub__(self, o): return self + (-Interval.of(o))
    def __rsub__(self, o): return Interval.of(o) - self
    def __mul__(self, o):
        o = Interval.of(o)
        p = [a * b if not (a == 0 or b == 0) else 0.0 for a in (self.lo, self.hi) for b in (o.lo, o.hi)]
        return Interval(min(p), max(p))
    __rmul__ = __mul__
    def __truediv__(self, o):
        o = Interval.of(o)
        if o.contains(0):
            return Interval(-math.inf, math.inf)
        return self * Interval(1 / o.hi, 1 / o.lo)
    def contains(self, v) -> bool: return self.lo <= v <= self.hi
    def join(self, o): return Interval(min(self.lo, o.lo), max(self.hi, o.hi))
    def meet(self, o): return Interval(max(self.lo, o.lo), min(self.hi, o.hi))
    def is_empty(self): return self.lo > self.hi
    def monotone(self, f): return Interval(f(self.lo), f(self.hi))
    def sign(self) -> str: return "zero" if self.lo == self.hi == 0 else "positive" if self.lo > 0 else "non-negative" if self.lo >= 0 else "negative" if self.hi < 0 else "non-positive" if self.hi <= 0 else "unknown"
    def widen(self, o): return Interval(self.lo if o.lo >= self.lo else -math.inf, self.hi if o.hi <= self.hi else math.inf)


def _safe_exp(v): return math.exp(v) if v < 700 else math.inf
def _sigmoid(v): return 1 / (1 + math.exp(-v)) if v > -700 else 0.0


class AbstractInterpreter:
    """Propagates one interval per tensor (a bound on every element) through a traced graph and reports operations whose
    inputs may be outside their domain."""

    def __init__(self, gm: torch.fx.GraphModule): self.gm, self.mods, self.warnings = gm, dict(gm.named_modules()), []

    def run(self, *inputs: Interval) -> dict[str, Interval]:
        env, it = {}, iter(inputs)
        val = lambda a: env[a.name] if isinstance(a, torch.fx.Node) else Interval.of(a)
        for n in self.gm.graph.nodes:
            if n.op == "placeholder":
                env[n.name] = next(it)
            elif n.op == "output":
                self.output = val(n.args[0]) if isinstance(n.args[0], torch.fx.Node) else None
            elif n.op == "get_attr":
                t = self._attr(n.target)
                env[n.name] = Interval(float(t.min()), float(t.max()))
            else:
                env[n.name] = self._transfer(n, val)
        return env

    def _attr(self, target):
        o = self.gm
        for p in target.split("."):
            o = getattr(o, p)
        return o

    def _transfer(self, n, val) -> Interval:
        if n.op == "call_module":
            m = self.mods[n.target]
            x = val(n.args[0])
            if isinstance(m, torch.nn.Linear):
                w = m.weight.detach().double()
                lo = (w.clamp(min=0) * x.lo + w.clamp(max=0) * x.hi).sum(1)
                hi = (w.clamp(min=0) * x.hi + w.clamp(max=0) * x.lo).sum(1)
                if m.bias is not None:
                    lo, hi = lo + m.bias.detach().double(), hi + m.bias.detach().double()
                return Interval(float(lo.min()), float(hi.max()))
            name = type(m).__name__.lower()
            if isinstance(m, torch.nn.Dropout) or isinstance(m, torch.nn.Identity):
                return x if not isinstance(m, torch.nn.Dropout) or not m.training else x.join(x * (1 / (1 - m.p))).join(Interval(0, 0))
            if isinstance(m, torch.nn.Softmax):
                return Interval(0.0, 1.0)
            if isinstance(m, torch.nn.LayerNorm) and not m.elementwise_affine:
                d = math.prod(m.normalized_shape)
                return Interval(-math.sqrt(d - 1), math.sqrt(d - 1))
            return self._unary(name, x, n)
        name = getattr(n.target, "__name__", str(n.target)) if n.op == "call_function" else n.target
        name = name.rstrip("_") if name not in ("__",) else name
        a = [val(x) for x in n.args if isinstance(x, (torch.fx.Node, int, float))]
        if name in ("add",):
            return a[0] + a[1]
        if name in ("sub",):
            return a[0] - a[1]
        if name in ("mul",):
            return a[0] * a[1] if n.args[0] is not n.args[1] else self._unary("square", a[0], n)
        if name in ("truediv", "div"):
            if a[1].contains(0):
                self.warnings.append({"node": n.name, "kind": "division_by_zero", "message": f"denominator range [{a[1].lo:g}, {a[1].hi:g}] contains zero"})
            return a[0] / a[1]
        if name == "neg":
            return -a[0]
        if name in ("clamp", "clip"):
            lo, hi = n.kwargs.get("min", n.args[1] if len(n.args) > 1 else None), n.kwargs.get("max", n.args[2] if len(n.args) > 2 else None)
            return Interval(max(a[0].lo, lo) if lo is not None else a[0].lo, min(a[0].hi, hi) if hi is not None else a[0].hi)
        if name in ("maximum", "max") and len(a) == 2:
            return Interval(max(a[0].lo, a[1].lo), max(a[0].hi, a[1].hi))
        if name in ("minimum", "min") and len(a) == 2:
            return Interval(min(a[0].lo, a[1].lo), min(a[0].hi, a[1].hi))
        if name == "softmax":
            return Interval(0.0, 1.0)
        return self._unary(name, a[0], n)

    def _unary(self, name, x: Interval, n) -> Interval:
        if name == "relu":
            return Interval(max(x.lo, 0.0), max(x.hi, 0.0))
        if name == "sigmoid":
            return x.monotone(_sigmoid)
        if name == "tanh":
            return x.monotone(math.tanh)
        if name == "exp":
            if x.hi > 88.7:
                self.warnings.append({"node": n.name, "kind": "overflow", "message": f"exp of values up to {x.hi:g} overflows float32"})
            return x.monotone(_safe_exp)
        if name in ("log", "sqrt", "rsqrt"):
            if x.lo < 0 or (name != "sqrt" and x.lo <= 0):
                self.warnings.append({"node": n.name, "kind": "domain", "message": f"{name} of range [{x.lo:g}, {x.hi:g}]"})
            c = Interval(max(x.lo, 0.0), max(x.hi, 0.0))
            if name == "sqrt":
                return c.monotone(math.sqrt)
            if name == "log":
                return Interval(math.log(c.lo) if c.lo > 0 else -math.inf, math.log(c.hi) if c.hi > 0 else -math.inf)
            return Interval(1 / math.sqrt(c.hi) if c.hi > 0 else math.inf, 1 / math.sqrt(c.lo) if c.lo > 0 else math.inf)
        if name == "abs":
            return Interval(0.0 if x.contains(0) else min(abs(x.lo), abs(x.hi)), max(abs(x.lo), abs(x.hi)))
        if name == "square":
            a = self._unary("abs", x, n)
            return Interval(a.lo ** 2, a.hi ** 2)
        if name in ("gelu", "silu"):
            return Interval(min(-0.28 if x.lo < 0 else 0.0, 0.0) if x.lo < 0 else (x.lo * _sigmoid(x.lo) if name == "silu" else 0.5 * x.lo * (1 + math.erf(x.lo / math.sqrt(2)))), max(x.hi, 0.0))
        if name in ("leakyrelu", "leaky_relu"):
            return Interval(min(x.lo, 0.01 * x.lo), max(x.hi, 0.01 * x.hi))
        if name in ("flatten", "reshape", "view", "contiguous", "transpose", "permute", "squeeze", "unsqueeze", "identity", "detach", "clone", "t", "float", "to"):
            return x
        if name in ("sin", "cos"):
            return Interval(-1.0, 1.0)
        return Interval(-math.inf, math.inf)


# ================================================================================================ symbolic execution
class Sym:
    """Expression over named scalar inputs; arithmetic builds a tree, comparisons ask the running executor which branch
    to take."""
    _exec: "SymbolicExecutor | None" = None

    def __init__(self, expr: str, fn: Callable[[dict], float]): self.expr, self.fn = expr, fn
    @staticmethod
    def lift(v): return v if isinstance(v, Sym) else Sym(repr(v), lambda env, v=v: v)

    def _bin(self, o, sym, f, rev=False):
        o = Sym.lift(o); a, b = (o, self) if rev else (self, o)
        return Sym(f"({a.expr} {sym} {b.expr})", lambda env: f(a.fn(env), b.fn(env)))
    def __add__(self, o): return self._bin(o, "+", operator.add)
    def __radd__(self, o): return self._bin(o, "+", operator.add, True)
    def __sub__(self, o): return self._bin(o, "-", operator.sub)
    def __rsub__(self, o): return self._bin(o, "-", operator.sub, True)
    def __mul__(self, o): return self._bin(o, "*", operator.mul)
    def __rmul__(self, o): return self._bin(o, "*", operator.mul, True)
    def __truediv__(self, o): return self._bin(o, "/", lambda a, b: a / b if b else math.inf)
    def __neg__(self): return Sym(f"(-{self.expr})", lambda env: -self.fn(env))
    def _cmp(self, o, sym, f):
        o = Sym.lift(o)
        return SymBool(f"{self.expr} {sym} {o.expr}", lambda env: f(self.fn(env), o.fn(env)), [c for c in (self._const(), o._const()) if c is not None])
    def _const(self):
        try:
            return float(self.expr)
        except ValueError:
            return None
    def __lt__(self, o): return self._cmp(o, "<", operator.lt)
    def __le__(self, o): return self._cmp(o, "<=", operator.le)
    def __gt__(self, o): return self._cmp(o, ">", operator.gt)
    def __ge__(self, o): return self._cmp(o, ">=", operator.ge)
    def __eq__(self, o): return self._cmp(o, "==", operator.eq)                       # noqa: D105
    def __ne__(self, o): return self._cmp(o, "!=", operator.ne)
    __hash__ = None


class SymBool:
    def __init__(self, expr, fn, consts=()): self.expr, self.fn, self.consts = expr, fn, list(consts)
    def __bool__(self): return Sym._exec._decide(self)
    def negate(self): return SymBool(f"not ({self.expr})", lambda env: not self.fn(env), self.consts)


@dataclass
class SymPath:
    conditions: list
    result: Any
    witness: dict | None
    error: str | None = None

    @property
    def feasible(self): return self.witness is not None


class SymbolicExecutor:
    """Runs a Python function on symbolic scalars once per path: every ``if`` on a symbolic comparison is explored both
    ways (depth-first, by re-execution with a prefix of forced decisions).  A path is feasible when a witness satisfying all
    its conditions is found among values derived from the constants the conditions mention."""

    def __init__(self, max_paths: int = 64, domain: tuple[float, float] = (-100.0, 100.0)): self.max_paths, self.domain = max_paths, domain

    def _decide(self, cond: SymBool) -> bool:
        i = len(self._taken)
        choice = self._forced[i] if i < len(self._forced) else True
        self._taken.append((cond, choice))
        return choice

    def explore(self, fn: Callable, names: Sequence[str] | None = None) -> list[SymPath]:
        names = list(names or inspect.signature(fn).parameters)
        work, paths = [[]], []
        while work and len(paths) < self.max_paths:
            self._forced, self._taken = work.pop(), []
            Sym._exec = self
            err = res = None
            try:
                res = fn(*[Sym(n, lambda env, n=n: env[n]) for n in names])
            except Exception as e:                                               # the path itself raises: that is a finding
                err = f"{type(e).__name__}: {e}"
            finally:
                Sym._exec = None
            conds = [c if ch else c.negate() for c, ch in self._taken]
            for j in range(len(self._forced), len(self._taken)):
                work.append([ch for _, ch in self._taken[:j]] + [False])
            paths.append(SymPath([c.expr for c in conds], res.expr if isinstance(res, Sym) else res, self._solve(conds, names), err))
        return paths

    def _solve(self, conds, names):
        pts = {0.0, 1.0, -1.0, *self.domain}
        for c in conds:
            for k in c.consts:
                pts |= {k, k + 1, k - 1, k + 0.5, k - 0.5, 2 * k, k / 2}
        pts = sorted(p for p in pts if self.domain[0] <= p <= self.domain[1])
        for combo in itertools.islice(itertools.product(pts, repeat=len(names)), 200000):
            env = dict(zip(names, combo))
            try:
                if all(c.fn(env) for c in conds):
                    return env
            except (ZeroDivisionError, OverflowError):
                continue
        return None


# ================================================================================================ partial evaluation
def partial_evaluate(fn: Callable, **static) -> tuple[torch.fx.GraphModule, dict]:
    """Specialises ``fn`` on known arguments: Python control flow on them disappears at trace time, then constants fold and
    dead code is removed.  Returns the residual program and what was removed."""
    from . import fx as tfx
    gm = torch.fx.symbolic_trace(fn, concrete_args=static)
    before = len(list(gm.graph.nodes))
    folded, dead = tfx.constant_folding(gm), tfx.dead_code_elimination(gm)
    gm.recompile()
    return gm, {"nodes_before": before, "nodes_after": len(list(gm.graph.nodes)), "folded": folded, "dead": dead, "static": sorted(static)}


# ================================================================================================ generics
class GenericFunction:
    """``@generic(T=(torch.float32, torch.bfloat16))``: the body is instantiated once per binding of its type parameters (from
    the argument dtypes) and cached; bindings outside the constraint are rejected."""

    def __init__(self, fn, constraints: dict): self.fn, self.constraints, self.instances, self.params = fn, constraints, {}, [p for p, a in fn.__annotations__.items() if a in constraints]

    def bind(self, *args, **kw):
        bound = inspect.signature(self.fn).bind(*args, **kw).arguments
        binding = {}
        for p in self.params:
            tv, dt = self.fn.__annotations__[p], bound[p].dtype
            if binding.setdefault(tv, dt) != dt:
                raise TypeError(f"type parameter {tv} bound to both {binding[tv]} and {dt}")
            if dt not in self.constraints[tv]:
                raise TypeError(f"{dt} does not satisfy the constraint on {tv}: {self.constraints[tv]}")
        return tuple(sorted(binding.items(), key=lambda kv: kv[0]))

    def __call__(self, *args, **kw):
        key = self.bind(*args, **kw)
        if key not in self.instances:
            types = dict(key)
            def inst(*a, __types=types, **k): return self.fn(*a, **k, **({"types": __types} if "types" in inspect.signature(self.fn).parameters else {}))
            inst.__name__ = self.fn.__name__ + "<" + ", ".join(str(v).replace("torch.", "") for _, v in key) + ">"
            self.instances[key] = inst
        return self.instances[key](*args, **kw)

    def instantiations(self): return [f.__name__ for f in self.instances.values()]


def generic(**constraints): return lambda fn: GenericFunction(fn, constraints)


# ================================================================================================ metaprogramming
class CodeTemplate:
    """``string.Template`` source turned into a function; generated sources are kept for inspection."""

    def __init__(self, source: str, name: str): self.t, self.name, self.generated = string.Template(source), name, {}

    def instantiate(self, **subs) -> Callable:
        src = self.t.substitute(**subs)
        if src not in self.generated:
            ns: dict = {"torch": torch, "math": math}
            exec(compile(src, f"<template {self.name}>", "exec"), ns)             # noqa: S102 - the source is the caller's own template
            self.generated[src] = ns[self.name]
        return self.generated[src]


def unroll_loop(body: str, var: str, count: int, name: str = "unrolled", args: str = "x") -> tuple[Callable, str]:
    """Function whose body is ``body`` repeated for ``var = 0 .. count - 1`` with the index substituted as a literal."""
    lines = [f"def {name}({args}):"] + [f"    {re.sub(rf'\b{var}\b', str(i), body)}" for i in range(count)] + [f"    return {args.split(',')[0].strip()}"]
    src = "\n".join(lines)
    ns: dict = {"torch": torch, "math": math}
    exec(compile(src, f"<unrolled {name}>", "exec"), ns)                           # noqa: S102
    return ns[name], src


def reflect(gm: torch.fx.GraphModule) -> dict:
    ops = Counter((n.op, getattr(n.target, "__name__", str(n.target)) if n.op != "call_module" else type(dict(gm.named_modules())[n.target]).__name__) for n in gm.graph.nodes)
    return {"inputs": [n.name for n in gm.graph.nodes if n.op == "placeholder"], "operations": {f"{k[0]}:{k[1]}": v for k, v in ops.items() if k[0] not in ("placeholder", "output")},
            "parameters": {k: tuple(v.shape) for k, v in gm.named_parameters()}, "depth": _graph_depth(gm)}


def _graph_depth(gm):
    d = {}
    for n in gm.graph.nodes:
        d[n] = 1 + max((d[i] for i in n.all_input_nodes), default=0)
    return max(d.values(), default=0)


# ================================================================================================ advisor
_EW = {"add", "sub", "mul", "truediv", "relu", "gelu", "tanh", "sigmoid", "exp", "neg", "silu", "ReLU", "GELU", "Tanh", "Sigmoid", "SiLU", "Dropout"}


class OptimizationAdvisor:
    """Reads a traced graph (and optionally per-node timings) and lists what would make it faster, largest estimated gain
    first."""

    def __init__(self, gm: torch.fx.GraphModule, node_times: dict[str, float] | None = None): self.gm, self.mods, self.times = gm, dict(gm.named_modules()), node_times or {}

    def _kind(self, n):
        if n.op == "call_module":
            return type(self.mods[n.target]).__name__
        return getattr(n.target, "__name__", str(n.target)) if n.op in ("call_function", "call_method") else n.op

    def advise(self) -> list[dict]:
        recs, nodes = [], list(self.gm.graph.nodes)
        total = sum(self.times.values()) or None
        share = lambda names: sum(self.times.get(x, 0.0) for x in names) / total if total else None
        # element-wise chains
        seen = set()
        for n in nodes:
            if self._kind(n) in _EW and n not in seen:
                chain, cur = [n], n
                while len(cur.users) == 1 and self._kind(next(iter(cur.users))) in _EW:
                    cur = next(iter(cur.users)); chain.append(cur)
                seen.update(chain)
                if len(chain) >= 2:
                    recs.append({"kind": "fuse_elementwise", "nodes": [c.name for c in chain], "gain": (share([c.name for c in chain]) or 0.05 * len(chain)) * (1 - 1 / len(chain)),
                                 "message": f"{len(chain)} element-wise operations read and write the same tensor {len(chain)} times: one generated kernel reads it once"})
        # linear followed by activation
        for n in nodes:
            if self._kind(n) == "Linear" and len(n.users) == 1 and self._kind(next(iter(n.users))) in ("ReLU", "GELU", "relu", "gelu", "SiLU", "silu"):
                u = next(iter(n.users))
                recs.append({"kind": "fuse_epilogue", "nodes": [n.name, u.name], "gain": share([u.name]) or 0.1, "message": "apply the activation in the GEMM epilogue while the accumulator is still on chip"})
        # duplicated expressions
        sig = defaultdict(list)
        for n in nodes:
            if n.op in ("call_function", "call_method"):
                sig[(n.target, tuple(str(a) for a in n.args), tuple(sorted((k, str(v)) for k, v in n.kwargs.items())))].append(n.name)
        for names in sig.values():
            if len(names) > 1:
                recs.append({"kind": "common_subexpression", "nodes": names, "gain": share(names[1:]) or 0.03 * (len(names) - 1), "message": f"{len(names)} identical computations: keep one"})
        dead = [n.name for n in nodes if n.op not in ("output", "placeholder") and not n.users]
        if dead:
            recs.append({"kind": "dead_code", "nodes": dead, "gain": share(dead) or 0.02 * len(dead), "message": "results that nothing uses"})
        f32 = [k for k, p in self.gm.named_parameters() if p.dtype == torch.float32 and p.dim() >= 2]
        if f32:
            recs.append({"kind": "precision", "nodes": f32, "gain": 0.3, "message": "float32 matrices keep the tensor cores at a fraction of their bf16 rate: cast weights and activations to bfloat16"})
        if total:
            hot = max(self.times, key=self.times.get)
            if self.times[hot] / total > 0.5:
                recs.append({"kind": "hotspot", "nodes": [hot], "gain": 0.0, "message": f"{hot} takes {self.times[hot] / total:.0%} of the time: optimise it before anything else"})
        return sorted(recs, key=lambda r: -r["gain"])


# ================================================================================================ profile-guided optimisation
class ProfilingInterpreter(torch.fx.Interpreter):
    """Runs a graph node by node, accumulating call counts, time and the shapes each node saw."""

    def __init__(self, gm):
        super().__init__(gm)
        self.counts, self.times, self.shapes = Counter(), defaultdict(float), defaultdict(Counter)

    def run_node(self, n):
        t0 = time.perf_counter()
        r = super().run_node(n)
        if n.op not in ("placeholder", "output"):
            self.counts[n.name] += 1; self.times[n.name] += time.perf_counter() - t0
            if isinstance(r, torch.Tensor):
                self.shapes[n.name][tuple(r.shape)] += 1
        return r

    def profile(self): return {"counts": dict(self.counts), "times": dict(self.times), "shapes": {k: dict(v) for k, v in self.shapes.items()}}


class ProfileGuidedDispatcher:
    """Ordered list of ``(guard, implementation)``; after ``reoptimize`` the guards are tested in order of how often they
    held, and shapes seen often enough get an entry in a direct-lookup table that skips the guards altogether."""

    def __init__(self, fallback: Callable, hot_threshold: int = 10): self.variants, self.fallback, self.hits, self.shape_hits, self.table, self.hot, self.guard_evals = [], fallback, Counter(), Counter(), {}, hot_threshold, 0
    def add(self, name: str, guard: Callable, impl: Callable): self.variants.append((name, guard, impl)); return self

    def __call__(self, x: torch.Tensor):
        key = tuple(x.shape)
        self.shape_hits[key] += 1
        if key in self.table:
            return self.table[key](x)
        for name, g, impl in self.variants:
            self.guard_evals += 1
            if g(x):
                self.hits[name] += 1
                self._last = impl
                return impl(x)
        self.hits["fallback"] += 1; self._last = self.fallback
        return self.fallback(x)

    def reoptimize(self):
        self.variants.sort(key=lambda v: -self.hits[v[0]])
        for key, c in self.shape_hits.items():
            if c >= self.hot and key not in self.table:
                probe = torch.empty(key, device="meta")
                self.table[key] = next((impl for _, g, impl in self.variants if g(probe)), self.fallback)
        return [v[0] for v in self.variants]


# ================================================================================================ polyhedral loop nests
@dataclass
class Access:
    array: str
    index: list                                                                     # one dict per dimension: {loop var: coefficient, "": constant}
    write: bool = False


@dataclass
class LoopNest:
    """Perfect loop nest with affine accesses.  ``loops`` is ``[(var, lower, upper)]``, outermost first; ``statement`` is a
    Python expression template executed in the innermost body."""
    loops: list
    accesses: list
    statement: str = ""

    def dependences(self) -> list[tuple]:
        """Distance vectors of the uniform dependences between every write and every access to the same array (same linear
        part, different constants).  Non-uniform pairs are returned as ``None`` components (unknown distance) when the GCD
        test cannot exclude them."""
        vars_, out = [v for v, _, _ in self.loops], []
        for w in (a for a in self.accesses if a.write):
            for r in self.accesses:
                if r.array != w.array or (r is w):
                    continue
                dist, known, possible = {}, True, True
                for dw, dr in zip(w.index, r.index):
                    lin_w, lin_r = {k: v for k, v in dw.items() if k}, {k: v for k, v in dr.items() if k}
                    dc = dw.get("", 0) - dr.get("", 0)
                    if lin_w == lin_r:
                        if len(lin_w) == 1:
                            (v, c), = lin_w.items()
                            if dc % c:
                                possible = False
                            elif v in dist and dist[v] != dc // c:
                                possible = False
                            else:
                                dist[v] = dc // c
                        elif len(lin_w) == 0:
                            possible = possible and dc == 0
                        else:
                            known = False
                    else:
                        g = math.gcd(*[abs(c) for c in list(lin_w.values()) + list(lin_r.values())]) if lin_w or lin_r else 0
                        if g and dc % g:
                            possible = False
                        known = False
                if not possible:
                    continue
                vec = tuple(dist.get(v, 0 if known else None) for v in vars_) if known else tuple(dist.get(v) for v in vars_)
                if known:
                    if all(c == 0 for c in vec):
                        continue                                                 # same iteration: no loop-carried dependence
                    first = next(c for c in vec if c != 0)
                    vec = vec if first > 0 else tuple(-c for c in vec)          # source precedes sink
                out.append(vec)
        return sorted(set(out), key=str)

    def can_permute(self, order: Sequence[int]) -> bool:
        for d in self.dependences():
            if any(c is None for c in d):
                return False
            p = [d[i] for i in order]
            first = next((c for c in p if c != 0), 0)
            if first < 0:
                return False
        return True

    def can_tile(self) -> bool:
        """A band is tilable when it is fully permutable: every dependence component is non-negative."""
        return all(all(c is not None and c >= 0 for c in d) for d in self.dependences())

    def parallel_loops(self) -> list[str]: return [v for i, (v, _, _) in enumerate(self.loops) if all(d[i] == 0 for d in self.dependences())]

    def generate(self, order: Sequence[int] | None = None, tiles: dict | None = None, name: str = "kernel", arrays: str = "A") -> tuple[Callable, str]:
        order, tiles = list(order or range(len(self.loops))), tiles or {}
        if order != sorted(order) and not self.can_permute(order):
            raise ValueError("this loop order reverses a dependence")
        if tiles and not self.can_tile():
            raise ValueError("the nest is not fully permutable: tiling would reverse a dependence")
        lines, ind = [f"def {name}({arrays}):"], 1
        for i in order:                                                             # tile loops first
            v, lo, hi = self.loops[i]
            if v in tiles:
                lines.append("    " * ind + f"for {v}_t in range({lo}, {hi}, {tiles[v]}):"); ind += 1
        for i in order:
            v, lo, hi = self.loops[i]
            rng = f"range({v}_t, min({v}_t + {tiles[v]}, {hi}))" if v in tiles else f"range({lo}, {hi})"
            lines.append("    " * ind + f"for {v} in {rng}:"); ind += 1
        lines.append("    " * ind + self.statement)
        src = "\n".join(lines)
        ns: dict = {}
        exec(compile(src, f"<loopnest {name}>", "exec"), ns)                       # noqa: S102
        return ns[name], src


# ================================================================================================ probabilistic compilation
class ShapeDistribution:
    """Empirical distribution over a size parameter (observed values with weights)."""

    def __init__(self, values: Sequence[int], weights: Sequence[float] | None = None):
        w = torch.tensor(weights if weights is not None else [1.0] * len(values), dtype=torch.float64)
        self.values, self.p = list(values), w / w.sum()
    @classmethod
    def from_observations(cls, obs: Sequence[int]): c = Counter(obs); return cls(list(c), list(c.values()))
    def expectation(self, f: Callable[[int], float]) -> float: return float(sum(p * f(v) for v, p in zip(self.values, self.p.tolist())))
    def variance(self, f): m = self.expectation(f); return self.expectation(lambda v: (f(v) - m) ** 2)
    def quantile(self, f, q: float):
        pairs = sorted((f(v), p) for v, p in zip(self.values, self.p.tolist()))
        acc = 0.0
        for c, p in pairs:
            acc += p
            if acc >= q - 1e-12:
                return c
        return pairs[-1][0]


def choose_variant(variants: dict[str, Callable[[int], float]], dist: ShapeDistribution, risk_aversion: float = 0.0, tail: float | None = None) -> dict:
    """Variant with the lowest ``E[cost] + risk_aversion * std`` (or the lowest ``tail`` quantile when given)."""
    rows = {k: {"mean": dist.expectation(f), "std": math.sqrt(dist.variance(f)), "p99": dist.quantile(f, 0.99)} for k, f in variants.items()}
    score = (lambda r: dist.quantile(variants[r], tail)) if tail is not None else (lambda r: rows[r]["mean"] + risk_aversion * rows[r]["std"])
    best = min(rows, key=score)
    return {"choice": best, "table": rows}


# ================================================================================================ program synthesis
_SYNTH_UNARY = {"neg": torch.neg, "relu": torch.relu, "abs": torch.abs, "square": torch.square, "exp": torch.exp, "sigmoid": torch.sigmoid, "tanh": torch.tanh}
_SYNTH_BINARY = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "maximum": torch.maximum}


def synthesize(examples: Sequence[tuple[Sequence[torch.Tensor], torch.Tensor]], n_inputs: int, max_depth: int = 3, atol: float = 1e-6, constants: Sequence[float] = ()) -> dict | None:
    """Bottom-up enumeration of expressions over the inputs, smallest first; candidates that compute the same values on the
    examples as an earlier one are dropped (observational equivalence).  Returns the first expression matching every
    example."""
    ins = [torch.stack([e[0][i] for e in examples]) for i in range(n_inputs)]
    target = torch.stack([e[1] for e in examples])
    level = [(f"x{i}", v, (lambda *a, i=i: a[i])) for i, v in enumerate(ins)] + [(repr(c), torch.full_like(target, c), (lambda *a, c=c: torch.full_like(a[0], c))) for c in constants]
    seen, pool, tried = set(), [], 0
    def sig(v): return tuple(torch.nan_to_num(v, nan=1e30, posinf=1e31, neginf=-1e31).flatten().mul(1e6).round().tolist())
    def admit(cands):
        nonlocal tried
        new = []
        for e, v, f in cands:
            tried += 1
            if v.shape == target.shape and torch.allclose(v, target, atol=atol):
                return (e, f), new
            s = sig(v)
            if s not in seen and torch.isfinite(v).all():
                seen.add(s); new.append((e, v, f))
        return None, new
    hit, fresh = admit(level)
    pool += fresh
    depth = 1
    while hit is None and depth < max_depth:
        cands = [(f"{n}({e})", op(v), (lambda *a, op=op, f=f: op(f(*a)))) for n, op in _SYNTH_UNARY.items() for e, v, f in fresh]
        for n, op in _SYNTH_BINARY.items():
            for (e1, v1, f1), (e2, v2, f2) in itertools.chain(itertools.product(fresh, pool), itertools.product(pool, fresh)):
                if v1.shape == v2.shape and not (n in ("add", "mul", "maximum") and e1 > e2):
                    cands.append((f"{n}({e1}, {e2})", op(v1, v2), (lambda *a, op=op, f1=f1, f2=f2: op(f1(*a), f2(*a)))))
        hit, fresh = admit(cands)
        pool += fresh
        depth += 1
    return None if hit is None else {"expression": hit[0], "fn": hit[1], "candidates_tried": tried, "depth": depth}


# ================================================================================================ speculation
class SpeculativeFunction:
    """Runs a specialised implementation while its guard holds; a failed guard deoptimises that call to the general
    implementation, and a speculation that fails too often is dropped."""

    def __init__(self, general: Callable, max_failure_rate: float = 0.3, min_calls: int = 10): self.general, self.max_fail, self.min_calls, self.specs, self.stats = general, max_failure_rate, min_calls, [], {}

    def speculate(self, name: str, guard: Callable, fast: Callable):
        self.specs.append((name, guard, fast)); self.stats[name] = {"hits": 0, "deopts": 0, "active": True}; return self

    def __call__(self, *args):
        for name, guard, fast in self.specs:
            s = self.stats[name]
            if not s["active"]:
                continue
            if guard(*args):
                s["hits"] += 1
                return fast(*args)
            s["deopts"] += 1
            n = s["hits"] + s["deopts"]
            if n >= self.min_calls and s["deopts"] / n > self.max_fail:
                s["active"] = False
        return self.general(*args)


# ================================================================================================ differentiable and neural compilation
class DifferentiableScheduler(torch.nn.Module):
    """Relaxes the choice among kernel variants into a softmax over logits: the expected cost is differentiable in the
    logits, so measured costs pull the distribution toward the cheapest variant; a continuous knob (tile size) is optimised
    against a smooth cost model in the same way."""

    def __init__(self, variants: Sequence[str], temperature: float = 1.0):
        super().__init__()
        self.names, self.logits, self.temperature = list(variants), torch.nn.Parameter(torch.zeros(len(variants))), temperature

    def probabilities(self): return torch.softmax(self.logits / self.temperature, 0)
    def expected_cost(self, costs: torch.Tensor) -> torch.Tensor: return (self.probabilities() * costs).sum()
    def sample(self, generator=None) -> str: return self.names[int(torch.multinomial(self.probabilities().detach(), 1, generator=generator))]
    def best(self) -> str: return self.names[int(self.logits.argmax())]

    def fit(self, measure: Callable[[str], float], steps: int = 100, lr: float = 0.5, entropy: float = 0.01) -> list[float]:
        opt, hist = torch.optim.Adam([self.logits], lr=lr), []
        est, cnt = torch.zeros(len(self.names)), torch.zeros(len(self.names))
        for i in range(steps):
            k = i % len(self.names) if i < 2 * len(self.names) else int(torch.multinomial(self.probabilities().detach(), 1))
            cnt[k] += 1; est[k] += (measure(self.names[k]) - est[k]) / cnt[k]
            p = self.probabilities()
            loss = (p * est / est[cnt > 0].mean()).sum() + entropy * (p * p.clamp_min(1e-12).log()).sum()
            opt.zero_grad(); loss.backward(); opt.step()
            hist.append(float(self.expected_cost(est).detach()))
        return hist


def optimise_continuous_knob(cost: Callable[[torch.Tensor], torch.Tensor], init: float, lo: float, hi: float, steps: int = 200, lr: float = 0.05) -> float:
    """Gradient descent on a knob parameterised through a sigmoid so that it stays in ``[lo, hi]``."""
    z = torch.tensor(math.log((init - lo) / (hi - init)), requires_grad=True)
    opt = torch.optim.Adam([z], lr=lr)
    for _ in range(steps):
        opt.zero_grad(); cost(lo + (hi - lo) * torch.sigmoid(z)).backward(); opt.step()
    return float(lo + (hi - lo) * torch.sigmoid(z.detach()))


def graph_features(gm: torch.fx.GraphModule, example_inputs: Sequence[torch.Tensor]) -> torch.Tensor:
    """``[log flops, log bytes, matmul nodes, element-wise nodes, depth, log parameters]`` from one shape-propagating run."""
    from .fx import ShapeProp
    ShapeProp(gm).run(*example_inputs)
    mods, flops, nbytes, mm, ew = dict(gm.named_modules()), 0.0, 0.0, 0, 0
    for n in gm.graph.nodes:
        shp = n.meta.get("shape")
        if shp is None or n.op in ("placeholder", "output"):
            continue
        numel = math.prod(shp)
        nbytes += 4 * numel
        m = mods.get(n.target) if n.op == "call_module" else None
        if isinstance(m, torch.nn.Linear):
            flops += 2 * numel * m.in_features; nbytes += 4 * m.weight.numel(); mm += 1
        elif getattr(n.target, "__name__", "") == "matmul":
            flops += 2 * numel * n.all_input_nodes[0].meta["shape"][-1]; mm += 1
        else:
            flops += numel; ew += 1
    return torch.tensor([math.log1p(flops), math.log1p(nbytes), float(mm), float(ew), float(_graph_depth(gm)), math.log1p(sum(p.numel() for p in gm.parameters()))])


class LearnedCostModel(torch.nn.Module):
    """Small regressor from graph features to log run time, trained on measured programs and used to rank candidates
    without running them."""

    def __init__(self, n_features: int = 6, hidden: int = 32):
        super().__init__()
        self.net = torch.nn.Sequential(torch.nn.Linear(n_features, hidden), torch.nn.Tanh(), torch.nn.Linear(hidden, 1))
        self.register_buffer("mu", torch.zeros(n_features)); self.register_buffer("sd", torch.ones(n_features))

    def forward(self, f): return self.net((f - self.mu) / self.sd).squeeze(-1)

    def fit(self, feats: torch.Tensor, seconds: torch.Tensor, steps: int = 500, lr: float = 1e-2):
        self.mu, self.sd = feats.mean(0), feats.std(0).clamp_min(1e-6)
        opt, y = torch.optim.Adam(self.parameters(), lr=lr), seconds.log()
        for _ in range(steps):
            opt.zero_grad(); loss = torch.nn.functional.mse_loss(self(feats), y); loss.backward(); opt.step()
        return float(loss.detach())

    def predict_seconds(self, f): return self(f).detach().exp()
    def rank(self, feats: torch.Tensor) -> list[int]: return self(feats).detach().argsort().tolist()


# ================================================================================================ debug symbols
class DebugSymbolTable:
    """Maps every node of a traced graph to the user's source line that created it, and every line of the generated code back
    to its node."""

    def __init__(self, gm: torch.fx.GraphModule):
        self.symbols, self.code_map = {}, {}
        for n in gm.graph.nodes:
            st = n.stack_trace or n.meta.get("stack_trace")
            if st:
                m = re.findall(r'File "([^"]+)", line (\d+), in (\S+)(?:\n\s+(.*))?', st)
                if m:
                    import linecache
                    f, line, fn, text = m[-1]
                    self.symbols[n.name] = {"file": f, "line": int(line), "function": fn, "source": (text or linecache.getline(f, int(line))).strip()}
        for i, line in enumerate(gm.code.splitlines(), 1):
            m = re.match(r"\s+(\w+)(?:\s*:\s*[^=]+)?\s*=", line)
            if m and m.group(1) in self.symbols:
                self.code_map[i] = m.group(1)

    @classmethod
    def trace(cls, fn) -> tuple[torch.fx.GraphModule, "DebugSymbolTable"]:
        from .jit_compiler import trace_with_source
        gm = trace_with_source(fn)
        return gm, cls(gm)

    def lookup(self, node_name: str): return self.symbols.get(node_name)
    def source_of_generated_line(self, line: int):
        n = self.code_map.get(line)
        return None if n is None else self.symbols[n]
    def to_json(self) -> str: return json.dumps({"symbols": self.symbols, "lines": self.code_map}, indent=1)

    def annotate_error(self, node_name: str, error: BaseException) -> str:
        s = self.lookup(node_name)
        return f"{type(error).__name__}: {error}" + (f"\n  at {s['file']}:{s['line']} in {s['function']}\n    {s['source']}" if s else f"\n  at node {node_name}")


# ================================================================================================ hardware tuning
@dataclass(frozen=True)
class HardwareProfile:
    name: str = "B200"
    sms: int = 148
    smem_per_cta: int = 227 * 1024
    tmem_columns: int = 512
    l2_bytes: int = 126 << 20
    warp: int = 32
    max_threads: int = 1024


def tune_gemm_tiles(m: int, n: int, k: int, hw: HardwareProfile = HardwareProfile(), element_size: int = 2, candidates=((128, 256, 64), (128, 128, 64), (256, 128, 64), (128, 64, 64), (64, 128, 64), (64, 64, 64))) -> dict:
    """Tile ``(BM, BN, BK)`` and pipeline depth for a tcgen05 GEMM: the fp32 accumulator must fit the tensor memory columns
    (``BN`` columns per 128 rows, doubled for an overlapped epilogue), the operand stages must fit shared memory, and among
    the tiles that fit, the one with the best product of wave efficiency and operand reuse wins (ties: larger tile)."""
    best = None
    for bm, bn, bk in candidates:
        cols = bn * (2 if 2 * bn <= hw.tmem_columns else 1) * (bm // 128 if bm > 128 else 1)
        if cols > hw.tmem_columns:
            continue
        stage = (bm + bn) * bk * element_size
        stages = min(8, (hw.smem_per_cta - bm * bn * element_size - 1024) // stage)
        if stages < 2:
            continue
        tiles = math.ceil(m / bm) * math.ceil(n / bn)
        waves = math.ceil(tiles / hw.sms)
        eff = (m * n) / (waves * hw.sms * bm * bn)
        intensity = bm * bn / (bm + bn)
        key = (round(eff * min(1.0, intensity / (128 * 256 / 384)), 3), intensity)  # a smaller tile re-reads operands: scale by its FLOPs per operand byte
        if best is None or key > best[0]:
            best = (key, {"tile": (bm, bn, bk), "stages": int(stages), "tmem_columns": cols, "smem_bytes": int(stages * stage + bm * bn * element_size), "ctas": tiles, "waves": waves, "wave_efficiency": eff,
                          "double_buffered_accumulator": 2 * bn <= hw.tmem_columns, "split_k": max(1, min(8, hw.sms // tiles)) if tiles < hw.sms // 2 and k >= 4096 else 1})
    return best[1]


def tune_elementwise(numel: int, element_size: int = 2, hw: HardwareProfile = HardwareProfile(), threads: int = 256) -> dict:
    vec = 16 // element_size
    per_cta = threads * vec
    needed = math.ceil(numel / per_cta)
    resident = hw.sms * (2048 // threads)
    grid = needed if needed <= resident else resident
    return {"threads": threads, "vector_width": vec, "grid": grid, "persistent": needed > resident, "iterations_per_thread": math.ceil(needed / grid), "fits_l2": numel * element_size * 2 <= hw.l2_bytes}


# ================================================================================================ LLVM IR text
_LLVM_UNARY = {"neg": "fneg float {a}", "exp": "call float @llvm.exp.f32(float {a})", "sqrt": "call float @llvm.sqrt.f32(float {a})", "abs": "call float @llvm.fabs.f32(float {a})"}
_LLVM_BINARY = {"add": "fadd", "sub": "fsub", "mul": "fmul", "div": "fdiv"}


def emit_llvm_ir(ops: Sequence[tuple], n_inputs: int, name: str = "fused") -> str:
    """One loop over ``n`` elements computing a chain of operations.  ``ops`` is a list of ``(op, operand, ...)`` where an operand
    is ``"in<k>"``, ``"t<k>"`` (result of the k-th operation) or a float literal; the last result is stored.  ``relu`` and
    ``max`` lower to ``llvm.maxnum``."""
    args = ", ".join([f"float* noalias %in{i}" for i in range(n_inputs)] + ["float* noalias %out", "i64 %n"])
    L = [f"define void @{name}({args}) {{", "entry:", "  %empty = icmp sle i64 %n, 0", "  br i1 %empty, label %exit, label %loop", "loop:", "  %i = phi i64 [ 0, %entry ], [ %i.next, %loop ]"]
    for k in range(n_inputs):
        L += [f"  %p{k} = getelementptr inbounds float, float* %in{k}, i64 %i", f"  %in{k}.v = load float, float* %p{k}, align 4"]
    ref = lambda o: f"%{o}.v" if isinstance(o, str) and o.startswith("in") else f"%{o}" if isinstance(o, str) else f"{float(o):e}"
    decl = set()
    for k, (op, *operands) in enumerate(ops):
        a = [ref(o) for o in operands]
        if op in _LLVM_BINARY:
            L.append(f"  %t{k} = {_LLVM_BINARY[op]} float {a[0]}, {a[1]}")
        elif op in ("relu", "max"):
            decl.add("declare float @llvm.maxnum.f32(float, float)")
            L.append(f"  %t{k} = call float @llvm.maxnum.f32(float {a[0]}, float {a[1] if op == 'max' else '0.000000e+00'})")
        elif op in _LLVM_UNARY:
            if "call" in _LLVM_UNARY[op]:
                decl.add(f"declare float @llvm.{ {'exp': 'exp', 'sqrt': 'sqrt', 'abs': 'fabs'}[op] }.f32(float)")
            L.append(f"  %t{k} = " + _LLVM_UNARY[op].format(a=a[0]))
        else:
            raise NotImplementedError(op)
    L += [f"  %po = getelementptr inbounds float, float* %out, i64 %i", f"  store float %t{len(ops) - 1}, float* %po, align 4", "  %i.next = add nuw nsw i64 %i, 1", "  %done = icmp eq i64 %i.next, %n",
          "  br i1 %done, label %exit, label %loop", "exit:", "  ret void", "}"]
    return "\n".join(sorted(decl) + L) + "\n"


def interpret_llvm_ir(ir: str, inputs: Sequence[torch.Tensor]) -> torch.Tensor:
    """Evaluates the loop body of IR produced by :func:`emit_llvm_ir` on whole tensors (a check that the text computes what
    the chain says, without an LLVM toolchain)."""
    env: dict[str, torch.Tensor] = {f"%in{i}.v": t.float() for i, t in enumerate(inputs)}
    val = lambda tok: env[tok] if tok.startswith("%") else torch.full_like(inputs[0], float(tok), dtype=torch.float32)
    out = None
    for line in ir.splitlines():
        line = line.strip()
        m = re.match(r"(%t\d+) = (fadd|fsub|fmul|fdiv) float (\S+), (\S+)", line)
        if m:
            env[m.group(1)] = {"fadd": torch.add, "fsub": torch.sub, "fmul": torch.mul, "fdiv": torch.div}[m.group(2)](val(m.group(3)), val(m.group(4))); continue
        m = re.match(r"(%t\d+) = fneg float (\S+)", line)
        if m:
            env[m.group(1)] = -val(m.group(2)); continue
        m = re.match(r"(%t\d+) = call float @llvm\.(\w+)\.f32\(float ([^,)]+)(?:, float ([^)]+))?\)", line)
        if m:
            f = {"exp": torch.exp, "sqrt": torch.sqrt, "fabs": torch.abs}.get(m.group(2))
            env[m.group(1)] = f(val(m.group(3))) if f else torch.maximum(val(m.group(3)), val(m.group(4))); continue
        m = re.match(r"store float (%t\d+)", line)
        if m:
            out = env[m.group(1)]
    return out
