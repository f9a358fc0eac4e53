"""Shape algebra and run-time environment analysis (``crates/torsh-core/src``): symbolic dimensions with arithmetic,
constraints and unification (``symbolic_shape.rs``), symbolic shape inference for common operations and a cached shape graph
(``shape_graph.rs``, ``gpu_shape_ops.rs``), index and stride helpers (``shape_utils.rs``), shape-annotated function signatures
checked at call time (``type_level_shapes.rs``), allocation-trace analysis with size-class and arena recommendations
(``alloc_optimizer.rs``) and detection of processor and accelerator capabilities (``backend_detection.rs``)."""
from __future__ import annotations

import functools
import inspect
import math
import os
import platform
import re
from collections import Counter, defaultdict
from dataclasses import dataclass, field
from typing import Any, Callable, Sequence

import torch


# ================================================================================================ symbolic dimensions
_OP_SIGNS = {"add": "+", "sub": "-", "mul": "*", "floordiv": "//", "mod": "%"}


class Sym:
    """Integer expression over named dimensions: a polynomial-free tree of ``+``, ``*``, ``//`` and ``%`` with constant folding.
    Equality is structural after normalising sums and products of constants."""

    def __init__(self, op: str, args: tuple = ()): self.op, self.args = op, args
    @staticmethod
    def dim(name: str) -> "Sym": return Sym("dim", (name,))
    @staticmethod
    def lift(v) -> "Sym": return v if isinstance(v, Sym) else Sym("const", (int(v),))

    def _bin(self, op, other, rev=False):
        a, b = (Sym.lift(other), self) if rev else (self, Sym.lift(other))
        if a.op == "const" and b.op == "const":
            x, y = a.args[0], b.args[0]
            return Sym.lift({"add": x + y, "mul": x * y, "floordiv": x // y if y else 0, "mod": x % y if y else 0, "sub": x - y}[op])
        if op == "mul":
            (c1, f1), (c2, f2) = _factors(a), _factors(b)
            return _build(c1 * c2, f1 + f2)
        if op == "add":
            if a.op == "const" and a.args[0] == 0:
                return b
            if b.op == "const" and b.args[0] == 0:
                return a
            if repr(a) > repr(b):
                a, b = b, a
        if op == "sub" and b.op == "const" and b.args[0] == 0:
            return a
        if op == "sub" and a == b:
            return Sym.lift(0)
        if op == "floordiv":
            if b.op == "const" and b.args[0] == 1:
                return a
            if a == b:
                return Sym.lift(1)
            (c1, f1), (c2, f2) = _factors(a), _factors(b)                           # cancel common factors: (8 * B * T) // (B * T) -> 8
            rest, ok = list(f1), c2 != 0 and c1 % c2 == 0
            for atom in f2:
                hit = next((k for k, r in enumerate(rest) if r == atom), None)
                if hit is None:
                    ok = False; break
                rest.pop(hit)
            if ok:
                return _build(c1 // c2, rest)
        return Sym(op, (a, b))

    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, True)
    def __sub__(self, o): return self._bin("sub", o)
    def __rsub__(self, o): return self._bin("sub", o, True)
    def __mul__(self, o): return self._bin("mul", o)
    def __rmul__(self, o): return self._bin("mul", o, True)
    def __floordiv__(self, o): return self._bin("floordiv", o)
    def __mod__(self, o): return self._bin("mod", o)
    def __eq__(self, o): return isinstance(o, (Sym, int)) and repr(self) == repr(Sym.lift(o))
    def __hash__(self): return hash(repr(self))
    def __repr__(self):
        if self.op in ("dim", "const"):
            return str(self.args[0])
        return f"({self.args[0]!r} {_OP_SIGNS[self.op]} {self.args[1]!r})"

    def free(self) -> set[str]:
        if self.op == "dim":
            return {self.args[0]}
        return set().union(*[a.free() for a in self.args if isinstance(a, Sym)]) if self.op != "const" else set()

    def evaluate(self, env: dict[str, int]) -> int:
        if self.op == "const":
            return self.args[0]
        if self.op == "dim":
            if self.args[0] not in env:
                raise KeyError(f"dimension {self.args[0]!r} is unbound")
            return env[self.args[0]]
        a, b = (x.evaluate(env) for x in self.args)
        return {"add": a + b, "sub": a - b, "mul": a * b, "floordiv": a // b, "mod": a % b}[self.op]

    def is_const(self): return self.op == "const"


def _factors(s: Sym) -> tuple[int, list]:
    if s.op == "const":
        return s.args[0], []
    if s.op == "mul":
        (c1, f1), (c2, f2) = _factors(s.args[0]), _factors(s.args[1])
        return c1 * c2, f1 + f2
    return 1, [s]


def _build(coef: int, atoms: list) -> Sym:
    """Canonical product: constant first, then the atoms in the order of their text."""
    if coef == 0:
        return Sym.lift(0)
    out = None
    for a in sorted(atoms, key=repr):
        out = a if out is None else Sym("mul", (out, a))
    if out is None:
        return Sym.lift(coef)
    return out if coef == 1 else Sym("mul", (Sym.lift(coef), out))


def sym_shape(*dims) -> tuple: return tuple(Sym.dim(d) if isinstance(d, str) else Sym.lift(d) for d in dims)


class ShapeEnv:
    """Bindings of dimension names, range constraints and equalities learnt by unification."""

    def __init__(self): self.bind: dict[str, int] = {}; self.ranges: dict[str, tuple[int, int]] = {}; self.alias: dict[str, Sym] = {}

    def constrain(self, name: str, lo: int = 1, hi: int = 2 ** 40): self.ranges[name] = (lo, hi); return self

    def unify(self, a, b, where: str = "") -> None:
        """Makes two dimensions equal: binds a free name to a concrete value (or to another expression) or checks constants."""
        a, b = self.resolve(Sym.lift(a)), self.resolve(Sym.lift(b))
        if a == b:
            return
        if a.is_const() and b.is_const():
            raise ValueError(f"shape mismatch{' in ' + where if where else ''}: {a} != {b}")
        if b.op == "dim" and not a.op == "dim":
            a, b = b, a
        if a.op == "dim":
            name = a.args[0]
            if b.is_const():
                lo, hi = self.ranges.get(name, (0, 2 ** 62))
                if not lo <= b.args[0] <= hi:
                    raise ValueError(f"dimension {name} = {b} violates its range [{lo}, {hi}]" + (f" in {where}" if where else ""))
                self.bind[name] = b.args[0]
            else:
                if name in b.free():
                    raise ValueError(f"cannot unify {a} with {b}: the dimension occurs in the expression")
                self.alias[name] = b
            return
        free = (a.free() | b.free()) - set(self.bind)
        if not free:
            if a.evaluate(self.bind) != b.evaluate(self.bind):
                raise ValueError(f"shape mismatch{' in ' + where if where else ''}: {a} = {a.evaluate(self.bind)} but {b} = {b.evaluate(self.bind)}")
            return
        self.pending = getattr(self, "pending", []) + [(a, b, where)]                 # checked once the names are bound

    def resolve(self, s: Sym) -> Sym:
        if s.op == "dim":
            n = s.args[0]
            if n in self.bind:
                return Sym.lift(self.bind[n])
            if n in self.alias:
                return self.resolve(self.alias[n])
            return s
        if s.op == "const":
            return s
        a, b = (self.resolve(x) for x in s.args)
        return a._bin(s.op, b)

    def concrete(self, shape: Sequence) -> tuple[int, ...]:
        out = tuple(self.resolve(Sym.lift(d)) for d in shape)
        missing = set().union(*[d.free() for d in out]) if out else set()
        if missing:
            raise KeyError(f"unbound dimensions: {sorted(missing)}")
        for a, b, where in getattr(self, "pending", []):
            if not (a.free() | b.free()) - set(self.bind) and a.evaluate(self.bind) != b.evaluate(self.bind):
                raise ValueError(f"shape mismatch{' in ' + where if where else ''}: {a} != {b}")
        return tuple(d.args[0] for d in out)


# ================================================================================================ symbolic shape inference
def infer_shape(op: str, env: ShapeEnv, *shapes, **attrs) -> tuple:
    """Output shape of ``matmul``, ``linear``, ``broadcast`` (element-wise), ``cat``, ``reshape`` (one ``-1`` allowed), ``transpose``,
    ``conv2d``, ``pool2d``, ``flatten``, ``reduce`` on symbolic inputs; equalities implied by the operation are recorded in ``env``."""
    L = Sym.lift
    if op == "matmul":
        a, b = shapes
        env.unify(a[-1], b[-2] if len(b) > 1 else b[-1], "matmul inner dimension")
        batch = infer_shape("broadcast", env, a[:-2], b[:-2]) if len(a) > 2 or len(b) > 2 else ()
        return tuple(batch) + ((a[-2],) if len(a) > 1 else ()) + ((b[-1],) if len(b) > 1 else ())
    if op == "linear":
        x, w = shapes
        env.unify(x[-1], w[1], "linear input features")
        return tuple(x[:-1]) + (w[0],)
    if op == "broadcast":
        a, b = (tuple(L(d) for d in s) for s in shapes)
        n = max(len(a), len(b))
        a, b = (L(1),) * (n - len(a)) + a, (L(1),) * (n - len(b)) + b
        out = []
        for x, y in zip(a, b):
            x, y = env.resolve(x), env.resolve(y)
            if x == 1:
                out.append(y)
            elif y == 1:
                out.append(x)
            else:
                env.unify(x, y, "broadcast"); out.append(env.resolve(x))
        return tuple(out)
    if op == "cat":
        dim = attrs.get("dim", 0)
        first = list(shapes[0])
        total = L(first[dim])
        for s in shapes[1:]:
            for i, (x, y) in enumerate(zip(first, s)):
                if i != dim % len(first):
                    env.unify(x, y, f"cat dimension {i}")
            total = total + L(s[dim])
        first[dim] = total
        return tuple(first)
    if op == "reshape":
        src, target = shapes[0], list(attrs["shape"])
        numel = functools.reduce(lambda a, b: a * b, [L(d) for d in src], L(1))
        known = functools.reduce(lambda a, b: a * b, [L(d) for d in target if not (isinstance(d, int) and d == -1)], L(1))
        if any(isinstance(d, int) and d == -1 for d in target):
            target[[i for i, d in enumerate(target) if isinstance(d, int) and d == -1][0]] = env.resolve(numel) // env.resolve(known)
        else:
            env.unify(numel, known, "reshape element count")
        return tuple(L(d) for d in target)
    if op == "transpose":
        s = list(shapes[0]); a, b = attrs["dims"]; s[a], s[b] = s[b], s[a]
        return tuple(s)
    if op in ("conv2d", "pool2d"):
        x = shapes[0]
        k, st, p, d = (attrs.get(n, v) for n, v in (("kernel", 3), ("stride", 1), ("padding", 0), ("dilation", 1)))
        k, st, p, d = [(v, v) if isinstance(v, int) else tuple(v) for v in (k, st, p, d)]
        size = lambda n, i: (L(n) + 2 * p[i] - d[i] * (k[i] - 1) - 1) // st[i] + 1
        if op == "conv2d":
            w = shapes[1]
            env.unify(x[1], L(w[1]) * attrs.get("groups", 1), "conv2d channels")
            return (x[0], L(w[0]), size(x[2], 0), size(x[3], 1))
        return (x[0], x[1], size(x[2], 0), size(x[3], 1))
    if op == "flatten":
        s, start = shapes[0], attrs.get("start", 1)
        return tuple(s[:start]) + (functools.reduce(lambda a, b: a * b, [L(d) for d in s[start:]], L(1)),)
    if op == "reduce":
        s, dim, keep = list(shapes[0]), attrs["dim"], attrs.get("keepdim", False)
        if keep:
            s[dim] = L(1)
        else:
            del s[dim]
        return tuple(s)
    raise ValueError(f"no shape rule for {op!r}")


class ShapeGraph:
    """Named tensors and the operations between them; ``infer`` propagates symbolic shapes once and caches them, ``specialize``
    evaluates every shape for concrete bindings, ``explain`` traces where a shape came from."""

    def __init__(self): self.env, self.shapes, self.ops, self.cache_hits = ShapeEnv(), {}, [], 0
    def input(self, name: str, *dims): self.shapes[name] = sym_shape(*dims); return name
    def op(self, out: str, kind: str, *inputs: str, **attrs): self.ops.append((out, kind, inputs, attrs)); return out

    def infer(self) -> dict[str, tuple]:
        for out, kind, inputs, attrs in self.ops:
            if out in self.shapes:
                self.cache_hits += 1; continue
            self.shapes[out] = infer_shape(kind, self.env, *[self.shapes[i] for i in inputs], **attrs)
        return {k: tuple(self.env.resolve(Sym.lift(d)) for d in v) for k, v in self.shapes.items()}

    def specialize(self, **bindings: int) -> dict[str, tuple[int, ...]]:
        self.infer()
        env = ShapeEnv(); env.bind, env.alias, env.ranges = {**self.env.bind}, dict(self.env.alias), dict(self.env.ranges)
        env.pending = list(getattr(self.env, "pending", []))
        for k, v in bindings.items():
            env.unify(Sym.dim(k), v, f"binding {k}")
        return {k: env.concrete(v) for k, v in self.shapes.items()}

    def explain(self, name: str) -> list[str]:
        lines, todo = [], [name]
        while todo:
            n = todo.pop()
            prod = next((o for o in self.ops if o[0] == n), None)
            shp = [repr(self.env.resolve(Sym.lift(d))) for d in self.shapes.get(n, ())]
            lines.append(f"{n}: [{', '.join(shp)}]" + (f" = {prod[1]}({', '.join(prod[2])})" if prod else " (input)"))
            if prod:
                todo += list(prod[2])
        return lines


# ================================================================================================ index and stride helpers
def contiguous_strides(shape: Sequence[int]) -> tuple[int, ...]:
    out, s = [], 1
    for d in reversed(shape):
        out.append(s); s *= max(d, 1)
    return tuple(reversed(out))


def is_contiguous(shape, strides) -> bool: return all(st == ex for d, st, ex in zip(shape, strides, contiguous_strides(shape)) if d > 1)
def ravel_index(index: Sequence[int], shape: Sequence[int]) -> int: return sum(i * s for i, s in zip(index, contiguous_strides(shape)))
def unravel_index(flat: int, shape: Sequence[int]) -> tuple[int, ...]:
    out = []
    for s in contiguous_strides(shape):
        out.append(flat // s); flat %= s
    return tuple(out)
def normalize_dim(dim: int, ndim: int) -> int:
    if not -ndim <= dim < ndim:
        raise IndexError(f"dimension {dim} is out of range for {ndim} dimensions")
    return dim % ndim
def broadcast_strides(shape, strides, target) -> tuple[int, ...]:
    """Strides that view a tensor of ``shape`` as ``target`` without copying (expanded dimensions get stride 0)."""
    pad = len(target) - len(shape)
    out = [0] * pad
    for d, st, t in zip(shape, strides, target[pad:]):
        if d != t and d != 1:
            raise ValueError(f"cannot broadcast {tuple(shape)} to {tuple(target)}")
        out.append(st if d == t and d != 1 else 0 if d == 1 and t != 1 else st)
    return tuple(out)
def can_view(shape, strides, new_shape) -> bool:
    """Whether ``new_shape`` can alias the same memory (no copy): checked by merging contiguous runs of dimensions."""
    try:
        need = 1 + sum((d - 1) * st for d, st in zip(shape, strides))
        torch.empty(need, device="meta").as_strided(tuple(shape), tuple(strides)).view(tuple(new_shape)); return True
    except RuntimeError:
        return False


# ================================================================================================ shape-annotated signatures
def typed_shapes(spec: str):
    """``@typed_shapes("x: B T D, w: D K -> B T K")`` checks tensor arguments (by name) and the result against named dimensions;
    equal names must agree within one call, integers are literal, ``...`` matches any leading dimensions."""
    ins, _, out = spec.partition("->")
    arg_specs = {a.split(":")[0].strip(): a.split(":")[1].split() for a in ins.split(",") if ":" in a}
    out_spec = out.split() if out.strip() else None

    def check(name, t, pattern, env):
        dims = list(t.shape)
        if pattern and pattern[0] == "...":
            k = len(pattern) - 1
            if len(dims) < k:
                raise TypeError(f"{name}: expected at least {k} dimensions, got shape {tuple(t.shape)}")
            lead, dims = dims[:len(dims) - k], dims[len(dims) - k:]
            if "..." in env and env["..."] != lead:
                raise TypeError(f"{name}: leading dimensions {lead} differ from {env['...']}")
            env["..."] = lead; pattern = pattern[1:]
        if len(dims) != len(pattern):
            raise TypeError(f"{name}: expected {len(pattern)} dimensions ({' '.join(pattern)}), got shape {tuple(t.shape)}")
        for p, d in zip(pattern, dims):
            if p.isdigit():
                if int(p) != d:
                    raise TypeError(f"{name}: dimension {p} expected, got {d} in shape {tuple(t.shape)}")
            elif env.setdefault(p, d) != d:
                raise TypeError(f"{name}: dimension {p} = {d} but it was {env[p]} elsewhere in this call")

    def deco(fn):
        sig = inspect.signature(fn)
        @functools.wraps(fn)
        def wrapper(*a, **k):
            bound = sig.bind(*a, **k); bound.apply_defaults()
            env = {}
            for name, pattern in arg_specs.items():
                check(name, bound.arguments[name], pattern, env)
            res = fn(*a, **k)
            if out_spec is not None:
                check("result", res, out_spec, env)
            return res
        wrapper.shape_spec = spec
        return wrapper
    return deco


# ================================================================================================ allocation analysis
@dataclass
class AllocEvent:
    time: float
    size: int
    kind: str                                                                        # "alloc" or "free"
    id: int


def analyze_allocations(events: Sequence[AllocEvent], small: int = 4096) -> dict:
    """From a trace of allocations and frees: peak live bytes, lifetime statistics per power-of-two size class, the share of
    small short-lived allocations (candidates for an arena), classes that are allocated repeatedly with the same size
    (candidates for a free list) and a recommended pool configuration."""
    live, born, peak, cur = {}, {}, 0, 0
    lifetimes, counts = defaultdict(list), Counter()
    for e in events:
        if e.kind == "alloc":
            live[e.id] = e.size; born[e.id] = e.time; cur += e.size; peak = max(peak, cur)
            counts[e.size] += 1
        elif e.id in live:
            cls = 1 << max(0, (live[e.id] - 1).bit_length())
            lifetimes[cls].append(e.time - born[e.id]); cur -= live.pop(e.id)
    total = sum(counts.values())
    med = lambda v: sorted(v)[len(v) // 2] if v else 0.0
    all_life = [t for v in lifetimes.values() for t in v]
    short = med(all_life)
    small_short = sum(1 for cls, v in lifetimes.items() if cls <= small for t in v if t <= short)
    repeated = {s: c for s, c in counts.items() if c >= 8}
    classes = {cls: {"count": len(v), "median_lifetime": med(v)} for cls, v in sorted(lifetimes.items())}
    recs = []
    if total and small_short / total > 0.3:
        recs.append({"kind": "arena", "reason": f"{small_short / total:.0%} of allocations are at most {small} bytes and short-lived", "arena_bytes": max(64 * 1024, 64 * small)})
    for s, c in sorted(repeated.items(), key=lambda kv: -kv[1])[:4]:
        recs.append({"kind": "free_list", "size": s, "reason": f"{c} allocations of exactly {s} bytes", "keep": min(c, 16)})
    if live:
        recs.append({"kind": "leak_check", "reason": f"{len(live)} allocations ({sum(live.values())} bytes) were never freed", "ids": sorted(live)[:10]})
    return {"peak_bytes": peak, "allocations": total, "leaked": len(live), "size_classes": classes, "repeated_sizes": repeated, "small_short_fraction": small_short / total if total else 0.0, "recommendations": recs}


# ================================================================================================ capability detection
def detect_capabilities(cpuinfo_text: str | None = None) -> dict:
    """Processor vector extensions (from ``/proc/cpuinfo`` when present), core counts, accelerators visible to the process with
    their compute capability, and the features this framework keys on (bf16 tensor cores, fp8, thread-block clusters, tensor
    memory) derived from the capability."""
    text = cpuinfo_text
    if text is None:
        try:
            text = open("/proc/cpuinfo").read()
        except OSError:
            text = ""
    m = re.search(r"^flags\s*:\s*(.*)$", text, re.M) or re.search(r"^Features\s*:\s*(.*)$", text, re.M)
    flags = set(m.group(1).split()) if m else set()
    simd = [n for n, f in (("sse4_2", "sse4_2"), ("avx", "avx"), ("avx2", "avx2"), ("fma", "fma"), ("avx512f", "avx512f"), ("avx512_bf16", "avx512_bf16"), ("amx_bf16", "amx_bf16"), ("neon", "asimd"), ("sve", "sve")) if f in flags]
    model = re.search(r"^model name\s*:\s*(.*)$", text, re.M)
    out = {"machine": platform.machine(), "cpu_model": model.group(1).strip() if model else platform.processor(), "logical_cores": os.cpu_count(), "simd": simd, "best_simd_bits": 512 if "avx512f" in simd else 256 if "avx2" in simd or "avx" in simd else 128 if simd else 0,
           "torch_threads": torch.get_num_threads(), "accelerators": []}
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            out["accelerators"].append({"index": i, "name": p.name, **features_for_capability(p.major, p.minor), "sms": p.multi_processor_count, "memory_gb": round(p.total_memory / 2 ** 30, 1)})
    out["preferred_device"] = "cuda" if out["accelerators"] else "cpu"
    return out


def features_for_capability(major: int, minor: int) -> dict:
    cc = major * 10 + minor
    return {"compute_capability": f"{major}.{minor}", "bf16_tensor_cores": cc >= 80, "fp8_tensor_cores": cc >= 89, "tma": cc >= 90, "thread_block_clusters": cc >= 90, "wgmma": cc == 90, "tcgen05_tensor_memory": cc >= 100, "fp4_tensor_cores": cc >= 100,
            "max_shared_memory_kb": 227 if cc >= 90 else 163 if cc >= 80 else 96, "arch_flag": f"sm_{cc}a" if cc >= 90 else f"sm_{cc}"}
