"""Backward-graph analysis and planning (``crates/torsh-autograd/src/graph_opt/``, ``stable_api.rs``, ``onnx_integration.rs``,
``hardware_acceleration.rs``): a graph of the backward functions under an output with what each saved for backward
(``graph_builder.rs``, ``graph_types.rs``), execution order, duplicate-work and dead-branch detection, fusable chains
(``optimization.rs``), a memory timeline over forward plus backward with peak prediction and checkpoint placement
(``memory_planning.rs``), ONNX export / import of differentiable functions, API stability levels with version checks, and
device selection for differentiation workloads."""
from __future__ import annotations

import math
import time
from collections import Counter, defaultdict
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch
from torch import nn


# ================================================================================================ graph
@dataclass
class GraphNode:
    id: int
    name: str
    inputs: list                                                                     # ids of the nodes this backward function feeds (towards the leaves)
    saved_bytes: int = 0
    is_leaf: bool = False
    leaf_shape: tuple | None = None
    requires_grad: bool = True


class BackwardGraph:
    """Nodes are the backward functions reachable from ``output.grad_fn``; an edge ``a -> b`` means the gradient leaving ``a``
    enters ``b``.  Saved-tensor sizes are measured by running ``fn`` again under a saved-tensor hook when ``fn`` and ``inputs`` are
    given (each saved tensor is attributed to the backward node created next)."""

    def __init__(self, output: torch.Tensor):
        self.nodes: dict[int, GraphNode] = {}
        self._fns = {}
        ids, stack = {}, [output.grad_fn]
        self.root = None
        while stack:
            f = stack.pop()
            if f is None or id(f) in ids:
                continue
            ids[id(f)] = len(ids); self._fns[ids[id(f)]] = f
            stack += [n for n, _ in f.next_functions]
        for key, nid in ids.items():
            f = self._fns[nid]
            leaf = hasattr(f, "variable")
            self.nodes[nid] = GraphNode(nid, type(f).__name__, [ids[id(n)] for n, _ in f.next_functions if n is not None], is_leaf=leaf, leaf_shape=tuple(f.variable.shape) if leaf else None)
        self.root = ids[id(output.grad_fn)] if output.grad_fn is not None else None

    @classmethod
    def from_function(cls, fn: Callable, *inputs: torch.Tensor) -> "BackwardGraph":
        saved = []
        with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t.numel() * t.element_size()) or t, lambda t: t):
            out = fn(*inputs)
        g = cls(out)
        g.total_saved_bytes = sum(saved)
        g.saved_tensor_count = len(saved)
        return g

    def node_count(self) -> int: return len(self.nodes)
    def edge_count(self) -> int: return sum(len(n.inputs) for n in self.nodes.values())
    def operations(self) -> Counter: return Counter(n.name for n in self.nodes.values() if not n.is_leaf)

    def execution_order(self) -> list[int]:
        """Order in which the engine can run the backward functions: a node runs after every node that feeds it."""
        indeg = Counter(i for n in self.nodes.values() for i in n.inputs)
        ready, order = [self.root], []
        while ready:
            v = ready.pop()
            order.append(v)
            for i in self.nodes[v].inputs:
                indeg[i] -= 1
                if indeg[i] == 0:
                    ready.append(i)
        return order

    def depth(self) -> int:
        memo = {}
        def d(v):
            if v not in memo:
                memo[v] = 1 + max((d(i) for i in self.nodes[v].inputs), default=0)
            return memo[v]
        return d(self.root) if self.root is not None else 0

    def dead_branches(self) -> list[int]:
        """Backward functions none of whose descendants is a leaf that accumulates a gradient: their work is wasted."""
        memo = {}
        def useful(v):
            if v not in memo:
                n = self.nodes[v]
                memo[v] = n.is_leaf or any(useful(i) for i in n.inputs)
            return memo[v]
        return sorted(v for v in self.nodes if not useful(v))

    def fusable_chains(self, min_length: int = 2) -> list[list[str]]:
        """Maximal chains of element-wise backward functions with a single consumer each (candidates for one fused kernel)."""
        ew = ("Add", "Sub", "Mul", "Div", "Neg", "Tanh", "Sigmoid", "Relu", "Exp", "Log", "Pow", "Gelu", "Silu", "Sqrt", "Abs")
        is_ew = lambda n: any(n.name.startswith(p + "Backward") for p in ew)
        consumers = Counter(i for n in self.nodes.values() for i in n.inputs)
        chains, seen = [], set()
        for v in self.execution_order():
            if v in seen or not is_ew(self.nodes[v]):
                continue
            chain, cur = [v], v
            while True:
                nxt = [i for i in self.nodes[cur].inputs if is_ew(self.nodes[i]) and consumers[i] == 1 and i not in seen]
                if len(nxt) != 1:
                    break
                cur = nxt[0]; chain.append(cur)
            seen.update(chain)
            if len(chain) >= min_length:
                chains.append([self.nodes[c].name for c in chain])
        return chains

    def summary(self) -> dict:
        return {"nodes": self.node_count(), "edges": self.edge_count(), "depth": self.depth(), "leaves": sum(n.is_leaf for n in self.nodes.values()), "operations": dict(self.operations()), "saved_bytes": getattr(self, "total_saved_bytes", None)}


def duplicate_subexpressions(fn: Callable, *example_inputs) -> list[list[str]]:
    """Groups of forward nodes that compute the same thing (same target and inputs) in a symbolic trace of ``fn``; each group
    costs one forward and one backward evaluation more than necessary."""
    gm = torch.fx.symbolic_trace(fn)
    sig = defaultdict(list)
    canon = {}
    for n in gm.graph.nodes:
        if n.op in ("call_function", "call_method"):
            key = (n.op, str(n.target), tuple(canon.get(a, a) if isinstance(a, torch.fx.Node) else repr(a) for a in n.args), tuple(sorted((k, repr(v)) for k, v in n.kwargs.items())))
            sig[key].append(n.name)
            canon[n] = sig[key][0]                                                  # later users of a duplicate compare equal too
    return [v for v in sig.values() if len(v) > 1]


# ================================================================================================ memory planning
@dataclass
class LayerCost:
    name: str
    activation_bytes: int                                                            # what the layer keeps for its backward
    output_bytes: int
    flops: float = 0.0


def profile_layers(model: nn.Sequential, x: torch.Tensor) -> list[LayerCost]:
    costs = []
    for name, m in model.named_children():
        saved = []
        with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t.numel() * t.element_size()) or t, lambda t: t):
            y = m(x)
        w = sum(p.numel() for p in m.parameters())
        costs.append(LayerCost(name, sum(saved), y.numel() * y.element_size(), 2.0 * w * (y.numel() / max(y.shape[-1], 1)) if w else y.numel()))
        x = y.detach().requires_grad_(True)
    return costs


def memory_timeline(costs: Sequence[LayerCost], checkpoints: Sequence[int] = ()) -> dict:
    """Live activation bytes after every forward and backward step.  Without checkpoints every layer's saved tensors live
    until its backward.  With checkpoints (indices of layers whose *input* is kept) only segment inputs live through the
    forward pass; in backward each segment is recomputed (its saved tensors appear), consumed and freed."""
    n, timeline, live = len(costs), [], 0
    if not checkpoints:
        for c in costs:
            live += c.activation_bytes; timeline.append(("fwd:" + c.name, live))
        for c in reversed(costs):
            timeline.append(("bwd:" + c.name, live)); live -= c.activation_bytes
        peak = max(v for _, v in timeline)
        return {"timeline": timeline, "peak_bytes": peak, "recompute_flops": 0.0}
    cps = sorted(set(checkpoints) | {0})
    bounds = cps + [n]
    held = 0
    for s, e in zip(bounds, bounds[1:]):
        held += costs[s - 1].output_bytes if s > 0 else 0
        timeline.append((f"fwd:segment[{s}:{e}]", held + max(c.activation_bytes for c in costs[s:e])))    # transient: one layer's saved tensors at a time
    peak_fwd = max(v for _, v in timeline)
    recompute = 0.0
    for s, e in reversed(list(zip(bounds, bounds[1:]))):
        seg = sum(c.activation_bytes for c in costs[s:e])
        timeline.append((f"bwd:segment[{s}:{e}]", held + seg))
        recompute += sum(c.flops for c in costs[s:e])
        held -= costs[s - 1].output_bytes if s > 0 else 0
    return {"timeline": timeline, "peak_bytes": max(v for _, v in timeline), "recompute_flops": recompute, "forward_peak": peak_fwd}


def plan_checkpoints(costs: Sequence[LayerCost], budget_bytes: float | None = None, segments: int | None = None) -> dict:
    """Segment boundaries minimising the peak: ``segments`` given, or the square-root rule, or the smallest number of segments
    whose peak fits ``budget_bytes``.  Boundaries are placed to balance saved bytes per segment (dynamic programming over
    prefix sums: minimise the largest segment)."""
    n = len(costs)
    def balanced(k):
        pref = [0]
        for c in costs:
            pref.append(pref[-1] + c.activation_bytes)
        INF = float("inf")
        best = [[INF] * (n + 1) for _ in range(k + 1)]; cut = [[0] * (n + 1) for _ in range(k + 1)]
        best[0][0] = 0
        for j in range(1, k + 1):
            for i in range(1, n + 1):
                for p in range(j - 1, i):
                    v = max(best[j - 1][p], pref[i] - pref[p])
                    if v < best[j][i]:
                        best[j][i], cut[j][i] = v, p
        cps, i = [], n
        for j in range(k, 0, -1):
            i = cut[j][i]; cps.append(i)
        return sorted(c for c in cps if c > 0)
    base = memory_timeline(costs)
    if segments is None and budget_bytes is None:
        segments = max(1, round(math.sqrt(n)))
    if segments is not None:
        cps = balanced(segments)
        return {"checkpoints": cps, **{k: v for k, v in memory_timeline(costs, cps).items() if k != "timeline"}, "baseline_peak": base["peak_bytes"]}
    for k in range(1, n + 1):
        cps = balanced(k)
        t = memory_timeline(costs, cps) if cps else base
        if t["peak_bytes"] <= budget_bytes:
            return {"checkpoints": cps, "peak_bytes": t["peak_bytes"], "recompute_flops": t["recompute_flops"], "baseline_peak": base["peak_bytes"], "fits": True}
    return {"checkpoints": balanced(n), "peak_bytes": memory_timeline(costs, balanced(n))["peak_bytes"], "baseline_peak": base["peak_bytes"], "fits": False, "recompute_flops": sum(c.flops for c in costs)}


def apply_checkpoints(model: nn.Sequential, checkpoints: Sequence[int]) -> nn.Module:
    """Wraps the segments between the boundaries in activation checkpointing."""
    from torch.utils.checkpoint import checkpoint
    layers = list(model.children())
    bounds = sorted(set(checkpoints) | {0}) + [len(layers)]
    segs = [nn.Sequential(*layers[s:e]) for s, e in zip(bounds, bounds[1:])]
    class _Ck(nn.Module):
        def __init__(self): super().__init__(); self.segments = nn.ModuleList(segs)
        def forward(self, x):
            for s in self.segments:
                x = checkpoint(s, x, use_reentrant=False) if x.requires_grad or any(p.requires_grad for p in s.parameters()) else s(x)
            return x
    return _Ck()


# ================================================================================================ ONNX bridge
def export_differentiable(module: nn.Module, example_inputs, path=None) -> bytes:
    """Serialises the forward function as ONNX; the importer below rebuilds it from tensor operations, so the imported
    model is differentiable again."""
    from ..onnx_io import export_onnx
    return export_onnx(module, example_inputs, path)


def import_differentiable(path_or_bytes) -> nn.Module:
    from ..onnx_io import load_onnx
    return load_onnx(path_or_bytes)


def verify_roundtrip_gradients(module: nn.Module, example: torch.Tensor, atol: float = 1e-5) -> dict:
    """Exports, imports and compares outputs and input gradients of the two models."""
    data = export_differentiable(module, (example,))
    back = import_differentiable(data)
    a, b = example.clone().requires_grad_(True), example.clone().requires_grad_(True)
    ya, yb = module(a), back(b)
    ga, = torch.autograd.grad(ya.sum(), a); gb, = torch.autograd.grad(yb.sum(), b)
    return {"output_max_diff": float((ya - yb).detach().abs().max()), "gradient_max_diff": float((ga - gb).abs().max()), "ok": bool(torch.allclose(ya, yb, atol=atol) and torch.allclose(ga, gb, atol=atol)), "bytes": len(data)}


# ================================================================================================ API stability
STABILITY_LEVELS = ("stable", "beta", "experimental", "deprecated")


class ApiCompatibilityChecker:
    """Features carry a stability level and the version that introduced (or removed) them; a program states the version it
    was written for and asks whether what it uses is available and stable."""

    def __init__(self, current_version: str = "0.1.3"): self.current, self.features = self._v(current_version), {}
    @staticmethod
    def _v(s): return tuple(int(p) for p in s.split("."))

    def register(self, name: str, level: str, since: str, removed_in: str | None = None, replacement: str | None = None):
        if level not in STABILITY_LEVELS:
            raise ValueError(level)
        self.features[name] = {"level": level, "since": since, "removed_in": removed_in, "replacement": replacement}; return self

    def with_defaults(self):
        for n, l, s in (("backward", "stable", "0.1.0"), ("grad", "stable", "0.1.0"), ("checkpoint", "stable", "0.1.0"), ("functional.jacobian", "stable", "0.1.0"), ("functional.hessian", "beta", "0.1.1"), ("graph_opt", "beta", "0.1.2"),
                        ("forward_ad", "experimental", "0.1.2"), ("quantum_autograd", "experimental", "0.1.3")):
            self.register(n, l, s)
        return self.register("Variable", "deprecated", "0.1.0", removed_in="0.2.0", replacement="Tensor.requires_grad_")

    def is_stable(self, name): return self.features[name]["level"] == "stable"
    def is_experimental(self, name): return self.features[name]["level"] == "experimental"
    def is_deprecated(self, name): return self.features[name]["level"] == "deprecated"

    def check(self, used: Sequence[str], written_for: str | None = None, allow: Sequence[str] = ("stable", "beta")) -> dict:
        target = self._v(written_for) if written_for else self.current
        problems = []
        for u in used:
            f = self.features.get(u)
            if f is None:
                problems.append({"feature": u, "problem": "unknown"}); continue
            if self._v(f["since"]) > target:
                problems.append({"feature": u, "problem": f"introduced in {f['since']}, later than {'.'.join(map(str, target))}"})
            if f["removed_in"] and self._v(f["removed_in"]) <= self.current:
                problems.append({"feature": u, "problem": f"removed in {f['removed_in']}", "replacement": f["replacement"]})
            elif f["level"] not in allow:
                problems.append({"feature": u, "problem": f"stability level is {f['level']}", "replacement": f["replacement"]})
        return {"compatible": not problems, "problems": problems}


# ================================================================================================ device selection
def select_device_for_workload(numel: int, flops_per_element: float = 10.0, devices: Sequence[dict] | None = None, transfer_gbps: float = 50.0, launch_us: float = 8.0) -> dict:
    """Where a differentiation workload of ``numel`` elements runs fastest: the host, or an accelerator once its launch overhead
    and the transfer of inputs and gradients are paid.  ``devices`` defaults to what the process can see."""
    if devices is None:
        devices = [{"name": "cpu", "tflops": 0.5 * (torch.get_num_threads() / 8), "resident": True}]
        if torch.cuda.is_available():
            devices.append({"name": "cuda", "tflops": 60.0, "resident": False})
    rows = {}
    for d in devices:
        compute = numel * flops_per_element / (d["tflops"] * 1e12)
        move = 0.0 if d.get("resident") else 2 * numel * 4 / (transfer_gbps * 1e9)
        rows[d["name"]] = compute + move + (0.0 if d["name"] == "cpu" else launch_us * 1e-6)
    best = min(rows, key=rows.get)
    return {"device": best, "seconds": rows, "speedup_over_cpu": rows.get("cpu", rows[best]) / rows[best]}
