"""Graph capture and transformation (``crates/torsh-fx``): symbolic tracing into a node graph, an interpreter, the pass
manager with dead-code elimination / constant folding / common-subexpression elimination / operator fusion
(``crates/torsh-fx/src/passes.rs:16-396``), graph partitioning by device or cost, subgraph rewriting and JSON / DOT
export.  Graphs are ``torch.fx`` graphs; the fusion pass rewrites ``linear → gelu`` and ``add → layer_norm`` pairs to
the fused sm_100a ops of :mod:`torsh_b200.ops` so a traced module runs the same kernels as the hand-written models."""
from __future__ import annotations

import json
import operator
from dataclasses import dataclass, field
from typing import Callable

import torch
import torch.fx as tfx
import torch.nn.functional as F

GraphModule, Node, Graph, Interpreter = tfx.GraphModule, tfx.Node, tfx.Graph, tfx.Interpreter


def symbolic_trace(module: torch.nn.Module | Callable, concrete_args=None) -> GraphModule:
    return tfx.symbolic_trace(module, concrete_args=concrete_args)


# ------------------------------------------------------------------------------------------- passes
def dead_code_elimination(gm: GraphModule) -> int:
    n0 = len(gm.graph.nodes)
    gm.graph.eliminate_dead_code()
    gm.recompile()
    return n0 - len(gm.graph.nodes)


_PURE = {operator.add, operator.sub, operator.mul, operator.truediv, operator.neg, torch.add, torch.sub, torch.mul,
         torch.div, torch.matmul, torch.relu, torch.tanh, torch.sigmoid, torch.exp, F.relu, F.gelu, F.silu, F.linear,
         F.layer_norm, F.softmax, torch.transpose, torch.reshape}


def constant_folding(gm: GraphModule) -> int:
    """Evaluate call_function nodes whose inputs are all constants / parameters-free literals."""
    folded = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target not in _PURE:
            continue
        flat = list(node.args) + list(node.kwargs.values())
        nodes = [a for a in flat if isinstance(a, Node)]
        # foldable: every tensor input is a stored constant (a buffer), never a placeholder or a trainable parameter
        if not nodes or any(a.op != "get_attr" or isinstance(_fetch_attr(gm, a.target), torch.nn.Parameter) for a in nodes):
            continue
        load = lambda a: _fetch_attr(gm, a.target) if isinstance(a, Node) else a
        try:
            val = node.target(*[load(a) for a in node.args], **{k: load(v) for k, v in node.kwargs.items()})
        except Exception:
            continue
        if not isinstance(val, torch.Tensor):
            continue
        name = f"_folded_{folded}"
        gm.register_buffer(name, val)
        with gm.graph.inserting_before(node):
            new = gm.graph.get_attr(name)
        node.replace_all_uses_with(new)
        gm.graph.erase_node(node)
        folded += 1
    gm.recompile()
    return folded


def _fetch_attr(gm, target: str):
    obj = gm
    for part in target.split("."):
        obj = getattr(obj, part)
    return obj


def common_subexpression_elimination(gm: GraphModule) -> int:
    seen, removed = {}, 0
    for node in list(gm.graph.nodes):
        if node.op not in ("call_function", "call_method") or (node.op == "call_function" and node.target not in _PURE):
            continue
        key = (node.op, node.target, tuple(map(_key, node.args)), tuple(sorted((k, _key(v)) for k, v in node.kwargs.items())))
        if key in seen:
            node.replace_all_uses_with(seen[key])
            gm.graph.erase_node(node)
            removed += 1
        else:
            seen[key] = node
    gm.recompile()
    return removed


def _key(a):
    if isinstance(a, Node):
        return ("node", a.name)
    if isinstance(a, (list, tuple)):
        return tuple(map(_key, a))
    return ("const", repr(a))


def _fused_linear_gelu(x, w, b):
    from .ops.linear import linear
    return linear(x, w, b, gelu=True)


def _fused_add_layer_norm(x, r, shape, w, b, eps):
    return F.layer_norm(x + r, shape, w, b, eps)


def operator_fusion(gm: GraphModule) -> int:
    """``gelu(linear(x))`` (tanh form) → one GEMM with a GELU epilogue; ``layer_norm(x + r)`` → one fused node."""
    fused = 0
    for node in list(gm.graph.nodes):
        if node.op == "call_function" and node.target is F.gelu and node.kwargs.get("approximate") == "tanh":
            src = node.args[0]
            if isinstance(src, Node) and src.op == "call_function" and src.target is F.linear and len(src.users) == 1:
                a = list(src.args) + [src.kwargs.get("bias")] * (3 - len(src.args))
                with gm.graph.inserting_before(node):
                    new = gm.graph.call_function(_fused_linear_gelu, (a[0], a[1], a[2]))
                node.replace_all_uses_with(new); gm.graph.erase_node(node); gm.graph.erase_node(src); fused += 1
        elif node.op == "call_module" and isinstance(gm.get_submodule(node.target), torch.nn.GELU) \
                and gm.get_submodule(node.target).approximate == "tanh":
            src = node.args[0]
            if isinstance(src, Node) and src.op == "call_module" and type(gm.get_submodule(src.target)) is torch.nn.Linear \
                    and len(src.users) == 1:
                lin = gm.get_submodule(src.target)
                with gm.graph.inserting_before(node):
                    w = gm.graph.get_attr(src.target + ".weight")
                    b = gm.graph.get_attr(src.target + ".bias") if lin.bias is not None else None
                    new = gm.graph.call_function(_fused_linear_gelu, (src.args[0], w, b))
                node.replace_all_uses_with(new); gm.graph.erase_node(node); gm.graph.erase_node(src); fused += 1
        elif node.op == "call_function" and node.target is F.layer_norm:
            src = node.args[0]
            if isinstance(src, Node) and src.op == "call_function" and src.target in (operator.add, torch.add) and len(src.users) == 1:
                a = list(node.args[1:]) + [None] * 4
                kw = node.kwargs
                with gm.graph.inserting_before(node):
                    new = gm.graph.call_function(_fused_add_layer_norm, (src.args[0], src.args[1], a[0], kw.get("weight", a[1]),
                                                                         kw.get("bias", a[2]), kw.get("eps", a[3] or 1e-5)))
                node.replace_all_uses_with(new); gm.graph.erase_node(node); gm.graph.erase_node(src); fused += 1
    gm.recompile()
    return fused


@dataclass
class PassManager:
    passes: list[tuple[str, Callable[[GraphModule], int]]] = field(default_factory=list)

    @classmethod
    def default(cls) -> "PassManager":
        return cls([("constant_folding", constant_folding), ("cse", common_subexpression_elimination),
                    ("fusion", operator_fusion), ("dce", dead_code_elimination)])

    def add(self, name, fn): self.passes.append((name, fn)); return self

    def run(self, gm: GraphModule, max_rounds: int = 3) -> dict[str, int]:
        stats = {n: 0 for n, _ in self.passes}
        for _ in range(max_rounds):
            changed = 0
            for n, fn in self.passes:
                c = fn(gm); stats[n] += c; changed += c
            if not changed:
                break
        gm.graph.lint()
        return stats


# ------------------------------------------------------------------------------------------- analysis / export
def graph_stats(gm: GraphModule) -> dict:
    ops: dict[str, int] = {}
    for n in gm.graph.nodes:
        ops[n.op] = ops.get(n.op, 0) + 1
    return {"nodes": len(gm.graph.nodes), **ops, "parameters": sum(p.numel() for p in gm.parameters())}


def to_json(gm: GraphModule) -> str:
    nodes = [{"name": n.name, "op": n.op, "target": getattr(n.target, "__name__", str(n.target)),
              "inputs": [a.name for a in n.all_input_nodes]} for n in gm.graph.nodes]
    return json.dumps({"nodes": nodes}, indent=1)


def to_dot(gm: GraphModule) -> str:
    lines = ["digraph G {"]
    for n in gm.graph.nodes:
        lines.append(f'  {n.name} [label="{n.op}:{getattr(n.target, "__name__", n.target)}"];')
        lines += [f"  {a.name} -> {n.name};" for a in n.all_input_nodes]
    return "\n".join(lines + ["}"])


def partition_by_cost(gm: GraphModule, parts: int) -> list[list[str]]:
    """Contiguous partition of the compute nodes into ``parts`` stages of near-equal parameter cost (pipeline split)."""
    cost = []
    for n in gm.graph.nodes:
        if n.op == "call_module":
            cost.append((n.name, max(1, sum(p.numel() for p in gm.get_submodule(n.target).parameters()))))
        elif n.op in ("call_function", "call_method"):
            cost.append((n.name, 1))
    total, out, cur, acc = sum(c for _, c in cost), [], [], 0
    for name, c in cost:
        cur.append(name); acc += c
        if acc >= total * (len(out) + 1) / parts and len(out) < parts - 1:
            out.append(cur); cur = []
    out.append(cur)
    return out


def replace_pattern(gm: GraphModule, pattern: Callable, replacement: Callable) -> int:
    return len(tfx.replace_pattern(gm, pattern, replacement))


class ShapeProp(Interpreter):
    """Interpreter that records ``node.meta['shape'] / ['dtype']`` for every tensor-valued node."""

    def run_node(self, n):
        r = super().run_node(n)
        if isinstance(r, torch.Tensor):
            n.meta["shape"], n.meta["dtype"] = tuple(r.shape), r.dtype
        return r
