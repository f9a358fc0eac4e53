"""Graph tooling on top of :mod:`torsh_b200.fx` (the rest of ``crates/torsh-fx``):

* source generation: a traced graph as stand-alone Python / NumPy source or as C++ (plain loops or libtorch calls)
  (``codegen.rs``, ``python_codegen.rs``, ``cpp_codegen.rs``);
* analysis: metrics, lint rules, pattern detection and graph diff (``graph_analysis.rs``);
* rewriting: conv+bn folding, linear/conv + relu fusion, user patterns (``subgraph_rewriter.rs``);
* dynamic shapes: symbolic dimensions with constraints and shape rules (``dynamic_shapes.rs``);
* an editor with undo / redo (``interactive_editor.rs``), graph checkpoints and a resumable interpreter
  (``checkpointing.rs``), liveness-based memory analysis and buffer reuse (``memory_optimization.rs``);
* placement of nodes on devices by a cost model (``heterogeneous_computing.rs``, ``graph_partitioning.rs``), an execution
  backend registry (``custom_backends.rs``), result caching (``performance.rs``);
* post-training and quantisation-aware passes over a graph (``quantization/{ptq,qat}.rs``);
* architecture search over a cell search space (``neural_architecture_search/``).
"""
from __future__ import annotations

import copy
import hashlib
import json
import math
import operator
import time
from dataclasses import dataclass, field
from typing import Callable

import torch
import torch.fx as tfx
import torch.nn as nn
import torch.nn.functional as F

from .fx import GraphModule, Interpreter, Node, ShapeProp, _fetch_attr, symbolic_trace


def _tname(t) -> str:
    return t if isinstance(t, str) else getattr(t, "__name__", str(t))


# ================================================================================================ source generation
_PY_FN = {operator.add: "({0} + {1})", operator.sub: "({0} - {1})", operator.mul: "({0} * {1})", operator.truediv: "({0} / {1})",
          operator.neg: "(-{0})", operator.matmul: "({0} @ {1})", operator.getitem: "{0}[{1}]"}
_NP_FN = {"relu": "np.maximum({0}, 0)", "tanh": "np.tanh({0})", "sigmoid": "(1 / (1 + np.exp(-{0})))", "exp": "np.exp({0})",
          "matmul": "({0} @ {1})", "add": "({0} + {1})", "mul": "({0} * {1})", "sub": "({0} - {1})", "sum": "np.sum({0})",
          "linear": "({0} @ {1}.T + {2})", "flatten": "{0}.reshape({0}.shape[0], -1)", "transpose": "np.swapaxes({0}, {1}, {2})"}
_CPP_FN = {"relu": "torch::relu({0})", "tanh": "torch::tanh({0})", "sigmoid": "torch::sigmoid({0})", "exp": "torch::exp({0})",
           "matmul": "torch::matmul({0}, {1})", "add": "({0} + {1})", "mul": "({0} * {1})", "sub": "({0} - {1})",
           "truediv": "({0} / {1})", "linear": "torch::linear({0}, {1}, {2})", "gelu": "torch::gelu({0})",
           "flatten": "torch::flatten({0}, 1)", "softmax": "torch::softmax({0}, {1})", "layer_norm": "torch::layer_norm({0}, {1}, {2}, {3}, {4})"}


@dataclass
class CompiledCode:
    source: str
    language: str
    entry: str
    constants: dict = field(default_factory=dict)

    def load(self) -> Callable:
        """Python / NumPy targets only: execute the source and return the entry function bound to its constants."""
        if self.language not in ("python", "numpy"):
            raise ValueError("only Python targets can be loaded in-process")
        ns: dict = {}
        exec(compile(self.source, f"<generated {self.entry}>", "exec"), ns)
        fn, consts = ns[self.entry], self.constants
        return lambda *a: fn(consts, *a)


class PythonCodeGen:
    """Emits one flat function ``entry(consts, *inputs)``; parameters and buffers travel in ``consts`` by qualified name."""

    def __init__(self, with_torch: bool = True, indent: int = 4):
        self.torch, self.indent = with_torch, " " * indent

    def _arg(self, a):
        if isinstance(a, Node):
            return a.name
        if isinstance(a, (tuple, list)):
            inner = ", ".join(self._arg(v) for v in a)
            return f"({inner},)" if isinstance(a, tuple) else f"[{inner}]"
        if isinstance(a, (torch.dtype, torch.device)):
            return repr(a)
        return repr(a)

    def generate(self, gm: GraphModule, entry: str = "forward") -> CompiledCode:
        lines, consts, inputs = [], {}, []
        mod_calls = dict(gm.named_modules())
        for n in gm.graph.nodes:
            args = [self._arg(a) for a in n.args]
            kw = [f"{k}={self._arg(v)}" for k, v in n.kwargs.items()]
            if n.op == "placeholder":
                inputs.append(n.name)
            elif n.op == "get_attr":
                v = _fetch_attr(gm, n.target)
                consts[n.target] = v.detach() if self.torch else v.detach().cpu().numpy()
                lines.append(f"{n.name} = consts[{n.target!r}]")
            elif n.op == "call_function":
                name = _tname(n.target)
                if self.torch:
                    if n.target in _PY_FN and not kw:
                        lines.append(f"{n.name} = " + _PY_FN[n.target].format(*args))
                    else:
                        modname = getattr(n.target, "__module__", "") or ""
                        prefix = "F." if "functional" in modname else "torch."
                        lines.append(f"{n.name} = {prefix}{name}({', '.join(args + kw)})")
                else:
                    if name not in _NP_FN:
                        raise NotImplementedError(f"no NumPy lowering for {name}")
                    lines.append(f"{n.name} = " + _NP_FN[name].format(*args))
            elif n.op == "call_method":
                if self.torch:
                    lines.append(f"{n.name} = {args[0]}.{n.target}({', '.join(args[1:] + kw)})")
                else:
                    if n.target not in _NP_FN:
                        raise NotImplementedError(f"no NumPy lowering for method {n.target}")
                    lines.append(f"{n.name} = " + _NP_FN[n.target].format(*args))
            elif n.op == "call_module":
                m = mod_calls[n.target]
                lines.append(f"{n.name} = " + self._module_expr(m, n.target, args, consts))
            elif n.op == "output":
                lines.append(f"return {self._arg(n.args[0])}")
        head = ["import torch", "import torch.nn.functional as F"] if self.torch else ["import numpy as np"]
        body = "\n".join(self.indent + ln for ln in lines)
        src = "\n".join(head) + f"\n\n\ndef {entry}(consts, {', '.join(inputs)}):\n{body}\n"
        return CompiledCode(src, "python" if self.torch else "numpy", entry, consts)

    def _module_expr(self, m, qual, args, consts):
        def c(name):
            v = getattr(m, name)
            if v is None:
                return "None"
            consts[f"{qual}.{name}"] = v.detach() if self.torch else v.detach().cpu().numpy()
            return f"consts[{qual + '.' + name!r}]"
        if isinstance(m, nn.Linear):
            return f"F.linear({args[0]}, {c('weight')}, {c('bias')})" if self.torch else _NP_FN["linear"].format(args[0], c("weight"), c("bias") if m.bias is not None else "0")
        if isinstance(m, nn.ReLU):
            return f"torch.relu({args[0]})" if self.torch else _NP_FN["relu"].format(args[0])
        if isinstance(m, nn.Tanh):
            return f"torch.tanh({args[0]})" if self.torch else _NP_FN["tanh"].format(args[0])
        if isinstance(m, nn.Sigmoid):
            return f"torch.sigmoid({args[0]})" if self.torch else _NP_FN["sigmoid"].format(args[0])
        if self.torch and isinstance(m, nn.GELU):
            return f"F.gelu({args[0]}, approximate={m.approximate!r})"
        if self.torch and isinstance(m, nn.LayerNorm):
            return f"F.layer_norm({args[0]}, {tuple(m.normalized_shape)!r}, {c('weight')}, {c('bias')}, {m.eps!r})"
        if self.torch and isinstance(m, nn.Conv2d):
            return (f"F.conv2d({args[0]}, {c('weight')}, {c('bias')}, {m.stride!r}, {m.padding!r}, {m.dilation!r}, {m.groups})")
        if isinstance(m, nn.Flatten) and m.start_dim == 1 and m.end_dim == -1:
            return f"torch.flatten({args[0]}, 1)" if self.torch else _NP_FN["flatten"].format(args[0])
        if isinstance(m, (nn.Identity, nn.Dropout)):
            return args[0]
        raise NotImplementedError(f"no source lowering for module {type(m).__name__}")


class CppCodeGen:
    """C++ source for a graph: libtorch calls (``with_libtorch``) or plain loops over row-major float buffers for graphs
    of linear / relu / tanh / sigmoid / add / mul nodes.  The text is meant for a downstream build; it is not compiled here
    unless the caller does so."""

    def __init__(self, with_libtorch: bool = True, indent: int = 2):
        self.libtorch, self.indent = with_libtorch, " " * indent

    def generate(self, gm: GraphModule, entry: str = "forward") -> CompiledCode:
        return self._libtorch(gm, entry) if self.libtorch else self._plain(gm, entry)

    def _libtorch(self, gm, entry):
        ins, lines, consts = [], [], {}
        mods = dict(gm.named_modules())
        for n in gm.graph.nodes:
            a = [x.name if isinstance(x, Node) else json.dumps(x) if not isinstance(x, (tuple, list)) else "{" + ", ".join(map(str, x)) + "}" for x in n.args]
            if n.op == "placeholder":
                ins.append(f"const torch::Tensor& {n.name}")
            elif n.op == "get_attr":
                consts[n.target] = _fetch_attr(gm, n.target).detach()
                lines.append(f"auto {n.name} = consts.at(\"{n.target}\");")
            elif n.op in ("call_function", "call_method"):
                name = _tname(n.target)
                if name not in _CPP_FN:
                    raise NotImplementedError(f"no C++ lowering for {name}")
                lines.append(f"auto {n.name} = " + _CPP_FN[name].format(*a) + ";")
            elif n.op == "call_module":
                m = mods[n.target]
                if isinstance(m, nn.Linear):
                    consts[f"{n.target}.weight"] = m.weight.detach()
                    b = "torch::Tensor()"
                    if m.bias is not None:
                        consts[f"{n.target}.bias"] = m.bias.detach()
                        b = f"consts.at(\"{n.target}.bias\")"
                    lines.append(f"auto {n.name} = torch::linear({a[0]}, consts.at(\"{n.target}.weight\"), {b});")
                elif type(m).__name__.lower() in _CPP_FN:
                    lines.append(f"auto {n.name} = " + _CPP_FN[type(m).__name__.lower()].format(*a) + ";")
                else:
                    raise NotImplementedError(f"no C++ lowering for module {type(m).__name__}")
            elif n.op == "output":
                lines.append(f"return {n.args[0].name};")
        src = ("#include <torch/torch.h>\n#include <string>\n#include <unordered_map>\n\n"
               f"torch::Tensor {entry}(const std::unordered_map<std::string, torch::Tensor>& consts, {', '.join(ins)}) {{\n"
               + "\n".join(self.indent + ln for ln in lines) + "\n}\n")
        return CompiledCode(src, "cpp-libtorch", entry, consts)

    @staticmethod
    def _suffix(small, full):
        return len(small) <= len(full) and tuple(full[len(full) - len(small):]) == tuple(small)

    def _plain(self, gm, entry):
        """Needs ``node.meta['shape']`` (run :class:`ShapeProp` first).  Signature:
        ``void entry(const float* const* consts, const float* in0, ..., float* out)`` with ``consts`` in the order of
        ``CompiledCode.constants``."""
        mods, consts, ins, lines, bufs = dict(gm.named_modules()), {}, [], [], []
        numel = lambda n: math.prod(n.meta["shape"])
        I = self.indent

        def cidx(name, t):
            consts[name] = t.detach().float().contiguous()
            return list(consts).index(name)

        for n in gm.graph.nodes:
            if n.op == "placeholder":
                ins.append(f"const float* {n.name}")
                continue
            if n.op == "output":
                src_n = n.args[0]
                lines.append(f"for (long i = 0; i < {numel(src_n)}; ++i) out[i] = {src_n.name}[i];")
                continue
            if n.op == "get_attr":
                lines.append(f"const float* {n.name} = consts[{cidx(n.target, _fetch_attr(gm, n.target))}];")
                continue
            bufs.append(f"std::vector<float> {n.name}_buf({numel(n)}); float* {n.name} = {n.name}_buf.data();")
            m = mods.get(n.target) if n.op == "call_module" else None
            kind = type(m).__name__.lower() if m is not None else _tname(n.target)
            x = n.args[0].name
            if isinstance(m, nn.Linear):
                rows, (o, k) = numel(n.args[0]) // m.in_features, m.weight.shape
                w = cidx(f"{n.target}.weight", m.weight)
                b = f"consts[{cidx(f'{n.target}.bias', m.bias)}][j]" if m.bias is not None else "0.f"
                lines += [f"for (long r = 0; r < {rows}; ++r) for (long j = 0; j < {o}; ++j) {{",
                          f"{I}float acc = {b};", f"{I}for (long k = 0; k < {k}; ++k) acc += {x}[r * {k} + k] * consts[{w}][j * {k} + k];",
                          f"{I}{n.name}[r * {o} + j] = acc;", "}"]
            elif kind in ("relu", "tanh", "sigmoid"):
                e = {"relu": f"{x}[i] > 0.f ? {x}[i] : 0.f", "tanh": f"std::tanh({x}[i])", "sigmoid": f"1.f / (1.f + std::exp(-{x}[i]))"}[kind]
                lines.append(f"for (long i = 0; i < {numel(n)}; ++i) {n.name}[i] = {e};")
            elif kind in ("add", "mul", "sub") and all(isinstance(a, Node) and self._suffix(a.meta["shape"], n.meta["shape"]) for a in n.args[:2]):
                op = {"add": "+", "mul": "*", "sub": "-"}[kind]                    # an operand whose shape is a suffix repeats
                y = n.args[1]
                lines.append(f"for (long i = 0; i < {numel(n)}; ++i) {n.name}[i] = {x}[i % {numel(n.args[0])}] {op} {y.name}[i % {numel(y)}];")
            else:
                raise NotImplementedError(f"no plain C++ lowering for {kind}")
        body = "\n".join(I + ln for ln in bufs + lines)
        src = (f"#include <cmath>\n#include <vector>\n\nextern \"C\" void {entry}(const float* const* consts, {', '.join(ins)}, float* out) {{\n{body}\n}}\n")
        return CompiledCode(src, "cpp", entry, consts)


class LazyCompiler:
    """Generates source on first use and caches it by a hash of the graph's structure and target."""

    def __init__(self):
        self.cache, self.hits, self.misses = {}, 0, 0

    def compile(self, gm: GraphModule, target: str = "python") -> CompiledCode:
        key = hashlib.sha256((target + str(gm.graph)).encode()).hexdigest()
        if key in self.cache:
            self.hits += 1
            return self.cache[key]
        self.misses += 1
        gen = {"python": PythonCodeGen(True), "numpy": PythonCodeGen(False), "cpp": CppCodeGen(False), "cpp-libtorch": CppCodeGen(True)}[target]
        self.cache[key] = gen.generate(gm)
        return self.cache[key]

    def cache_stats(self): return {"entries": len(self.cache), "hits": self.hits, "misses": self.misses}
    def clear_cache(self): self.cache.clear()


# ================================================================================================ analysis
def calculate_graph_metrics(gm: GraphModule) -> dict:
    nodes = list(gm.graph.nodes)
    depth: dict[Node, int] = {}
    for n in nodes:
        depth[n] = 1 + max((depth[a] for a in n.all_input_nodes), default=0)
    fan_out = [len(n.users) for n in nodes]
    compute = [n for n in nodes if n.op in ("call_function", "call_method", "call_module")]
    width: dict[int, int] = {}
    for n in compute:
        width[depth[n]] = width.get(depth[n], 0) + 1
    return {"nodes": len(nodes), "edges": sum(len(n.all_input_nodes) for n in nodes), "compute_nodes": len(compute),
            "depth": max(depth.values(), default=0), "max_width": max(width.values(), default=0),
            "max_fan_out": max(fan_out, default=0), "avg_fan_out": sum(fan_out) / max(len(nodes), 1),
            "parallelism": len(compute) / max(len(width), 1)}


@dataclass
class LintIssue:
    rule: str
    severity: str
    node: str
    message: str


_SEV = {"info": 0, "warning": 1, "error": 2}


class GraphLinter:
    """Rules are ``(name, severity, fn(gm, node) -> message | None)``; the built-in set covers unused values, duplicated
    computation, no-op arithmetic, chains of reshapes and very high fan-out."""

    def __init__(self, severity_threshold: str = "info"):
        self.threshold, self.rules = severity_threshold, []
        self.add_rule("unused-value", "warning", lambda gm, n: "value is never used" if n.op not in ("output", "placeholder") and not n.users else None)
        self.add_rule("unused-input", "info", lambda gm, n: "input is never used" if n.op == "placeholder" and not n.users else None)
        self.add_rule("noop-arithmetic", "warning", self._noop)
        self.add_rule("reshape-chain", "info", lambda gm, n: "reshape of a reshape" if self._is_reshape(n) and n.all_input_nodes and self._is_reshape(n.all_input_nodes[0]) else None)
        self.add_rule("high-fan-out", "info", lambda gm, n: f"{len(n.users)} consumers" if len(n.users) > 16 else None)

    @staticmethod
    def _is_reshape(n): return n.op in ("call_method", "call_function") and _tname(n.target) in ("reshape", "view", "flatten")

    @staticmethod
    def _noop(gm, n):
        if n.op != "call_function" or len(n.args) != 2:
            return None
        c = n.args[1]
        if n.target in (operator.add, torch.add, operator.sub, torch.sub) and isinstance(c, (int, float)) and c == 0:
            return "adds zero"
        if n.target in (operator.mul, torch.mul, operator.truediv, torch.div) and isinstance(c, (int, float)) and c == 1:
            return "multiplies by one"
        return None

    def add_rule(self, name, severity, fn): self.rules.append((name, severity, fn))

    def lint_graph(self, gm: GraphModule) -> list[LintIssue]:
        out, seen = [], {}
        for n in gm.graph.nodes:
            for name, sev, fn in self.rules:
                msg = fn(gm, n)
                if msg and _SEV[sev] >= _SEV[self.threshold]:
                    out.append(LintIssue(name, sev, n.name, msg))
            if n.op in ("call_function", "call_method"):
                key = (n.op, n.target, tuple(map(str, n.args)), tuple(sorted((k, str(v)) for k, v in n.kwargs.items())))
                if key in seen and _SEV["warning"] >= _SEV[self.threshold]:
                    out.append(LintIssue("duplicate-computation", "warning", n.name, f"same computation as {seen[key]}"))
                seen.setdefault(key, n.name)
        return out


def detect_patterns(gm: GraphModule) -> list[dict]:
    """Known idioms by structure: residual connections, attention cores, linear -> activation, normalisation -> linear."""
    mods, out = dict(gm.named_modules()), []
    kind = lambda n: type(mods[n.target]).__name__.lower() if n.op == "call_module" else _tname(n.target).lower() if n.op != "placeholder" else "input"
    anc: dict[Node, set] = {}
    for n in gm.graph.nodes:
        anc[n] = set().union(*[anc[a] | {a} for a in n.all_input_nodes]) if n.all_input_nodes else set()
    for n in gm.graph.nodes:
        k = kind(n) if n.op != "output" else "output"
        ins = n.all_input_nodes
        if k == "add" and len(ins) == 2 and (ins[0] in anc[ins[1]] or ins[1] in anc[ins[0]]):
            out.append({"pattern": "residual", "nodes": [n.name]})
        if k in ("relu", "gelu", "silu", "tanh", "sigmoid") and ins and kind(ins[0]) in ("linear", "conv2d"):
            out.append({"pattern": f"{kind(ins[0])}+activation", "nodes": [ins[0].name, n.name]})
        if k == "linear" and ins and kind(ins[0]) in ("layernorm", "layer_norm", "rmsnorm"):
            out.append({"pattern": "norm+linear", "nodes": [ins[0].name, n.name]})
        if k == "matmul" and ins and any(kind(a) == "softmax" for a in ins):
            sm = next(a for a in ins if kind(a) == "softmax")
            if any(kind(a) in ("matmul", "truediv", "mul") for a in sm.all_input_nodes):
                out.append({"pattern": "attention", "nodes": [sm.name, n.name]})
    return out


def graph_diff(a: GraphModule, b: GraphModule) -> dict:
    sig = lambda gm: {n.name: (n.op, _tname(n.target), tuple(x.name for x in n.all_input_nodes)) for n in gm.graph.nodes}
    sa, sb = sig(a), sig(b)
    return {"added": sorted(set(sb) - set(sa)), "removed": sorted(set(sa) - set(sb)),
            "changed": sorted(k for k in set(sa) & set(sb) if sa[k] != sb[k]), "identical": sa == sb}


# ================================================================================================ rewriting
def fold_conv_bn(gm: GraphModule) -> int:
    """Folds an eval-mode BatchNorm2d into the preceding Conv2d's weight and bias (conv must have no other consumer)."""
    mods, n_folded = dict(gm.named_modules()), 0
    for n in list(gm.graph.nodes):
        if n.op != "call_module" or not isinstance(mods.get(n.target), nn.BatchNorm2d):
            continue
        prev = n.args[0]
        if not (isinstance(prev, Node) and prev.op == "call_module" and isinstance(mods.get(prev.target), nn.Conv2d) and len(prev.users) == 1):
            continue
        bn, conv = mods[n.target], mods[prev.target]
        if bn.training or not bn.track_running_stats:
            continue
        scale = (bn.weight if bn.affine else torch.ones_like(bn.running_var)) * (bn.running_var + bn.eps).rsqrt()
        shift = (bn.bias if bn.affine else torch.zeros_like(bn.running_mean)) - bn.running_mean * scale
        with torch.no_grad():
            conv.weight.mul_(scale.reshape(-1, 1, 1, 1))
            bias = conv.bias * scale + shift if conv.bias is not None else shift
            conv.bias = nn.Parameter(bias.clone())
        n.replace_all_uses_with(prev)
        gm.graph.erase_node(n)
        n_folded += 1
    gm.graph.lint()
    gm.recompile()
    return n_folded


class _FusedActivation(nn.Module):
    def __init__(self, inner: nn.Module, act: str):
        super().__init__()
        self.inner, self.act = inner, act

    def forward(self, x):
        return getattr(F, self.act)(self.inner(x))


def fuse_module_activation(gm: GraphModule, kinds=(nn.Linear, nn.Conv2d), act=nn.ReLU) -> int:
    """Replaces ``module -> activation module`` pairs by a single call of a wrapper module (one graph node, one launch site)."""
    mods, fused = dict(gm.named_modules()), 0
    for n in list(gm.graph.nodes):
        if n.op != "call_module" or not isinstance(mods.get(n.target), act):
            continue
        prev = n.args[0]
        if not (isinstance(prev, Node) and prev.op == "call_module" and isinstance(mods.get(prev.target), kinds) and len(prev.users) == 1):
            continue
        name = prev.target.replace(".", "_") + "_fused"
        gm.add_module(name, _FusedActivation(mods[prev.target], act.__name__.lower()))
        with gm.graph.inserting_after(n):
            new = gm.graph.call_module(name, prev.args, prev.kwargs)
        n.replace_all_uses_with(new)
        gm.graph.erase_node(n)
        gm.graph.erase_node(prev)
        fused += 1
    gm.graph.lint()
    gm.recompile()
    return fused


class SubgraphRewriter:
    """Ordered list of rewrites: built-in fusions plus ``(pattern, replacement)`` function pairs matched structurally."""

    def __init__(self):
        self.steps: list = []

    def add_pattern(self, pattern: Callable, replacement: Callable):
        self.steps.append(("pattern", pattern, replacement))
        return self

    def with_common_fusions(self):
        self.steps += [("fn", fold_conv_bn), ("fn", fuse_module_activation)]
        return self

    def find_matches(self, gm: GraphModule, pattern: Callable) -> int:
        from torch.fx.passes.utils.matcher_utils import SubgraphMatcher
        return len(SubgraphMatcher(symbolic_trace(pattern).graph, match_output=False, match_placeholder=False, remove_overlapping_matches=True).match(gm.graph))

    def apply(self, gm: GraphModule) -> dict:
        report = {}
        for step in self.steps:
            if step[0] == "fn":
                report[step[1].__name__] = step[1](gm)
            else:
                report[step[1].__name__] = len(tfx.replace_pattern(gm, step[1], step[2]))
        return report


# ================================================================================================ dynamic shapes
class DynamicDim:
    """A dimension that is a known size, a named symbol, or unknown."""

    __slots__ = ("size", "name")

    def __init__(self, size: int | None = None, name: str | None = None):
        self.size, self.name = size, name

    @classmethod
    def static(cls, n): return cls(size=int(n))
    @classmethod
    def symbolic(cls, name): return cls(name=name)
    @classmethod
    def unknown(cls): return cls()
    def is_static(self): return self.size is not None
    def is_symbolic(self): return self.size is None and self.name is not None
    def is_unknown(self): return self.size is None and self.name is None
    def __eq__(self, o): return isinstance(o, DynamicDim) and (self.size, self.name) == (o.size, o.name)
    def __hash__(self): return hash((self.size, self.name))
    def __repr__(self): return str(self.size) if self.is_static() else self.name if self.is_symbolic() else "?"


class DynamicShape:
    def __init__(self, dims):
        self.dims = [d if isinstance(d, DynamicDim) else DynamicDim.symbolic(d) if isinstance(d, str) else DynamicDim.unknown() if d is None else DynamicDim.static(d) for d in dims]

    @property
    def rank(self): return len(self.dims)
    def is_static(self): return all(d.is_static() for d in self.dims)
    def symbols(self): return [d.name for d in self.dims if d.is_symbolic()]
    def has_unknown_dims(self): return any(d.is_unknown() for d in self.dims)
    def substitute(self, env: dict): return DynamicShape([DynamicDim.static(env[d.name]) if d.is_symbolic() and d.name in env else d for d in self.dims])

    def to_static_shape(self):
        if not self.is_static():
            raise ValueError(f"shape {self} still has symbolic or unknown dimensions")
        return tuple(d.size for d in self.dims)

    def __eq__(self, o): return isinstance(o, DynamicShape) and self.dims == o.dims
    def __repr__(self): return "[" + ", ".join(map(repr, self.dims)) + "]"


def broadcast_dynamic_shapes(a: DynamicShape, b: DynamicShape) -> DynamicShape:
    out = []
    for i in range(1, max(a.rank, b.rank) + 1):
        da = a.dims[-i] if i <= a.rank else DynamicDim.static(1)
        db = b.dims[-i] if i <= b.rank else DynamicDim.static(1)
        if da.is_static() and da.size == 1:
            out.append(db)
        elif db.is_static() and db.size == 1 or da == db:
            out.append(da)
        elif da.is_static() and db.is_static():
            raise ValueError(f"cannot broadcast {a} with {b}")
        else:
            out.append(da if da.is_static() else db if db.is_static() else DynamicDim.unknown() if da.is_unknown() or db.is_unknown() else da)
    return DynamicShape(out[::-1])


def matmul_dynamic_shape(a: DynamicShape, b: DynamicShape) -> DynamicShape:
    ka, kb = a.dims[-1], b.dims[-2] if b.rank > 1 else b.dims[-1]
    if ka.is_static() and kb.is_static() and ka.size != kb.size:
        raise ValueError(f"inner dimensions differ: {a} @ {b}")
    batch = broadcast_dynamic_shapes(DynamicShape(a.dims[:-2]), DynamicShape(b.dims[:-2])).dims if max(a.rank, b.rank) > 2 else []
    return DynamicShape(batch + a.dims[-2:-1] + (b.dims[-1:] if b.rank > 1 else []))


class DynamicShapeContext:
    """Symbols with ``min`` / ``max`` / ``multiple_of`` / ``equal`` constraints; resolves shapes against bindings."""

    def __init__(self):
        self.symbols: dict[str, dict] = {}
        self.equalities: list[tuple[str, str]] = []
        self.shapes: dict[str, DynamicShape] = {}

    def register_symbol(self, name, min: int = 1, max: int | None = None, multiple_of: int = 1):
        self.symbols[name] = {"min": min, "max": max, "multiple_of": multiple_of}

    def add_constraint(self, a: str, b: str): self.equalities.append((a, b))
    def set_shape(self, node: str, shape: DynamicShape): self.shapes[node] = shape
    def get_shape(self, node: str): return self.shapes.get(node)

    def validate_constraints(self, env: dict) -> list[str]:
        errs = []
        for s, c in self.symbols.items():
            if s not in env:
                continue
            v = env[s]
            if v < c["min"] or (c["max"] is not None and v > c["max"]):
                errs.append(f"{s}={v} outside [{c['min']}, {c['max']}]")
            if v % c["multiple_of"]:
                errs.append(f"{s}={v} is not a multiple of {c['multiple_of']}")
        errs += [f"{a}={env[a]} differs from {b}={env[b]}" for a, b in self.equalities if a in env and b in env and env[a] != env[b]]
        return errs

    def resolve_symbols(self, env: dict) -> dict[str, tuple]:
        errs = self.validate_constraints(env)
        if errs:
            raise ValueError("; ".join(errs))
        return {k: s.substitute(env).to_static_shape() for k, s in self.shapes.items()}

    def get_unresolved_symbols(self, env: dict): return sorted({s for sh in self.shapes.values() for s in sh.symbols()} - set(env))

    def infer(self, gm: GraphModule, input_shapes: dict[str, DynamicShape]):
        """Shape rules for element-wise ops, matmul / linear and reductions over the graph's nodes."""
        mods = dict(gm.named_modules())
        for n in gm.graph.nodes:
            ins = [self.shapes[a.name] for a in n.all_input_nodes if a.name in self.shapes]
            if n.op == "placeholder":
                self.shapes[n.name] = input_shapes[n.name]
            elif n.op == "call_module" and isinstance(mods[n.target], nn.Linear):
                self.shapes[n.name] = DynamicShape(ins[0].dims[:-1] + [DynamicDim.static(mods[n.target].out_features)])
            elif n.op == "call_function" and _tname(n.target) == "matmul":
                self.shapes[n.name] = matmul_dynamic_shape(*ins[:2])
            elif n.op in ("call_function", "call_method") and _tname(n.target) in ("sum", "mean") and ins:
                dim = n.kwargs.get("dim", n.args[1] if len(n.args) > 1 else None)
                self.shapes[n.name] = DynamicShape([]) if dim is None else DynamicShape([d for i, d in enumerate(ins[0].dims) if i != dim % ins[0].rank])
            elif len(ins) == 2:
                self.shapes[n.name] = broadcast_dynamic_shapes(*ins)
            elif len(ins) == 1 and n.op != "output":
                self.shapes[n.name] = ins[0]
        return self.shapes


# ================================================================================================ editor
class GraphEditor:
    """Programmatic graph edits with undo / redo; every edit snapshots the module before it runs."""

    def __init__(self, gm: GraphModule):
        self.gm, self._undo, self._redo = gm, [], []

    def _node(self, name) -> Node:
        return next(n for n in self.gm.graph.nodes if n.name == name)

    def _commit(self, fn):
        self._undo.append(copy.deepcopy(self.gm))
        self._redo.clear()
        fn()
        self.gm.graph.lint()
        self.gm.recompile()

    def insert_after(self, name: str, fn: Callable, *extra_args, **kw):
        def go():
            n = self._node(name)
            with self.gm.graph.inserting_after(n):
                new = self.gm.graph.call_function(fn, (n, *extra_args), kw)
            n.replace_all_uses_with(new, delete_user_cb=lambda u: u is not new)
        self._commit(go)

    def remove(self, name: str):
        """Removes a single-input node, wiring its consumers to its input."""
        def go():
            n = self._node(name)
            n.replace_all_uses_with(n.all_input_nodes[0])
            self.gm.graph.erase_node(n)
        self._commit(go)

    def replace_target(self, name: str, target):
        self._commit(lambda: setattr(self._node(name), "target", target))

    def rename(self, name: str, new: str):
        self._commit(lambda: setattr(self._node(name), "name", new))

    def undo(self) -> bool:
        if not self._undo:
            return False
        self._redo.append(self.gm)
        self.gm = self._undo.pop()
        return True

    def redo(self) -> bool:
        if not self._redo:
            return False
        self._undo.append(self.gm)
        self.gm = self._redo.pop()
        return True

    def export_graph(self, fmt: str = "json") -> str:
        from .fx import to_dot, to_json
        return to_json(self.gm) if fmt == "json" else to_dot(self.gm)


# ================================================================================================ checkpoints
def save_graph_checkpoint(gm: GraphModule, path, metadata: dict | None = None) -> str:
    """The module (graph + state) with a SHA-256 of the state, for :func:`load_graph_checkpoint` to verify."""
    state = {k: v.detach().cpu() for k, v in gm.state_dict().items()}
    digest = hashlib.sha256(b"".join(k.encode() + v.contiguous().numpy().tobytes() for k, v in sorted(state.items()))).hexdigest()
    torch.save({"module": gm, "checksum": digest, "metadata": metadata or {}, "saved": time.time()}, path)
    return digest


def load_graph_checkpoint(path, verify: bool = True):
    ck = torch.load(path, weights_only=False)
    gm = ck["module"]
    if verify:
        state = {k: v.detach().cpu() for k, v in gm.state_dict().items()}
        digest = hashlib.sha256(b"".join(k.encode() + v.contiguous().numpy().tobytes() for k, v in sorted(state.items()))).hexdigest()
        if digest != ck["checksum"]:
            raise ValueError("graph checkpoint checksum mismatch")
    return gm, ck["metadata"]


class ResumableInterpreter:
    """Runs a graph node by node, keeps the environment every ``frequency`` nodes, and can continue from a saved
    environment (the already computed values are not recomputed)."""

    def __init__(self, gm: GraphModule, frequency: int = 1):
        self.gm, self.frequency, self.executed = gm, frequency, []
        self.saved: dict | None = None

    def run(self, *args, stop_after: str | None = None, resume: dict | None = None):
        interp = Interpreter(self.gm)
        env = dict(resume["env"]) if resume else {}
        it = iter(args)
        self.executed = []
        for i, n in enumerate(self.gm.graph.nodes):
            if n.name in env:
                if n.op == "placeholder":
                    next(it, None)
                continue
            if n.op == "placeholder":
                env[n.name] = next(it)
                continue
            a, kw = tfx.node.map_arg((n.args, n.kwargs), lambda x: env[x.name])
            if n.op == "output":
                return a[0]
            env[n.name] = getattr(interp, n.op)(n.target, a, kw)
            self.executed.append(n.name)
            if (i + 1) % self.frequency == 0 or n.name == stop_after:
                self.saved = {"env": dict(env), "at": n.name}
            if n.name == stop_after:
                return None
        return None


# ================================================================================================ memory
class MemoryAnalyzer:
    """Liveness of every value (from :class:`ShapeProp` metadata), peak live bytes, the largest values, and a greedy
    assignment of values to reusable buffers (a value may take a buffer whose previous tenant died before it is made)."""

    def __init__(self, gm: GraphModule):
        self.gm = gm

    def analyze(self, *example_inputs) -> dict:
        ShapeProp(self.gm).run(*example_inputs)
        nodes = list(self.gm.graph.nodes)
        pos = {n: i for i, n in enumerate(nodes)}
        size = {n: math.prod(n.meta["shape"]) * n.meta["dtype"].itemsize for n in nodes if "shape" in n.meta and n.op not in ("get_attr", "output")}
        last = {n: max([pos[u] for u in n.users], default=pos[n]) for n in size}
        live, peak, peak_at = 0, 0, None
        dying: dict[int, list] = {}
        for n in size:
            dying.setdefault(last[n], []).append(n)
        for i, n in enumerate(nodes):
            if n in size:
                live += size[n]
                if live > peak:
                    peak, peak_at = live, n.name
            live -= sum(size[d] for d in dying.get(i, []))
        # greedy reuse: free list of (bytes, buffer id); best fit
        free, buffers, assign = [], [], {}
        for i, n in enumerate(nodes):
            if n in size and n.op != "placeholder":
                fit = min((b for b in free if buffers[b] >= size[n]), key=lambda b: buffers[b], default=None)
                if fit is None:
                    buffers.append(size[n])
                    fit = len(buffers) - 1
                else:
                    free.remove(fit)
                assign[n.name] = fit
            for d in dying.get(i, []):
                if d.name in assign:
                    free.append(assign[d.name])
        total = sum(s for n, s in size.items() if n.op != "placeholder")
        hot = sorted(((s, n.name) for n, s in size.items()), reverse=True)[:5]
        return {"peak_bytes": peak, "peak_at": peak_at, "total_intermediate_bytes": total, "planned_bytes": sum(buffers),
                "buffers": len(buffers), "assignment": assign, "hotspots": [{"node": n, "bytes": s} for s, n in hot],
                "lifetimes": {n.name: (pos[n], last[n]) for n in size}}


# ================================================================================================ placement / backends
@dataclass
class DeviceCapability:
    name: str
    flops: float            # sustained FLOP/s
    bandwidth: float        # bytes/s of its own memory
    memory: float           # bytes
    link: float = 64e9      # bytes/s to other devices
    link_latency: float = 10e-6   # seconds per transfer
    launch: float = 2e-6    # seconds of fixed cost per operation


class HeterogeneousPlanner:
    """Assigns each compute node to the device that finishes it earliest (roofline time + cost of moving its inputs),
    in topological order; reports stages, transfers and the estimated makespan."""

    def __init__(self, devices: list[DeviceCapability]):
        self.devices = devices

    @staticmethod
    def _work(n, mods):
        out = math.prod(n.meta.get("shape", (1,)))
        byts = out * 4 + sum(math.prod(a.meta.get("shape", (1,))) * 4 for a in n.all_input_nodes)
        m = mods.get(n.target) if n.op == "call_module" else None
        if isinstance(m, nn.Linear):
            return 2.0 * out * m.in_features, byts + m.weight.numel() * 4
        if _tname(n.target) == "matmul" and len(n.all_input_nodes) == 2:
            return 2.0 * out * n.all_input_nodes[0].meta["shape"][-1], byts
        return float(out), byts

    def plan_execution(self, gm: GraphModule, *example_inputs, input_device: int = 0) -> dict:
        ShapeProp(gm).run(*example_inputs)
        mods = dict(gm.named_modules())
        where, ready, dev_free = {}, {}, [0.0] * len(self.devices)
        transfers, placement = [], {}
        for n in gm.graph.nodes:
            if n.op in ("placeholder", "get_attr"):
                where[n], ready[n] = (input_device if n.op == "placeholder" else None), 0.0
                continue
            if n.op == "output":
                continue
            flops, byts = self._work(n, mods)
            best = None
            for di, d in enumerate(self.devices):
                t_in = 0.0
                for a in n.all_input_nodes:
                    move = where[a] is not None and where[a] != di
                    t_in = max(t_in, ready[a] + (d.link_latency + math.prod(a.meta.get("shape", (1,))) * 4 / min(d.link, self.devices[where[a]].link) if move else 0.0))
                start = max(t_in, dev_free[di])
                end = start + d.launch + max(flops / d.flops, byts / d.bandwidth)
                if best is None or end < best[0]:
                    best = (end, di)
            end, di = best
            transfers += [{"value": a.name, "src": where[a], "dst": di} for a in n.all_input_nodes if where[a] is not None and where[a] != di]
            where[n], ready[n], dev_free[di], placement[n.name] = di, end, end, self.devices[di].name
        return {"placement": placement, "transfers": transfers, "makespan": max(dev_free), "device_busy_until": dev_free}


class BackendRegistry:
    """Named execution backends ``fn(gm, *inputs) -> outputs`` with declared capabilities; ``execute_with_auto_backend``
    takes the first registered backend that has every requested capability and falls back down the list on failure."""

    def __init__(self):
        self.backends: dict[str, dict] = {}
        self.register("eager", lambda gm, *a: gm(*a), {"cpu", "cuda", "autograd"})
        self.register("interpreter", lambda gm, *a: Interpreter(gm).run(*a), {"cpu", "cuda", "autograd", "debug"})
        self.register("generated-python", lambda gm, *a: PythonCodeGen().generate(gm).load()(*a), {"cpu", "cuda", "source"})

    def register(self, name, fn, capabilities=()): self.backends[name] = {"fn": fn, "capabilities": set(capabilities)}
    def unregister(self, name): self.backends.pop(name, None)
    def list_backends(self): return list(self.backends)
    def find_backends_with_capability(self, cap): return [k for k, v in self.backends.items() if cap in v["capabilities"]]
    def execute_with_backend(self, name, gm, *inputs): return self.backends[name]["fn"](gm, *inputs)

    def execute_with_auto_backend(self, gm, *inputs, require=()):
        errors = {}
        for name, b in self.backends.items():
            if set(require) <= b["capabilities"]:
                try:
                    return name, b["fn"](gm, *inputs)
                except Exception as e:                                        # next candidate
                    errors[name] = repr(e)
        raise RuntimeError(f"no backend could run the graph: {errors or 'none has ' + str(set(require))}")


class GraphCache:
    """Results keyed by graph structure and input fingerprints, with hit / miss counts and LRU eviction."""

    def __init__(self, capacity: int = 64):
        self.capacity, self.store, self.hits, self.misses = capacity, {}, 0, 0

    @staticmethod
    def _key(gm, inputs):
        h = hashlib.sha256(str(gm.graph).encode())
        for t in inputs:
            h.update(repr((tuple(t.shape), t.dtype)).encode() + t.detach().cpu().contiguous().numpy().tobytes())
        return h.hexdigest()

    def run(self, gm: GraphModule, *inputs):
        k = self._key(gm, inputs)
        if k in self.store:
            self.hits += 1
            self.store[k] = self.store.pop(k)
            return self.store[k]
        self.misses += 1
        self.store[k] = gm(*inputs)
        if len(self.store) > self.capacity:
            self.store.pop(next(iter(self.store)))
        return self.store[k]

    def statistics(self): return {"entries": len(self.store), "hits": self.hits, "misses": self.misses}


# ================================================================================================ quantisation passes
class _Observer(nn.Module):
    def __init__(self):
        super().__init__()
        self.register_buffer("lo", torch.tensor(math.inf))
        self.register_buffer("hi", torch.tensor(-math.inf))

    def forward(self, x):
        self.lo, self.hi = torch.minimum(self.lo, x.detach().min()), torch.maximum(self.hi, x.detach().max())
        return x


class _FakeQuant(nn.Module):
    """Affine 8-bit quantise / dequantise with a straight-through gradient; the range is fixed (PTQ) or learned (QAT)."""

    def __init__(self, lo: float, hi: float, bits: int = 8, learn: bool = False):
        super().__init__()
        lo, hi = min(lo, 0.0), max(hi, 0.0)
        self.levels = 2 ** bits - 1
        r = torch.tensor([lo, hi], dtype=torch.float32)
        self.range = nn.Parameter(r) if learn else nn.Buffer(r)

    def forward(self, x):
        lo, hi = self.range[0], self.range[1]
        scale = (hi - lo).clamp(min=1e-12) / self.levels
        q = torch.clamp((x - lo) / scale, 0, self.levels)
        q = q + (q.round() - q).detach()
        return q * scale + lo


def prepare_ptq(gm: GraphModule) -> GraphModule:
    """Inserts a range observer after every placeholder and compute node."""
    gm = copy.deepcopy(gm)
    for i, n in enumerate(list(gm.graph.nodes)):
        if n.op in ("output", "get_attr"):
            continue
        name = f"_obs_{i}"
        gm.add_module(name, _Observer())
        with gm.graph.inserting_after(n):
            o = gm.graph.call_module(name, (n,))
        n.replace_all_uses_with(o, delete_user_cb=lambda u: u is not o)
    gm.recompile()
    return gm


def convert_ptq(gm: GraphModule, bits: int = 8, learn: bool = False) -> GraphModule:
    """Turns calibrated observers into fake-quantisation nodes and quantises Linear / Conv weights per output channel."""
    gm = copy.deepcopy(gm)
    for name, m in list(gm.named_modules()):
        if isinstance(m, _Observer):
            if not math.isfinite(float(m.lo)):
                raise RuntimeError("observer saw no data: run calibration batches through the prepared module first")
            setattr(gm, name, _FakeQuant(float(m.lo), float(m.hi), bits, learn))
        elif isinstance(m, (nn.Linear, nn.Conv2d)) and not learn:
            w = m.weight.data
            s = w.abs().flatten(1).amax(1).clamp(min=1e-12) / (2 ** (bits - 1) - 1)
            shape = (-1,) + (1,) * (w.dim() - 1)
            m.weight.data = (w / s.reshape(shape)).round().clamp(-(2 ** (bits - 1)), 2 ** (bits - 1) - 1) * s.reshape(shape)
    gm.recompile()
    return gm


def prepare_qat(gm: GraphModule, *calibration_inputs, bits: int = 8) -> GraphModule:
    """Calibrates once, then inserts fake-quant nodes whose ranges train with the weights."""
    p = prepare_ptq(gm)
    with torch.no_grad():
        p(*calibration_inputs)
    return convert_ptq(p, bits, learn=True)


def quantization_error(ref: GraphModule, quant: GraphModule, *inputs) -> dict:
    with torch.no_grad():
        a, b = ref(*inputs), quant(*inputs)
    err = (a - b).float()
    return {"mse": float(err.pow(2).mean()), "max_abs": float(err.abs().max()),
            "sqnr_db": float(10 * torch.log10(a.float().pow(2).mean() / err.pow(2).mean().clamp(min=1e-30)))}


# ================================================================================================ architecture search
_NAS_OPS = {"identity": lambda d: nn.Identity(), "linear": lambda d: nn.Linear(d, d),
            "linear_relu": lambda d: nn.Sequential(nn.Linear(d, d), nn.ReLU()), "linear_tanh": lambda d: nn.Sequential(nn.Linear(d, d), nn.Tanh()),
            "bottleneck": lambda d: nn.Sequential(nn.Linear(d, max(d // 4, 1)), nn.ReLU(), nn.Linear(max(d // 4, 1), d)),
            "zero": lambda d: _Zero()}


class _Zero(nn.Module):
    def forward(self, x): return torch.zeros_like(x)


class _Cell(nn.Module):
    def __init__(self, genes, dim, din, dout):
        super().__init__()
        self.stem, self.head = nn.Linear(din, dim), nn.Linear(dim, dout)
        self.ops = nn.ModuleList(_NAS_OPS[g["op"]](dim) for g in genes)
        self.skip = [g["skip"] for g in genes]

    def forward(self, x):
        h = self.stem(x)
        for op, skip in zip(self.ops, self.skip):
            h = op(h) + h if skip else op(h)
        return self.head(h)


class ArchitectureSearch:
    """Evolutionary search (tournament selection, mutation, crossover) over chains of ``depth`` cells, each an operation
    from the op set with an optional skip connection.  Fitness = validation loss after a short training run, plus
    ``param_penalty`` per parameter."""

    def __init__(self, din: int, dout: int, dim: int = 16, depth: int = 3, ops=None, seed: int = 0, param_penalty: float = 0.0):
        self.din, self.dout, self.dim, self.depth = din, dout, dim, depth
        self.ops, self.gen, self.penalty = list(ops or _NAS_OPS), torch.Generator().manual_seed(seed), param_penalty
        self.history: list = []

    def _rand(self, n): return int(torch.randint(0, n, (1,), generator=self.gen))
    def random_architecture(self): return [{"op": self.ops[self._rand(len(self.ops))], "skip": bool(self._rand(2))} for _ in range(self.depth)]
    def build(self, genes): return _Cell(genes, self.dim, self.din, self.dout)

    def mutate(self, genes):
        g = copy.deepcopy(genes)
        i = self._rand(len(g))
        if self._rand(2):
            g[i]["op"] = self.ops[self._rand(len(self.ops))]
        else:
            g[i]["skip"] = not g[i]["skip"]
        return g

    def crossover(self, a, b):
        cut = 1 + self._rand(max(len(a) - 1, 1))
        return copy.deepcopy(a[:cut] + b[cut:])

    def evaluate(self, genes, train, val, steps: int = 60, lr: float = 0.02) -> float:
        torch.manual_seed(0)
        m = self.build(genes)
        opt = torch.optim.Adam(m.parameters(), lr)
        for _ in range(steps):
            loss = F.mse_loss(m(train[0]), train[1])
            opt.zero_grad(); loss.backward(); opt.step()
        with torch.no_grad():
            return float(F.mse_loss(m(val[0]), val[1])) + self.penalty * sum(p.numel() for p in m.parameters())

    def search(self, train, val, population: int = 8, generations: int = 4, steps: int = 60):
        pop = [self.random_architecture() for _ in range(population)]
        fit = [self.evaluate(g, train, val, steps) for g in pop]
        for gen in range(generations):
            self.history.append(min(fit))
            children = []
            while len(children) < population // 2:
                pick = lambda: min((self._rand(population) for _ in range(3)), key=lambda i: fit[i])
                child = self.mutate(self.crossover(pop[pick()], pop[pick()]))
                children.append(child)
            cf = [self.evaluate(c, train, val, steps) for c in children]
            merged = sorted(zip(fit + cf, range(len(pop) + len(children))), key=lambda t: t[0])[:population]
            allp = pop + children
            pop, fit = [allp[i] for _, i in merged], [f for f, _ in merged]
        self.history.append(min(fit))
        return pop[0], fit[0]
