"""A small compiler over traced graphs: lowering to an explicit IR with shapes and dtypes, constant evaluation and dead
code elimination, fusion of element-wise regions into generated CUDA kernels (``core.kernel_gen``), shape-specialised
compilation caches with tiered (interpret first, compile when hot) execution and profile counters, a stepping debugger with
breakpoints and value inspection, diagnostics that point at the traced source line, DOT / text visualisation, and a registry
for custom operators (lowering rule + evaluator, optionally an element-wise code template).

The reference's JIT crate names these subsystems (crates/torsh-jit/src/{ir,lowering,type_inference,const_eval,fusion,
optimizer,specialization,adaptive_compilation,pgo,debugger,error_diagnostics,trace_viz,custom_ops,plugin_system,runtime}.rs)
and generates Cranelift IR for the CPU; here the generated code is CUDA for ``sm_100a`` and the fallback is PyTorch.
"""
from __future__ import annotations

import operator
import time
from dataclasses import dataclass, field

import torch
import torch.fx

from .core import kernel_gen as kg

# ---- IR --------------------------------------------------------------------------------------------------------------
_EW_UNARY = {torch.relu: "relu", torch.nn.functional.relu: "relu", torch.tanh: "tanh", torch.sigmoid: "sigmoid", torch.exp: "exp",
             torch.log: "log", torch.sqrt: "sqrt", torch.rsqrt: "rsqrt", torch.abs: "abs", operator.neg: "neg", torch.neg: "neg",
             torch.nn.functional.silu: "silu", torch.square: "square", torch.reciprocal: "reciprocal"}
_EW_BINARY = {operator.add: "add", torch.add: "add", operator.sub: "sub", torch.sub: "sub", operator.mul: "mul", torch.mul: "mul",
              operator.truediv: "div", torch.div: "div", torch.maximum: "max", torch.minimum: "min", operator.pow: "pow", torch.pow: "pow"}
_EW_METHODS = {"relu": "relu", "tanh": "tanh", "sigmoid": "sigmoid", "exp": "exp", "log": "log", "sqrt": "sqrt", "abs": "abs", "neg": "neg",
               "add": "add", "sub": "sub", "mul": "mul", "div": "div", "pow": "pow"}
_EW_MODULES = {torch.nn.ReLU: "relu", torch.nn.Tanh: "tanh", torch.nn.Sigmoid: "sigmoid", torch.nn.SiLU: "silu"}


@dataclass
class IRNode:
    id: int
    op: str                      # "input", "const", "ew:<name>", "call", "fused", "output"
    inputs: list = field(default_factory=list)   # IRNode ids or Python scalars
    target: object = None        # callable for "call", Expr builder info for "fused"
    kwargs: dict = field(default_factory=dict)
    shape: tuple | None = None
    dtype: torch.dtype | None = None
    value: object = None         # constants
    name: str = ""
    source: str = ""             # file:line of the traced statement


class CompileError(Exception):
    """Carries the IR node and the traced source location of the failing operation."""

    def __init__(self, message: str, node: IRNode | None = None):
        where = f" (node %{node.id} {node.op} '{node.name}'" + (f", traced at {node.source}" if node and node.source else "") + ")" if node else ""
        super().__init__(message + where)
        self.node = node


class IRGraph:
    def __init__(self):
        self.nodes: list[IRNode] = []
        self.outputs: list[int] = []

    def add(self, op, inputs=(), **kw) -> IRNode:
        n = IRNode(len(self.nodes), op, list(inputs), **kw)
        self.nodes.append(n)
        return n

    def users(self) -> dict:
        u: dict[int, list[int]] = {n.id: [] for n in self.nodes}
        for n in self.nodes:
            for i in n.inputs:
                if isinstance(i, _Ref):
                    u[i.id].append(n.id)
        return u

    def to_text(self) -> str:
        lines = []
        for n in self.nodes:
            ins = ", ".join(f"%{i.id}" if isinstance(i, _Ref) else repr(i) for i in n.inputs)
            ty = f" : {str(n.dtype).replace('torch.', '')}{list(n.shape)}" if n.shape is not None else ""
            extra = f" [{n.target.key()}]" if n.op == "fused" else (f" [{getattr(n.target, '__name__', n.target)}]" if n.op == "call" else "")
            lines.append(f"%{n.id} = {n.op}({ins}){extra}{ty}")
        lines.append("return " + ", ".join(f"%{o}" for o in self.outputs))
        return "\n".join(lines)

    def to_dot(self) -> str:
        out = ["digraph ir {", "  rankdir=TB;"]
        for n in self.nodes:
            color = {"fused": "lightblue", "input": "lightgrey", "const": "khaki"}.get(n.op.split(":")[0], "white")
            out.append(f'  n{n.id} [label="%{n.id} {n.op}\\n{list(n.shape) if n.shape is not None else ""}", style=filled, fillcolor={color}];')
            out += [f"  n{i.id} -> n{n.id};" for i in n.inputs if isinstance(i, _Ref)]
        return "\n".join(out + ["}"])


@dataclass(frozen=True)
class _Ref:
    id: int


# ---- custom operators / plugins --------------------------------------------------------------------------------------
@dataclass
class CustomOp:
    name: str
    evaluate: object                    # callable(*tensors, **kwargs) -> tensor
    match: object = None                # callable(fx_node) -> bool : which traced calls lower to this op
    elementwise_expr: object = None     # callable(*Expr) -> Expr : lets the op join fused regions


class OpRegistry:
    def __init__(self):
        self.ops: dict[str, CustomOp] = {}
        self.passes: list = []              # plugin passes: callable(IRGraph) -> int

    def register_op(self, op: CustomOp):
        self.ops[op.name] = op
        return op

    def register_pass(self, fn):
        self.passes.append(fn)
        return fn


registry = OpRegistry()


class SourceTracer(torch.fx.Tracer):
    """fx tracer that records, for every node, the user frame (file and line) that created it."""

    def __init__(self):
        super().__init__()
        self.record_stack_traces = True

    def _filter_traceback_frames(self, user_stack_summary):
        import traceback
        here = __file__
        keep = [f for f in user_stack_summary if "/torch/" not in f.filename and f.filename != here and "importlib" not in f.filename]
        return traceback.StackSummary.from_list(keep[-1:])


def trace_with_source(fn) -> torch.fx.GraphModule:
    tracer = SourceTracer()
    graph = tracer.trace(fn)
    root = fn if isinstance(fn, torch.nn.Module) else tracer.root
    return torch.fx.GraphModule(root, graph)


# ---- lowering + type inference ---------------------------------------------------------------------------------------
def lower_fx(gm: torch.fx.GraphModule, example_inputs) -> IRGraph:
    """fx graph -> IR, with shapes / dtypes from one propagation of the example inputs."""
    from torch.fx.passes.shape_prop import ShapeProp
    ShapeProp(gm).propagate(*example_inputs)
    g, env = IRGraph(), {}
    mods = dict(gm.named_modules())

    def ref(a):
        if isinstance(a, torch.fx.Node):
            return _Ref(env[a].id)
        if isinstance(a, (int, float, bool)):
            return a
        raise CompileError(f"unsupported argument {a!r}")

    def meta(fx_node, n: IRNode):
        tm = fx_node.meta.get("tensor_meta")
        if hasattr(tm, "shape"):
            n.shape, n.dtype = tuple(tm.shape), tm.dtype
        n.name = fx_node.name
        st = fx_node.stack_trace or ""
        lines = [l.strip() for l in st.splitlines() if l.strip().startswith("File")]
        if lines:
            n.source = lines[-1].replace('File "', "").replace('", line ', ":").split(",")[0]

    for fn_ in gm.graph.nodes:
        if fn_.op == "placeholder":
            n = g.add("input")
        elif fn_.op == "get_attr":
            obj = gm
            for part in fn_.target.split("."):
                obj = getattr(obj, part)
            n = g.add("const", value=obj)
        elif fn_.op == "output":
            outs = fn_.args[0] if isinstance(fn_.args[0], (tuple, list)) else [fn_.args[0]]
            g.outputs = [env[o].id for o in outs]
            continue
        else:
            custom = next((c for c in registry.ops.values() if c.match is not None and c.match(fn_)), None)
            name = None
            if custom is None:
                if fn_.op == "call_function":
                    name = _EW_UNARY.get(fn_.target) or _EW_BINARY.get(fn_.target)
                elif fn_.op == "call_method":
                    name = _EW_METHODS.get(fn_.target)
                elif fn_.op == "call_module":
                    name = _EW_MODULES.get(type(mods[fn_.target]))
            if custom is not None:
                n = g.add(f"custom:{custom.name}", [ref(a) for a in fn_.args], kwargs=dict(fn_.kwargs))
            elif name is not None and not fn_.kwargs:
                n = g.add(f"ew:{name}", [ref(a) for a in fn_.args])
            else:
                if fn_.op == "call_module":
                    target = mods[fn_.target]
                elif fn_.op == "call_method":
                    target = (lambda meth: (lambda self_, *a, **k: getattr(self_, meth)(*a, **k)))(fn_.target)
                    target.__name__ = fn_.target
                else:
                    target = fn_.target
                try:
                    args = [ref(a) if not isinstance(a, (tuple, list)) else a for a in fn_.args]
                except CompileError:
                    args = list(fn_.args)
                n = g.add("call", args, target=target, kwargs=dict(fn_.kwargs))
                n.raw_args = fn_.args
                n.env_map = env
        meta(fn_, n)
        env[fn_] = n
    return g


# ---- passes ----------------------------------------------------------------------------------------------------------
def dead_code_elimination(g: IRGraph) -> int:
    live, stack = set(g.outputs), list(g.outputs)
    by_id = {n.id: n for n in g.nodes}
    while stack:
        for i in _deps(by_id[stack.pop()]):
            if i not in live:
                live.add(i)
                stack.append(i)
    before = len(g.nodes)
    g.nodes = [n for n in g.nodes if n.id in live or n.op == "input"]
    return before - len(g.nodes)


def _deps(n: IRNode):
    out = [i.id for i in n.inputs if isinstance(i, _Ref)]
    if n.op == "call":
        def walk(a):
            if isinstance(a, torch.fx.Node):
                out.append(n.env_map[a].id)
            elif isinstance(a, (tuple, list)):
                for x in a:
                    walk(x)
        walk(getattr(n, "raw_args", ()))
    return out


def constant_evaluation(g: IRGraph) -> int:
    """Element-wise nodes whose inputs are all constants / scalars are evaluated now."""
    by_id, folded = {n.id: n for n in g.nodes}, 0
    for n in g.nodes:
        if not n.op.startswith("ew:"):
            continue
        ins = [by_id[i.id] if isinstance(i, _Ref) else i for i in n.inputs]
        if all(not isinstance(i, IRNode) or i.op == "const" for i in ins) and any(isinstance(i, IRNode) for i in ins):
            vals = [i.value if isinstance(i, IRNode) else i for i in ins]
            n.value, n.op, n.inputs = _eval_ew(n.op[3:], vals), "const", []
            folded += 1
    return folded


def _eval_ew(name, vals):
    table = kg._UNARY if name in kg._UNARY else kg._BINARY
    vals = [v if isinstance(v, torch.Tensor) else torch.tensor(float(v)) for v in vals]
    return table[name][1](*vals)


def fuse_elementwise(g: IRGraph, min_ops: int = 2) -> int:
    """Greedy fusion: an element-wise node is merged into its consumer region when it has exactly one user, that user is
    element-wise (or already fused) and all tensors involved have the same shape. Each region becomes one ``fused`` node
    holding a ``kernel_gen`` expression over the region's external inputs."""
    users = g.users()
    by_id = {n.id: n for n in g.nodes}
    is_ew = lambda n: n.op.startswith("ew:") or (n.op.startswith("custom:") and registry.ops[n.op[7:]].elementwise_expr is not None)
    roots = [n for n in g.nodes if is_ew(n) and not (len(users[n.id]) == 1 and is_ew(by_id[users[n.id][0]]) and by_id[users[n.id][0]].shape == n.shape
                                                      and n.id not in g.outputs)]
    fused = 0
    for root in roots:
        ext: list[int] = []
        count = [0]

        def build(n: IRNode):
            count[0] += 1
            args = []
            for i in n.inputs:
                if not isinstance(i, _Ref):
                    args.append(kg.Expr._wrap(i))
                    continue
                m = by_id[i.id]
                inside = is_ew(m) and len(users[m.id]) == 1 and m.shape == root.shape and m.id not in g.outputs
                if inside:
                    args.append(build(m))
                elif m.op == "const" and isinstance(m.value, torch.Tensor) and m.value.numel() == 1:
                    args.append(kg.Expr._wrap(float(m.value)))
                else:
                    if m.shape != root.shape:
                        raise _NoFuse()
                    if m.id not in ext:
                        ext.append(m.id)
                    args.append(kg.Expr("input", (), ext.index(m.id)))
            if n.op.startswith("custom:"):
                return registry.ops[n.op[7:]].elementwise_expr(*args)
            return kg.Expr(n.op[3:], tuple(args))
        try:
            expr = build(root)
        except _NoFuse:
            continue
        if count[0] < min_ops or not ext:
            continue
        root.op, root.target, root.inputs = "fused", expr, [_Ref(i) for i in ext]
        root.fused_ops = count[0]
        fused += 1
    dead_code_elimination(g)
    return fused


class _NoFuse(Exception):
    pass


# ---- runtime + debugger ----------------------------------------------------------------------------------------------
class Executable:
    """Evaluates an IR graph. Fused nodes run as generated kernels on CUDA tensors (``kernel_gen.FusedElementwise``) and as
    the same expression in PyTorch elsewhere."""

    def __init__(self, g: IRGraph):
        self.g = g
        self._kernels: dict[int, kg.FusedElementwise] = {}
        self.node_time_s: dict[int, float] = {}
        self.profile = False

    def _run_node(self, n: IRNode, env: dict):
        get = lambda i: env[i.id] if isinstance(i, _Ref) else i
        if n.op == "const":
            return n.value
        if n.op.startswith("ew:"):
            vals = [get(i) for i in n.inputs]
            table = kg._UNARY if n.op[3:] in kg._UNARY else kg._BINARY
            ref_t = next(v for v in vals if isinstance(v, torch.Tensor))
            vals = [v if isinstance(v, torch.Tensor) else torch.tensor(v, dtype=ref_t.dtype, device=ref_t.device) for v in vals]
            return table[n.op[3:]][1](*vals)
        if n.op == "fused":
            xs = [get(i) for i in n.inputs]
            k = self._kernels.get(n.id)
            if k is None:
                k = kg.FusedElementwise.__new__(kg.FusedElementwise)
                k.expr, k.n_inputs, k.tune, k._libs = n.target, len(xs), True, {}
                self._kernels[n.id] = k
            return k(*xs)
        if n.op.startswith("custom:"):
            return registry.ops[n.op[7:]].evaluate(*[get(i) for i in n.inputs], **n.kwargs)
        if n.op == "call":
            def conv(a):
                if isinstance(a, torch.fx.Node):
                    return env[n.env_map[a].id]
                if isinstance(a, _Ref):
                    return env[a.id]
                if isinstance(a, (tuple, list)):
                    return type(a)(conv(x) for x in a)
                return a
            args = [conv(a) for a in getattr(n, "raw_args", n.inputs)]
            kwargs = {k: conv(v) for k, v in n.kwargs.items()}
            try:
                return n.target(*args, **kwargs)
            except Exception as e:
                raise CompileError(f"{type(e).__name__} while executing: {e}", n) from e
        raise CompileError(f"cannot execute op {n.op}", n)

    def __call__(self, *inputs, hook=None):
        env, k = {}, 0
        for n in self.g.nodes:
            if n.op == "input":
                env[n.id] = inputs[k]
                k += 1
                continue
            t0 = time.perf_counter() if self.profile else 0.0
            env[n.id] = self._run_node(n, env)
            if self.profile:
                self.node_time_s[n.id] = self.node_time_s.get(n.id, 0.0) + time.perf_counter() - t0
            if hook is not None:
                hook(n, env[n.id])
        outs = [env[o] for o in self.g.outputs]
        return outs[0] if len(outs) == 1 else tuple(outs)


class Debugger:
    """Steps through an executable node by node: ``breakpoints`` hold node ids or op-name substrings; ``run`` returns at
    each hit with the node and its value, ``watch`` collects per-node statistics (NaN / Inf counts, min, max)."""

    def __init__(self, exe: Executable):
        self.exe, self.breakpoints, self.hits, self.stats = exe, set(), [], {}

    def add_breakpoint(self, where):
        self.breakpoints.add(where)

    def run(self, *inputs, watch: bool = True):
        self.hits, self.stats = [], {}

        def hook(n, v):
            if watch and isinstance(v, torch.Tensor) and v.is_floating_point() and v.numel():
                f = v.detach().float()
                self.stats[n.id] = {"op": n.op, "nan": int(torch.isnan(f).sum()), "inf": int(torch.isinf(f).sum()),
                                    "min": float(f[torch.isfinite(f)].min()) if torch.isfinite(f).any() else float("nan"),
                                    "max": float(f[torch.isfinite(f)].max()) if torch.isfinite(f).any() else float("nan")}
            if n.id in self.breakpoints or any(isinstance(b, str) and b in n.op for b in self.breakpoints):
                self.hits.append((n.id, n.op, v.detach().clone() if isinstance(v, torch.Tensor) else v))
        out = self.exe(*inputs, hook=hook)
        return out

    def first_bad_node(self):
        """The first node whose value contains NaN / Inf, with its source location (for "where did the NaN start")."""
        for nid in sorted(self.stats):
            s = self.stats[nid]
            if s["nan"] or s["inf"]:
                n = next(x for x in self.exe.g.nodes if x.id == nid)
                return {"node": nid, "op": n.op, "source": n.source, **s}
        return None


# ---- tiered, specialised compilation -----------------------------------------------------------------------------------
@dataclass
class CompileStats:
    calls: int = 0
    interpreted: int = 0
    compiled_calls: int = 0
    specializations: int = 0
    fused_regions: int = 0
    ops_fused: int = 0
    compile_time_s: float = 0.0


class JitFunction:
    """``jit(fn)``: the first ``hot_threshold`` calls per input signature run the original callable (and count); then the
    function is traced, lowered, optimised and executed from the IR. Signatures = shapes + dtypes + devices of the tensor
    arguments, so each shape gets code specialised to it (constants folded, fusion decided on real shapes)."""

    def __init__(self, fn, hot_threshold: int = 2, fuse: bool = True, max_specializations: int = 8):
        self.fn, self.hot, self.fuse, self.max_spec = fn, hot_threshold, fuse, max_specializations
        self.counts: dict = {}
        self.cache: dict = {}
        self.stats = CompileStats()
        self.errors: list[str] = []

    @staticmethod
    def signature(args) -> tuple:
        return tuple((tuple(a.shape), a.dtype, a.device.type) if isinstance(a, torch.Tensor) else ("py", type(a).__name__, a) for a in args)

    def compile(self, *example) -> Executable:
        t0 = time.perf_counter()
        gm = trace_with_source(self.fn)
        g = lower_fx(gm, example)
        constant_evaluation(g)
        dead_code_elimination(g)
        if self.fuse:
            self.stats.fused_regions += fuse_elementwise(g)
            self.stats.ops_fused += sum(getattr(n, "fused_ops", 0) for n in g.nodes)
        for p in registry.passes:
            p(g)
        self.stats.compile_time_s += time.perf_counter() - t0
        return Executable(g)

    def __call__(self, *args):
        self.stats.calls += 1
        sig = self.signature(args)
        exe = self.cache.get(sig)
        if exe is None:
            c = self.counts[sig] = self.counts.get(sig, 0) + 1
            if c <= self.hot or len(self.cache) >= self.max_spec or sig in self.errors:
                self.stats.interpreted += 1
                return self.fn(*args)
            try:
                exe = self.cache[sig] = self.compile(*args)
                self.stats.specializations += 1
            except Exception as e:          # tracing can fail on data-dependent control flow: stay on the original
                self.errors.append(sig)
                self.last_error = e
                self.stats.interpreted += 1
                return self.fn(*args)
        self.stats.compiled_calls += 1
        return exe(*args)

    def graph_for(self, *args) -> IRGraph | None:
        e = self.cache.get(self.signature(args))
        return e.g if e else None


def jit(fn=None, **kw):
    return JitFunction(fn, **kw) if fn is not None else (lambda f: JitFunction(f, **kw))
