"""Compilation entry points (``crates/torsh-jit``).  The reference lowers a traced graph to Cranelift and its CUDA
generator returns "not implemented" (``crates/torsh-jit/src/codegen.rs:446-535``).  Here "compiling" a callable means:
trace it, run the fusion passes of :mod:`torsh_b200.fx` (``FusionStrategy`` picks which), and — on a GPU — capture the
result in a CUDA graph per input signature so a launch-bound model replays as one graph launch.

``trace(fn, example)`` / ``script(module)`` return a :class:`CompiledFunction`; ``GraphCache`` is the (shape, dtype)
keyed cache of captured graphs."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

import torch


class FusionStrategy(enum.Enum):
    NONE = "none"
    CONSERVATIVE = "conservative"   # CSE + DCE only
    DEFAULT = "default"             # + operator fusion
    AGGRESSIVE = "aggressive"       # + constant folding, repeated to a fixed point


@dataclass
class JitConfig:
    fusion: FusionStrategy = FusionStrategy.DEFAULT
    cuda_graphs: bool = True
    warmup: int = 2
    max_cached_graphs: int = 16


@dataclass
class _Captured:
    graph: "torch.cuda.CUDAGraph"
    inputs: list[torch.Tensor]
    output: object


@dataclass
class GraphCache:
    capacity: int = 16
    entries: dict = field(default_factory=dict)
    hits: int = 0
    misses: int = 0

    def get(self, key):
        e = self.entries.get(key)
        if e is None:
            self.misses += 1
        else:
            self.hits += 1
            self.entries[key] = self.entries.pop(key)   # most recently used last
        return e

    def put(self, key, value):
        if len(self.entries) >= self.capacity:
            self.entries.pop(next(iter(self.entries)))
        self.entries[key] = value


class CompiledFunction:
    def __init__(self, fn, config: JitConfig | None = None, graph_module=None, stats=None):
        self.fn, self.config = fn, config or JitConfig()
        self.graph_module, self.stats = graph_module, stats or {}
        self.cache = GraphCache(self.config.max_cached_graphs)

    @staticmethod
    def _sig(args):
        return tuple((tuple(a.shape), a.dtype, a.device.index) if isinstance(a, torch.Tensor) else ("py", a) for a in args)

    def __call__(self, *args):
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        use_graph = (self.config.cuda_graphs and tensors and all(t.is_cuda for t in tensors)
                     and not torch.is_grad_enabled() and not torch.cuda.is_current_stream_capturing())
        if not use_graph:
            return self.fn(*args)
        key = self._sig(args)
        cap = self.cache.get(key)
        if cap is None:
            static = [a.clone() if isinstance(a, torch.Tensor) else a for a in args]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(self.config.warmup):
                    self.fn(*static)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self.fn(*static)
            cap = _Captured(g, [a for a in static if isinstance(a, torch.Tensor)], out)
            self.cache.put(key, cap)
        for dst, src in zip(cap.inputs, tensors):
            dst.copy_(src)
        cap.graph.replay()
        return cap.output


def _optimise(gm, strategy: FusionStrategy) -> dict:
    from . import fx
    if strategy is FusionStrategy.NONE:
        return {}
    pm = fx.PassManager([("cse", fx.common_subexpression_elimination), ("dce", fx.dead_code_elimination)])
    if strategy in (FusionStrategy.DEFAULT, FusionStrategy.AGGRESSIVE):
        pm.passes.insert(1, ("fusion", fx.operator_fusion))
    if strategy is FusionStrategy.AGGRESSIVE:
        pm.passes.insert(0, ("constant_folding", fx.constant_folding))
    return pm.run(gm, max_rounds=4 if strategy is FusionStrategy.AGGRESSIVE else 1)


def script(module: torch.nn.Module, config: JitConfig | None = None) -> CompiledFunction:
    """Trace symbolically (falls back to the eager module when control flow defeats tracing) and optimise."""
    from . import fx
    config = config or JitConfig()
    try:
        gm = fx.symbolic_trace(module)
    except Exception:
        return CompiledFunction(module, config)
    return CompiledFunction(gm, config, gm, _optimise(gm, config.fusion))


def trace(fn, example_inputs=None, config: JitConfig | None = None) -> CompiledFunction:
    """``trace(fn, example)``: same as :func:`script` for modules; plain callables are wrapped for graph replay."""
    if isinstance(fn, torch.nn.Module):
        return script(fn, config)
    return CompiledFunction(fn, config)


def compile(fn, **kw) -> CompiledFunction:  # noqa: A001 - mirrors the reference's entry-point name
    return trace(fn, config=JitConfig(**kw) if kw else None)
