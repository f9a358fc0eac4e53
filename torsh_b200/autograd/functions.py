"""Custom-function registry and profile flame graphs (``crates/torsh-autograd/src/function.rs:19-341``,
``flamegraph.rs``).  Functions are ``torch.autograd.Function`` subclasses or plain forward/backward pairs registered by
name; ``compose`` chains registered functions.  ``folded_stacks`` turns profiler events into the
``frame;frame;frame value`` lines that flame-graph tools read, ``differential`` compares two such profiles."""
from __future__ import annotations

from collections import defaultdict

import torch


class FunctionRegistry:
    def __init__(self):
        self._fns: dict[str, type] = {}

    def register(self, name: str, forward=None, backward=None, function: type | None = None):
        """Register an autograd Function class, or build one from ``forward(ctx, *a)`` / ``backward(ctx, *g)``."""
        if function is None:
            if forward is None or backward is None:
                raise ValueError("give either function= or both forward= and backward=")
            function = type(name, (torch.autograd.Function,), {"forward": staticmethod(forward), "backward": staticmethod(backward)})
        if name in self._fns:
            raise KeyError(f"function {name!r} is already registered")
        self._fns[name] = function
        return function

    def get(self, name: str):
        if name not in self._fns:
            raise KeyError(f"unknown function {name!r}; registered: {sorted(self._fns)}")
        return self._fns[name]

    def apply(self, name: str, *args):
        return self.get(name).apply(*args)

    def names(self) -> list[str]: return sorted(self._fns)
    def unregister(self, name: str) -> None: self._fns.pop(name)

    def compose(self, *names: str):
        fns = [self.get(n) for n in names]

        def run(x):
            for f in fns:
                x = f.apply(x)
            return x
        return run


registry = FunctionRegistry()


def folded_stacks(events, value: str = "duration_us") -> list[str]:
    """``events``: objects / dicts with ``name``, ``category``, ``start_us``, ``duration_us`` (profiler events).
    Nesting is recovered from time containment per thread."""
    get = (lambda e, k: e[k]) if events and isinstance(events[0], dict) else getattr
    by_thread = defaultdict(list)
    for e in events:
        by_thread[get(e, "thread_id") if (isinstance(e, dict) and "thread_id" in e) or hasattr(e, "thread_id") else 0].append(e)
    acc: dict[str, float] = defaultdict(float)
    for evs in by_thread.values():
        evs = sorted(evs, key=lambda e: (get(e, "start_us"), -get(e, "duration_us")))
        stack: list = []
        for e in evs:
            while stack and get(e, "start_us") >= get(stack[-1], "start_us") + get(stack[-1], "duration_us"):
                stack.pop()
            if stack:   # self time of the parent shrinks by the child's time
                acc[";".join(get(s, "name") for s in stack)] -= get(e, value)
            stack.append(e)
            acc[";".join(get(s, "name") for s in stack)] += get(e, value)
    return [f"{k} {max(int(round(v)), 0)}" for k, v in sorted(acc.items())]


def differential(before: list[str], after: list[str]) -> list[tuple[str, int, int]]:
    """``(stack, before, after)`` sorted by absolute change."""
    parse = lambda lines: {l.rsplit(" ", 1)[0]: int(l.rsplit(" ", 1)[1]) for l in lines}
    a, b = parse(before), parse(after)
    keys = set(a) | set(b)
    return sorted(((k, a.get(k, 0), b.get(k, 0)) for k in keys), key=lambda t: -abs(t[2] - t[1]))
