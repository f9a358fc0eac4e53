"""Compute-side multi-stream orchestrator: a DAG of tasks with cost estimates is mapped onto a few CUDA streams by a
list scheduler and issued with the minimum of cross-stream events.

Policies (the reference's "intelligent scheduler" variants, crates/torsh-backend/src/cuda/{stream_advanced.rs,
intelligent_scheduler.rs, multi_stream_orchestrator.rs}):

* ``round_robin``    - task i goes to stream i mod K
* ``least_loaded``   - the stream whose queued work finishes first
* ``critical_path``  - tasks are ranked by the length of the longest cost path to a sink (upward rank, as in HEFT);
  the highest rank is placed first, on the stream where it can START earliest given where its predecessors ran
  (a predecessor on the same stream costs no event)

Streams are anything with the ``torch.cuda.Stream`` interface; events come from ``event_coordination`` (CUDA events on
a GPU, host events otherwise), so plans and issue order are testable without a device.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .event_coordination import OperationCoordinator, _new_event


@dataclass
class Task:
    name: str
    fn: object = None
    cost: float = 1.0                      # estimated device time, any unit
    deps: tuple = ()
    priority: int = 0                      # higher first among equal ranks


@dataclass
class Plan:
    assignment: dict = field(default_factory=dict)      # task -> stream index
    order: list = field(default_factory=list)           # issue order
    start: dict = field(default_factory=dict)           # estimated start time per task
    makespan: float = 0.0
    cross_stream_edges: int = 0


class MultiStreamOrchestrator:
    def __init__(self, streams, policy: str = "critical_path", event_factory=_new_event):
        if policy not in ("round_robin", "least_loaded", "critical_path"):
            raise ValueError(f"unknown policy {policy!r}")
        self.streams, self.policy, self._event_factory = list(streams), policy, event_factory
        self.tasks: dict[str, Task] = {}

    def add(self, name: str, fn=None, cost: float = 1.0, deps=(), priority: int = 0) -> "MultiStreamOrchestrator":
        if name in self.tasks:
            raise ValueError(f"task {name!r} already added")
        for d in deps:
            if d not in self.tasks:
                raise KeyError(f"{name!r} depends on unknown task {d!r}")
        self.tasks[name] = Task(name, fn, float(cost), tuple(deps), priority)
        return self

    # ---- planning ---------------------------------------------------------------------------------------------
    def _upward_rank(self) -> dict:
        succ: dict[str, list[str]] = {n: [] for n in self.tasks}
        for t in self.tasks.values():
            for d in t.deps:
                succ[d].append(t.name)
        rank: dict[str, float] = {}
        for n in reversed(list(self.tasks)):             # insertion order is topological (deps must exist when added)
            rank[n] = self.tasks[n].cost + max((rank[s] for s in succ[n]), default=0.0)
        return rank

    def plan(self) -> Plan:
        K = len(self.streams)
        names = list(self.tasks)
        if self.policy == "critical_path":
            rank = self._upward_rank()
            placed: set = set()
            order = []
            ready = lambda n: all(d in placed for d in self.tasks[n].deps)
            while len(order) < len(names):
                cand = [n for n in names if n not in placed and ready(n)]
                n = max(cand, key=lambda n: (rank[n], self.tasks[n].priority))
                order.append(n)
                placed.add(n)
        else:
            order = names
        free = [0.0] * K
        finish: dict[str, float] = {}
        plan = Plan()
        for i, n in enumerate(order):
            t = self.tasks[n]
            if self.policy == "round_robin":
                s = i % K
            elif self.policy == "least_loaded":
                s = min(range(K), key=lambda k: free[k])
            else:
                def start_on(k):
                    dep_ready = max((finish[d] for d in t.deps), default=0.0)
                    return max(free[k], dep_ready)
                # earliest start; ties go to a stream that already holds a predecessor (one event fewer)
                s = min(range(K), key=lambda k: (start_on(k), -sum(plan.assignment[d] == k for d in t.deps), k))
            st = max(free[s], max((finish[d] for d in t.deps), default=0.0))
            plan.assignment[n], plan.start[n] = s, st
            finish[n] = st + t.cost
            free[s] = finish[n]
            plan.cross_stream_edges += sum(plan.assignment[d] != s for d in t.deps)
        plan.order = order
        plan.makespan = max(finish.values(), default=0.0)
        return plan

    # ---- execution --------------------------------------------------------------------------------------------
    def run(self, plan: Plan | None = None) -> dict:
        """Issues every task on its stream in plan order (each body runs with its stream current when the stream object
        supports it) and returns ``{name: result}``; ``self.coordinator.stats`` then tells how many events were needed."""
        plan = plan or self.plan()
        coord = OperationCoordinator(self._event_factory)
        for n in plan.order:
            coord.add_operation(n, self.streams[plan.assignment[n]], self.tasks[n].deps)
        self.coordinator = coord
        out = {}
        for n in plan.order:
            stream, fn = self.streams[plan.assignment[n]], self.tasks[n].fn
            ctx = _stream_context(stream)
            with ctx:
                out[n] = coord.issue(n, fn)
        return out

    def join(self, onto=None):
        """Makes ``onto`` (default: the first stream) wait for the last event of every other stream."""
        onto = onto if onto is not None else self.streams[0]
        last: dict = {}
        for n, op in self.coordinator.ops.items():
            last[id(op.stream)] = op
        for op in last.values():
            if op.stream is not onto and op.event is not None:
                op.event.wait(onto)


class _Null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


def _stream_context(stream):
    try:
        import torch
        if isinstance(stream, torch.cuda.Stream):
            return torch.cuda.stream(stream)
    except Exception:
        pass
    return _Null()
