"""Distributed optimizer wrappers (``crates/torsh-optim/src/distributed/{core,async_sgd,elastic_sgd}.rs``).

* ``DistributedOptimizer``: averages gradients over the group before the inner step — flattened into buckets of
  ``bucket_mb`` so small tensors share a collective; strategies ``all_reduce`` (every step) and ``local_sgd``
  (parameters averaged every ``sync_every`` steps).
* ``AsyncSGD``: staleness-aware SGD against a :class:`~torsh_b200.parallel.parameter_server.ParameterServer`
  (learning rate scaled by ``1 / (1 + staleness)``).
* ``ElasticAveragingSGD``: local steps plus an elastic pull towards a centre variable that is averaged over ranks
  every ``tau`` steps (EASGD)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group):
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


class DistributedOptimizer:
    def __init__(self, optimizer, group=None, strategy: str = "all_reduce", bucket_mb: float = 25.0, sync_every: int = 1):
        self.inner, self.group, self.strategy, self.sync_every = optimizer, group, strategy, sync_every
        self.bucket_bytes = int(bucket_mb * 2**20)
        self.param_groups = optimizer.param_groups
        self.steps = 0
        self.stats = {"collectives": 0, "bytes": 0}

    def _params(self):
        return [p for g in self.inner.param_groups for p in g["params"]]

    def _average(self, tensors):
        w = _world(self.group)
        if w == 1 or not tensors:
            return
        bucket, size = [], 0
        for t in tensors + [None]:
            if t is not None and (not bucket or (size + t.numel() * t.element_size() <= self.bucket_bytes and t.dtype == bucket[0].dtype)):
                bucket.append(t); size += t.numel() * t.element_size()
                continue
            flat = torch.cat([b.reshape(-1) for b in bucket])
            dist.all_reduce(flat, group=self.group)
            flat.div_(w)
            off = 0
            for b in bucket:
                b.copy_(flat[off:off + b.numel()].view_as(b)); off += b.numel()
            self.stats["collectives"] += 1; self.stats["bytes"] += size
            bucket, size = ([t], t.numel() * t.element_size()) if t is not None else ([], 0)

    @torch.no_grad()
    def step(self):
        self.steps += 1
        if self.strategy == "all_reduce":
            self._average([p.grad for p in self._params() if p.grad is not None])
            self.inner.step()
        else:  # local SGD
            self.inner.step()
            if self.steps % self.sync_every == 0:
                self._average([p.data for p in self._params()])

    def zero_grad(self, set_to_none: bool = True):
        self.inner.zero_grad(set_to_none)


class AsyncSGD:
    def __init__(self, module: torch.nn.Module, client, lr: float = 0.01):
        self.module, self.client, self.lr = module, client, lr
        self.client.sync(module)
        self.staleness_seen: list[int] = []

    def step(self):
        """Push gradients computed on the local (possibly stale) copy, then pull what changed."""
        before = dict(self.client.versions)
        self.client.push_gradients(self.module)
        self.client.sync(self.module)
        self.staleness_seen.append(max((self.client.versions[k] - before.get(k, 0) - 1 for k in self.client.versions), default=0))

    def zero_grad(self):
        self.module.zero_grad(set_to_none=True)


class ElasticAveragingSGD:
    def __init__(self, params, lr: float = 0.01, rho: float = 0.1, tau: int = 4, group=None):
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.alpha, self.tau, self.group = lr, lr * rho, tau, group
        self.center = [p.detach().clone() for p in self.params]
        self.steps = 0

    @torch.no_grad()
    def step(self):
        self.steps += 1
        for p in self.params:
            if p.grad is not None:
                p.add_(p.grad, alpha=-self.lr)
        if self.steps % self.tau == 0:
            w = _world(self.group)
            for p, c in zip(self.params, self.center):
                diff = p - c
                p.sub_(diff, alpha=self.alpha)
                upd = diff * self.alpha
                if w > 1:
                    dist.all_reduce(upd, group=self.group)
                c.add_(upd)

    def zero_grad(self):
        for p in self.params:
            p.grad = None
