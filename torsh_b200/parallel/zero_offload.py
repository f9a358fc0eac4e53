"""ZeRO-3 style CPU offload of optimizer state (``crates/torsh-distributed/src/zero_3_cpu_offload``).

Defaults of the reference config (``config.rs``): offload params + grads + optimizer state, CPU budget 32 GB, GPU
parameter budget 2 GB, prefetch buffer 16, async prefetch, overlap, pinned memory. On 180 GB B200s the flat FSDP
engine keeps everything resident; this module provides the offload policy for models that do not fit: fp32 master
weights and Adam moments live in pinned host memory, the update runs on the CPU shard by shard while the next
shard's gradients are copied down on a side stream."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Zero3OffloadConfig:
    offload_params: bool = True
    offload_grads: bool = True
    offload_optimizer_states: bool = True
    cpu_memory_budget_gb: float = 32.0
    gpu_param_budget_gb: float = 2.0
    prefetch_buffer_size: int = 16
    async_prefetch: bool = True
    overlap_computation: bool = True
    pin_memory: bool = True
    chunk_numel: int = 1 << 24


class OffloadedAdamW:
    """AdamW (reference arithmetic) whose fp32 state lives on the host; ``params`` are device tensors."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, config: Zero3OffloadConfig | None = None):
        self.cfg = config or Zero3OffloadConfig()
        self.params = [p for p in params]
        self.lr, self.betas, self.eps, self.wd, self.t = lr, betas, eps, weight_decay, 0
        pin = self.cfg.pin_memory and torch.cuda.is_available()
        mk = lambda p: torch.zeros(p.numel(), dtype=torch.float32).pin_memory() if pin else torch.zeros(p.numel(), dtype=torch.float32)
        self.master = [mk(p).copy_(p.detach().float().reshape(-1).cpu()) for p in self.params]
        self.m = [mk(p) for p in self.params]
        self.v = [mk(p) for p in self.params]
        self.gbuf = [mk(p) for p in self.params]
        self.stream = torch.cuda.Stream() if torch.cuda.is_available() and self.params[0].is_cuda else None
        need = sum(p.numel() for p in self.params) * 16 / 2 ** 30
        if need > self.cfg.cpu_memory_budget_gb:
            raise MemoryError(f"offloaded state needs {need:.1f} GB of host memory, budget is {self.cfg.cpu_memory_budget_gb} GB")

    @torch.no_grad()
    def step(self):
        self.t += 1
        b1, b2 = self.betas
        bc1, bc2 = 1 - b1 ** self.t, 1 - b2 ** self.t
        evs = []
        for p, g in zip(self.params, self.gbuf):  # D2H of all gradients on the side stream
            if p.grad is None:
                evs.append(None)
                continue
            if self.stream is not None:
                self.stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.stream):
                    g.copy_(p.grad.reshape(-1).float(), non_blocking=True)
                    e = torch.cuda.Event()
                    e.record(self.stream)
                evs.append(e)
            else:
                g.copy_(p.grad.reshape(-1).float())
                evs.append(True)
        for p, w, m, v, g, e in zip(self.params, self.master, self.m, self.v, self.gbuf, evs):
            if e is None:
                continue
            if e is not True:
                e.synchronize()
            w.mul_(1 - self.lr * self.wd)
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            w.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(self.eps), value=-self.lr)
            p.data.copy_(w.view(p.shape), non_blocking=True)

    def zero_grad(self):
        for p in self.params:
            p.grad = None
