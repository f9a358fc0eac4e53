"""ZeRO-3 with CPU offload: parameters, gradients and optimizer state partitioned over the ranks and kept in (pinned)
host memory, brought to the device layer by layer.

Reference: ``crates/torsh-distributed/src/zero_3_cpu_offload`` - ``Zero3CpuOffloadManager`` (``mod.rs:120-515``: forward
= prefetch → ensure-on-GPU → compute → offload, backward in reverse + gradient partition reduction, optimizer step on the
owned partitions), ``Zero3CpuOffloadConfig`` with its defaults (``config.rs:11-60``: offload params + grads + optimizer
states, CPU budget 32 GB, GPU parameter budget 2 GB, prefetch buffer 16, async prefetch, overlap, pinned memory),
``CpuCompressionMethod`` (``:195-245``), ``AutoMemoryStrategy`` thresholds (``:249-290``) and ``Zero3RankMapping``
(round-robin partition ownership, ``:294-370``). There every movement is simulated on host vectors.

Here one *partition* is one layer (a child of the layer list given to the manager). Every rank keeps 1 / world of each
partition: the fp32 master shard and both Adam moments in host memory (pinned when a GPU is present), plus a transfer
copy of the shard in the compression dtype. A layer's forward and backward hooks

* wait for the layer's parameters (host → device copy of the own shard on a copy stream, then an all-gather over the
  group into the layer's full buffer) and start the same for the next ``prefetch_buffer_size`` layers while the GPU
  parameter budget allows,
* release the full buffer afterwards (the storage is shrunk to zero bytes, so tensors that autograd saved stay valid
  and see the data again after the next gather) when the memory strategy says so,
* after the layer's backward, reduce-scatter the gradient, move the rank's gradient shard to the host on the copy
  stream and drop the device gradients.

``step()`` runs AdamW (the reference's arithmetic order) on the host shards, or on device-resident state when
``offload_optimizer_states`` is off. The flat FSDP engine of this package keeps everything resident; this manager is
the path for models whose parameters do not fit in the device budget.
"""
from __future__ import annotations

import time
from collections import OrderedDict
from dataclasses import dataclass, field
from enum import Enum

import torch
import torch.distributed as dist

from . import collectives as coll


def _all_gather_into(full: torch.Tensor, mine: torch.Tensor, group) -> None:
    full.copy_(coll.all_gather_into_tensor(mine.contiguous(), group))


class CpuCompressionMethod(Enum):
    NONE = "none"
    FP16 = "fp16"
    BF16 = "bf16"
    INT8 = "int8"
    QUANTIZATION = "quantization"
    LOSSLESS = "lossless"

    def ratio(self) -> float:
        return {"none": 1.0, "fp16": 0.5, "bf16": 0.5, "int8": 0.25, "quantization": 0.25, "lossless": 0.7}[self.value]

    def is_lossy(self) -> bool:
        return self in (CpuCompressionMethod.FP16, CpuCompressionMethod.BF16, CpuCompressionMethod.INT8,
                        CpuCompressionMethod.QUANTIZATION)


class AutoMemoryStrategy(Enum):
    CONSERVATIVE = "conservative"
    BALANCED = "balanced"
    AGGRESSIVE = "aggressive"
    EXTREME = "extreme"

    def pressure_threshold(self) -> float:
        return {"conservative": 0.9, "balanced": 0.75, "aggressive": 0.6, "extreme": 0.4}[self.value]

    def aggressiveness(self) -> float:
        return {"conservative": 0.2, "balanced": 0.5, "aggressive": 0.8, "extreme": 1.0}[self.value]


@dataclass
class Zero3OffloadConfig:
    offload_params: bool = True
    offload_grads: bool = True
    offload_optimizer_states: bool = True
    cpu_memory_budget_gb: float = 32.0
    gpu_param_budget_gb: float = 2.0
    max_gpu_memory_mb: int = 8 * 1024
    max_cpu_memory_mb: int = 64 * 1024
    prefetch_buffer_size: int = 16
    async_prefetch: bool = True
    overlap_computation: bool = True
    pin_memory: bool = True
    cpu_compression: CpuCompressionMethod = CpuCompressionMethod.NONE
    auto_memory_management: AutoMemoryStrategy = AutoMemoryStrategy.AGGRESSIVE
    chunk_numel: int = 1 << 24

    def validate(self) -> None:
        if self.cpu_memory_budget_gb <= 0 or self.gpu_param_budget_gb <= 0:
            raise ValueError("memory budgets must be positive")
        if self.prefetch_buffer_size < 0:
            raise ValueError("prefetch_buffer_size must be >= 0")
        if self.cpu_compression in (CpuCompressionMethod.INT8, CpuCompressionMethod.QUANTIZATION, CpuCompressionMethod.LOSSLESS):
            raise ValueError(f"host compression {self.cpu_compression.value!r} has no codec here: use none, fp16 or bf16")

    def effective_cpu_memory_budget(self) -> int:
        """Host bytes usable for parameter shards after compression (``config.rs:188``)."""
        return int(self.cpu_memory_budget_gb * 2 ** 30 / self.cpu_compression.ratio())


Zero3CpuOffloadConfig = Zero3OffloadConfig


class Zero3RankMapping:
    """Round-robin ownership of partitions (``config.rs:294-370``)."""

    def __init__(self, rank: int, world_size: int):
        if not 0 <= rank < world_size:
            raise ValueError("rank must be less than world size")
        self.rank, self.world_size = rank, world_size

    def owns_partition(self, idx: int) -> bool:
        return idx % self.world_size == self.rank

    def get_parameter_owner(self, idx: int) -> int:
        return idx % self.world_size

    def owned_partitions(self, total: int) -> list[int]:
        return [i for i in range(total) if self.owns_partition(i)]

    def owned_partition_count(self, total: int) -> int:
        base, rem = divmod(total, self.world_size)
        return base + (1 if self.rank < rem else 0)

    def global_to_local_partition(self, g: int) -> int | None:
        return g // self.world_size if self.owns_partition(g) else None

    def local_to_global_partition(self, l: int) -> int:
        return l * self.world_size + self.rank

    def communication_group(self, param_indices) -> list[int]:
        return sorted({self.get_parameter_owner(i) for i in param_indices})


@dataclass
class Zero3Stats:
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    gathers: int = 0
    prefetch_hits: int = 0
    prefetch_misses: int = 0
    releases: int = 0
    evictions: int = 0
    steps: int = 0
    optimizer_seconds: float = 0.0
    layer_seconds: dict = field(default_factory=dict)

    def as_dict(self) -> dict:
        d = dict(self.__dict__)
        d["prefetch_hit_rate"] = self.prefetch_hits / max(1, self.prefetch_hits + self.prefetch_misses)
        return d


class _Partition:
    """One layer's parameters: host shards + an on-demand full device buffer whose storage is shrunk to zero when released."""

    def __init__(self, index: int, params, world: int, rank: int, device, cfg: Zero3OffloadConfig):
        self.index, self.params = index, [p for p in params]
        self.device, self.dtype = device, self.params[0].dtype
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += p.numel()
        self.numel = off
        self.shard = (off + world - 1) // world
        self.padded = self.shard * world
        pin = cfg.pin_memory and device.type == "cuda"
        host = lambda dt: torch.zeros(self.shard, dtype=dt).pin_memory() if pin else torch.zeros(self.shard, dtype=dt)
        xfer_dtype = {CpuCompressionMethod.NONE: self.dtype, CpuCompressionMethod.FP16: torch.float16,
                      CpuCompressionMethod.BF16: torch.bfloat16}[cfg.cpu_compression]
        state_dev = torch.device("cpu") if cfg.offload_optimizer_states else device
        mk_state = (lambda: host(torch.float32)) if cfg.offload_optimizer_states else (lambda: torch.zeros(self.shard, dtype=torch.float32, device=device))
        self.master, self.exp_avg, self.exp_avg_sq = mk_state(), mk_state(), mk_state()
        self.state_device = state_dev
        self.xfer = host(xfer_dtype) if cfg.offload_params else torch.zeros(self.shard, dtype=xfer_dtype, device=device)
        self.grad_host = host(torch.float32) if cfg.offload_grads else None
        self.grad_shard_dev = None
        self.grad_event = None
        # full device buffer (all ranks' shards); parameters are views of it
        self.full = torch.zeros(self.padded, dtype=self.dtype, device=device)
        flat = torch.cat([p.detach().reshape(-1) for p in self.params])
        self.full[:self.numel].copy_(flat)
        mine = self.full[rank * self.shard:(rank + 1) * self.shard]
        self.master.copy_(mine.float())
        self.xfer.copy_(mine.to(xfer_dtype))
        for p, o in zip(self.params, self.offsets):
            p.data = self.full[o:o + p.numel()].view(p.shape)
        self.nbytes = self.padded * self.full.element_size()
        self.resident = True
        self.ready_event = None
        self.in_use = False

    def release(self):
        if self.resident:
            self.full.untyped_storage().resize_(0)
            self.resident = False
            self.ready_event = None

    def allocate(self):
        if not self.resident:
            self.full.untyped_storage().resize_(self.nbytes)
            self.resident = True


class Zero3CpuOffloadManager:
    """ZeRO-3 + CPU offload over an ordered list of layers.

    ``layers``: the modules that run one after the other (for example ``model.h``); parameters outside them (embeddings,
    final norm, head) form a last partition that stays resident. Training loop::

        mgr = Zero3CpuOffloadManager(model, list(model.h), config=cfg, lr=3e-4)
        loss = model(x).loss; loss.backward(); mgr.step()
    """

    def __init__(self, model: torch.nn.Module, layers, group=None, config: Zero3OffloadConfig | None = None, lr: float = 1e-3,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        self.cfg = config or Zero3OffloadConfig()
        self.cfg.validate()
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank_mapping = Zero3RankMapping(self.rank, self.world)
        self.model, self.layers = model, list(layers)
        self.lr, self.betas, self.eps, self.weight_decay, self.t = lr, betas, eps, weight_decay, 0
        self.device = next(model.parameters()).device
        self.stats = Zero3Stats()
        self.copy_stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        if self.world > 1:
            for p in model.parameters():
                dist.broadcast(p.data, 0, group=self.group)
        in_layers = set()
        self.partitions: list[_Partition] = []
        for i, layer in enumerate(self.layers):
            ps = [p for p in layer.parameters() if id(p) not in in_layers and p.requires_grad]
            in_layers.update(id(p) for p in ps)
            self.partitions.append(_Partition(i, ps, self.world, self.rank, self.device, self.cfg) if ps else None)
        rest = [p for p in model.parameters() if id(p) not in in_layers and p.requires_grad]
        self.rest = _Partition(len(self.layers), rest, self.world, self.rank, self.device, self.cfg) if rest else None
        host_need = sum(pt.shard * (12 + pt.xfer.element_size()) for pt in self._all() if pt is not None)
        if self.cfg.offload_optimizer_states and host_need > self.cfg.effective_cpu_memory_budget():
            raise MemoryError(f"host shards need {host_need / 2 ** 30:.2f} GB, the CPU budget is {self.cfg.cpu_memory_budget_gb} GB")
        self.gpu_budget = int(self.cfg.gpu_param_budget_gb * 2 ** 30)
        self._lru: OrderedDict[int, _Partition] = OrderedDict()
        for i, layer in enumerate(self.layers):
            if self.partitions[i] is None:
                continue
            layer.register_forward_pre_hook(self._pre_forward(i))
            layer.register_forward_hook(self._post_forward(i))
            layer.register_full_backward_pre_hook(self._pre_backward(i))
            layer.register_full_backward_hook(self._post_backward(i))
        # start with every layer released (parameters offloaded), as after a step
        if self.cfg.offload_params:
            for pt in self.partitions:
                if pt is not None:
                    pt.release()

    def _all(self):
        return [pt for pt in self.partitions if pt is not None] + ([self.rest] if self.rest is not None else [])

    # ---- residency --------------------------------------------------------------------------------------
    def gpu_param_bytes(self) -> int:
        return sum(pt.nbytes for pt in self.partitions if pt is not None and pt.resident)

    def memory_pressure(self) -> float:
        return self.gpu_param_bytes() / max(self.gpu_budget, 1)

    def _evict_for(self, need: int, keep: set[int]):
        """Release least-recently-used layers that are not in use until `need` more bytes fit in the GPU budget."""
        for idx in list(self._lru.keys()):
            if self.gpu_param_bytes() + need <= self.gpu_budget:
                break
            pt = self._lru[idx]
            if idx in keep or pt.in_use or not pt.resident:
                continue
            pt.release()
            self._lru.pop(idx, None)
            self.stats.evictions += 1

    def _start_fetch(self, i: int, keep: set[int]) -> bool:
        """Begin bringing partition i to the device (own shard host → device, then all-gather). Returns False when the
        GPU parameter budget has no room even after evictions (the caller then fetches it when it is needed)."""
        pt = self.partitions[i]
        if pt is None or pt.resident:
            return True
        if self.gpu_param_bytes() + pt.nbytes > self.gpu_budget:
            self._evict_for(pt.nbytes, keep | {i})
            if self.gpu_param_bytes() + pt.nbytes > self.gpu_budget and any(p is not None and p.resident for p in self.partitions):
                return False
        pt.allocate()
        mine = pt.full[self.rank * pt.shard:(self.rank + 1) * pt.shard]

        def work():
            mine.copy_(pt.xfer, non_blocking=True)
            self.stats.h2d_bytes += pt.xfer.numel() * pt.xfer.element_size()
            if self.world > 1:
                _all_gather_into(pt.full, mine, self.group)
            self.stats.gathers += 1

        if self.copy_stream is not None and self.cfg.async_prefetch:
            self.copy_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.copy_stream):
                work()
                pt.ready_event = torch.cuda.Event()
                pt.ready_event.record(self.copy_stream)
        else:
            work()
        self._lru[i] = pt
        self._lru.move_to_end(i)
        return True

    def _ensure(self, i: int, direction: int):
        """Partition i is needed now; prefetch the next ones in `direction` (+1 forward, -1 backward)."""
        pt = self.partitions[i]
        if pt.resident:
            self.stats.prefetch_hits += 1
        else:
            self.stats.prefetch_misses += 1
            if not self._start_fetch(i, {i}):
                # nothing could be evicted: exceed the budget for the layer in use rather than fail
                pt.allocate()
                mine = pt.full[self.rank * pt.shard:(self.rank + 1) * pt.shard]
                mine.copy_(pt.xfer)
                if self.world > 1:
                    _all_gather_into(pt.full, mine, self.group)
                self._lru[i] = pt
        if pt.ready_event is not None:
            torch.cuda.current_stream().wait_event(pt.ready_event)
            pt.ready_event = None
        pt.in_use = True
        self._lru[i] = pt
        self._lru.move_to_end(i)
        keep = {i}
        for k in range(1, self.cfg.prefetch_buffer_size + 1):
            j = i + direction * k
            if not 0 <= j < len(self.partitions):
                break
            if self.partitions[j] is None:
                continue
            keep.add(j)
            if not self._start_fetch(j, keep):
                break

    def _maybe_release(self, i: int, last: bool):
        pt = self.partitions[i]
        pt.in_use = False
        if not self.cfg.offload_params:
            return
        # under the strategy's pressure threshold layers stay cached (they are needed again in backward); above it, or
        # with the extreme strategy, the layer is offloaded as soon as it has been used
        strat = self.cfg.auto_memory_management
        if strat is AutoMemoryStrategy.EXTREME or self.memory_pressure() > strat.pressure_threshold() or last:
            pt.release()
            self._lru.pop(i, None)
            self.stats.releases += 1

    # ---- hooks --------------------------------------------------------------------------------------------
    def _pre_forward(self, i):
        def hook(module, args):
            self._t0 = time.perf_counter()
            self._ensure(i, +1)
        return hook

    def _post_forward(self, i):
        def hook(module, args, output):
            self.stats.layer_seconds[i] = self.stats.layer_seconds.get(i, 0.0) + time.perf_counter() - getattr(self, "_t0", time.perf_counter())
            # during training the layer is needed again by its backward; keep the decision to the memory strategy
            self._maybe_release(i, last=not torch.is_grad_enabled())
        return hook

    def _pre_backward(self, i):
        def hook(module, grad_output):
            self._ensure(i, -1)
        return hook

    def _post_backward(self, i):
        def hook(module, grad_input, grad_output):
            self._reduce_partition(self.partitions[i])
            self._maybe_release(i, last=True)
        return hook

    # ---- gradients ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def _reduce_partition(self, pt: _Partition):
        """Reduce-scatter (mean) the partition's gradient, keep this rank's shard, move it to the host."""
        full = torch.zeros(pt.padded, dtype=torch.float32, device=pt.device)
        for p, o in zip(pt.params, pt.offsets):
            if p.grad is not None:
                full[o:o + p.numel()].copy_(p.grad.reshape(-1))
                p.grad = None
        if self.world > 1:
            shard = coll.reduce_scatter(full, coll.ReduceOp.SUM, self.group).div_(self.world)
        else:
            shard = full[:pt.shard]
        if pt.grad_host is not None:
            if self.copy_stream is not None and self.cfg.overlap_computation:
                self.copy_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.copy_stream):
                    pt.grad_host.copy_(shard, non_blocking=True)
                    pt.grad_event = torch.cuda.Event()
                    pt.grad_event.record(self.copy_stream)
                shard.record_stream(self.copy_stream)
            else:
                pt.grad_host.copy_(shard)
            self.stats.d2h_bytes += pt.shard * 4
        else:
            pt.grad_shard_dev = shard.clone()

    # ---- optimizer ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self):
        """AdamW on every shard this rank owns a slice of (decoupled decay first, both moments bias-corrected:
        ``crates/torsh-optim/src/adam.rs:809-950``), then refresh the transfer copies."""
        t0 = time.perf_counter()
        if self.rest is not None:
            self._reduce_partition(self.rest)
        self.t += 1
        b1, b2 = self.betas
        bc1, bc2 = 1 - b1 ** self.t, 1 - b2 ** self.t
        for pt in self._all():
            if pt.grad_event is not None:
                pt.grad_event.synchronize()
                pt.grad_event = None
            g = pt.grad_host if pt.grad_host is not None else pt.grad_shard_dev
            if g is None:
                continue
            g = g.to(pt.master.device, non_blocking=False) if g.device != pt.master.device else g
            w, m, v = pt.master, pt.exp_avg, pt.exp_avg_sq
            w.mul_(1 - self.lr * self.weight_decay)
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            w.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(self.eps), value=-self.lr)
            pt.xfer.copy_(w.to(pt.xfer.dtype) if w.device == pt.xfer.device else w.to(pt.xfer.device, pt.xfer.dtype))
            pt.grad_shard_dev = None
        # the resident remainder (embeddings, head) is refreshed in place from every rank's shard
        if self.rest is not None:
            pt = self.rest
            mine = pt.full[self.rank * pt.shard:(self.rank + 1) * pt.shard]
            mine.copy_(pt.xfer.to(self.device, pt.dtype))
            if self.world > 1:
                _all_gather_into(pt.full, mine, self.group)
        # layers still cached on the device hold the old values: drop them so the next use gathers the new ones
        for i, pt in enumerate(self.partitions):
            if pt is not None and pt.resident:
                if self.cfg.offload_params:
                    pt.release()
                    self._lru.pop(i, None)
                else:
                    mine = pt.full[self.rank * pt.shard:(self.rank + 1) * pt.shard]
                    mine.copy_(pt.xfer.to(self.device, pt.dtype))
                    if self.world > 1:
                        _all_gather_into(pt.full, mine, self.group)
        self.stats.steps += 1
        self.stats.optimizer_seconds += time.perf_counter() - t0

    def zero_grad(self):
        for p in self.model.parameters():
            p.grad = None

    @torch.no_grad()
    def gather_state_dict(self) -> dict:
        """name → full tensor for every managed parameter (all-gathers every partition once)."""
        names = {id(p): n for n, p in self.model.named_parameters()}
        out = {}
        for pt in self._all():
            full = torch.empty(pt.padded, dtype=pt.dtype, device=pt.device)
            mine = pt.xfer.to(pt.device, pt.dtype)
            if self.world > 1:
                _all_gather_into(full, mine, self.group)
            else:
                full[:pt.shard].copy_(mine)
            for p, o in zip(pt.params, pt.offsets):
                out[names[id(p)]] = full[o:o + p.numel()].view(p.shape).clone()
        return out

    def memory_report(self) -> dict:
        pts = self._all()
        return {"host_state_bytes": sum(pt.shard * 12 for pt in pts) if self.cfg.offload_optimizer_states else 0,
                "host_param_bytes": sum(pt.xfer.numel() * pt.xfer.element_size() for pt in pts) if self.cfg.offload_params else 0,
                "gpu_param_bytes_now": self.gpu_param_bytes(), "gpu_param_budget": self.gpu_budget,
                "compression": self.cfg.cpu_compression.value, "strategy": self.cfg.auto_memory_management.value}


class OffloadedAdamW:
    """AdamW (reference arithmetic) whose fp32 state lives on the host; ``params`` are device tensors. The optimizer-only
    form of the offload (ZeRO-Offload): parameters and gradients stay on the device."""

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
