"""Distributed data parallel: bucketed gradient all-reduce fused with the 1/world scale (and the
bf16 ↔ fp32-accumulate cast), launched from autograd hooks and overlapped with backward.

Reference (``crates/torsh-distributed/src/ddp.rs``): ``BucketConfig`` 25 MB max / 1 MB min (``:21-38``),
``OverlapConfig`` max_pending 4, timeout 30 s, detect_unused (``:124-144``), bucket assignment largest-first
greedy (``:268-327``), flatten → ``all_reduce(Sum)`` → ``/world`` → unflatten on the host (``:478-534``), an
explicit ``sync_gradients`` call after backward (``:555-672``) and hook registration that is a no-op
(``:676-683``). There the collective does nothing.

Here every gradient is a view into one flat buffer in symmetric memory, so there is no flatten /
unflatten copy at all; a bucket is a contiguous range of that buffer. When the last gradient of a
bucket has been accumulated (post-accumulate-grad hooks), one kernel on a side stream all-reduces the
range in the NVSwitch (``multimem.ld_reduce`` + ``multimem.st``), multiplies by 1/world and writes the
result in place on every rank. CPU tensors (gloo) take the same bucket path with ``dist.all_reduce``.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..nn.module import Module
from . import planner


@dataclass
class BucketConfig:
    max_bucket_size_mb: float = 25.0
    min_bucket_size_mb: float = 1.0
    enabled: bool = True
    order: str = "backward"  # "backward": reverse registration order (ready early); "reference": largest first


@dataclass
class OverlapConfig:
    enabled: bool = True
    max_pending: int = 4
    timeout_s: float = 30.0
    detect_unused: bool = True


class DistributedDataParallel(Module):
    def __init__(self, module: torch.nn.Module, process_group=None, bucket_cap_mb: float = 25.0,
                 bucket_config: BucketConfig | None = None, overlap_config: OverlapConfig | None = None,
                 broadcast_buffers: bool = True, comm_blocks: int | None = 64, use_nvls: bool | None = None):
        super().__init__()
        self.module = module
        self.group = getattr(process_group, "group", process_group) or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.bucket_cfg = bucket_config or BucketConfig(max_bucket_size_mb=bucket_cap_mb)
        self.overlap_cfg = overlap_config or OverlapConfig()
        self.params = [p for p in module.parameters() if p.requires_grad]
        self.device = self.params[0].device
        self.on_gpu = self.device.type == "cuda"
        self.stats = {"buckets_reduced": 0, "bytes_reduced": 0, "unused_parameters": 0, "steps": 0}
        self._build_buckets()
        self._alloc(comm_blocks, use_nvls)
        with torch.no_grad():
            for p in module.parameters():
                dist.broadcast(p.data, 0, group=self.group)
            if broadcast_buffers:
                for b in module.buffers():
                    dist.broadcast(b.data, 0, group=self.group)
        self._ready = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)
        # False inside no_sync(): backward passes only accumulate locally (gradient accumulation over micro-batches)
        self.require_backward_grad_sync = True
        # the device status word of the step before is read (no host wait) at the next sync_gradients()
        self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory() if self.on_gpu else None
        self._status_event = torch.cuda.Event() if self.on_gpu else None
        self._status_queued = False
        for i, p in enumerate(self.params):
            p.register_post_accumulate_grad_hook(self._make_hook(i))

    # ---- layout ---------------------------------------------------------------------------------------
    def _build_buckets(self):
        cap = int(self.bucket_cfg.max_bucket_size_mb * 1024 * 1024)
        sizes = [p.numel() * 4 for p in self.params]  # the reference assumes f32 when sizing
        if self.bucket_cfg.order == "reference":
            assign = planner.assign_buckets(sizes, cap)
        else:
            assign, b, used = [0] * len(sizes), 0, 0
            for i in reversed(range(len(sizes))):
                if used and used + sizes[i] > cap:
                    b, used = b + 1, 0
                assign[i] = b
                used += sizes[i]
        nb = max(assign) + 1 if assign else 0
        self.buckets = [[i for i, a in enumerate(assign) if a == k] for k in range(nb)]
        self.bucket_of = assign

    def bucket_info(self) -> list[dict]:
        return [{"index": k, "num_params": len(b), "bytes": sum(self.params[i].numel() * 4 for i in b)}
                for k, b in enumerate(self.buckets)]

    def _alloc(self, comm_blocks, use_nvls):
        self.grad_dtype = self.params[0].dtype if all(p.dtype == self.params[0].dtype for p in self.params) else torch.float32
        offs, off, self.bucket_ranges = {}, 0, []
        for b in self.buckets:
            start = off
            for i in b:
                offs[i] = off
                off += (self.params[i].numel() + 127) // 128 * 128
            self.bucket_ranges.append((start, off - start))
        self.total = max(off, 128)
        if self.on_gpu and self.world > 1:
            from .collectives import FusedCollectives
            from .symm import SymmetricBuffer
            self.buf = SymmetricBuffer(self.total, self.grad_dtype, self.group)
            self.flat_grad = self.buf.tensor
            self.fused = FusedCollectives(self.group, nblocks=comm_blocks, use_nvls=use_nvls)
            self.comm_stream = torch.cuda.Stream()
        else:
            self.buf, self.fused, self.comm_stream = None, None, None
            self.flat_grad = torch.zeros(self.total, dtype=self.grad_dtype, device=self.device)
        for i, p in enumerate(self.params):
            p.grad = self.flat_grad[offs[i]:offs[i] + p.numel()].view(p.shape)
        self._offs = offs

    # ---- hooks ----------------------------------------------------------------------------------------
    def _make_hook(self, i: int):
        def hook(p):
            k = self.bucket_of[i]
            if p.grad.data_ptr() != self.flat_grad.data_ptr() + self._offs[i] * self.flat_grad.element_size():
                # autograd replaced the view (first backward after zero_grad(set_to_none=True)): copy back in
                view = self.flat_grad[self._offs[i]:self._offs[i] + p.numel()].view(p.shape)
                view.copy_(p.grad)
                p.grad = view
            if not self.require_backward_grad_sync:
                return  # no_sync(): the gradient stays a local sum; the synchronising backward reduces it
            if self._launched[k]:
                # the bucket was already averaged over the ranks in this step: adding another local gradient to it
                # would give avg(first) + local(second), different on every rank
                raise RuntimeError("DistributedDataParallel: a second backward() before sync_gradients(); run the "
                                   "earlier micro-batches of an accumulation step under no_sync()")
            self._ready[k] += 1
            if self._ready[k] == len(self.buckets[k]) and self.overlap_cfg.enabled:
                self._reduce_bucket(k)
        return hook

    def _reduce_bucket(self, k: int):
        if self._launched[k] or self.world == 1:
            self._launched[k] = True
            return
        self._launched[k] = True
        start, length = self.bucket_ranges[k]
        if self.fused is not None:
            cur = torch.cuda.current_stream()
            self.comm_stream.wait_stream(cur)
            with torch.cuda.stream(self.comm_stream):
                self.fused.all_reduce_(self.buf, numel=length, offset=start, scale=1.0 / self.world, mode="two_shot")
        else:
            view = self.flat_grad[start:start + length]
            dist.all_reduce(view, group=self.group)
            view.div_(self.world)
        self.stats["buckets_reduced"] += 1
        self.stats["bytes_reduced"] += length * self.flat_grad.element_size()

    # ---- user API -------------------------------------------------------------------------------------
    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    @contextlib.contextmanager
    def no_sync(self):
        """Backward passes inside this context accumulate gradients locally without any reduction; the first backward
        after it (followed by :meth:`sync_gradients`) reduces the accumulated sum. The reference reduces only in its
        explicit ``sync_gradients`` (``ddp.rs:555-672``), which gives the same accumulation semantics."""
        old = self.require_backward_grad_sync
        self.require_backward_grad_sync = False
        try:
            yield
        finally:
            self.require_backward_grad_sync = old

    def sync_gradients(self):
        """Finish the step's gradient synchronisation: reduce buckets whose hooks did not all fire (unused
        parameters), in ascending order on every rank, and join the comm stream. Call after ``backward()``."""
        for k in range(len(self.buckets)):
            if not self._launched[k]:
                if self.overlap_cfg.detect_unused:
                    self.stats["unused_parameters"] += len(self.buckets[k]) - self._ready[k]
                self._reduce_bucket(k)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        self._check_device_status()
        self._ready = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)
        self.stats["steps"] += 1

    def _check_device_status(self):
        """Raises :class:`KernelTimeout` when a collective kernel of the PREVIOUS step recorded a failed cross-rank wait
        (it then skipped its reduction), and queues the copy of this step's status word; no host wait on the new step."""
        if self.fused is None or torch.cuda.is_current_stream_capturing():
            return      # inside a CUDA-graph capture the owner of the graph reads the status word after its replays
        from .. import _native as nv
        if self._status_queued:
            self._status_event.synchronize()   # a whole step old: already complete
            code = int(self._status_host[0])
            if code != 0:
                nv.status_word(self.device).zero_()
                self._status_queued = False
                raise nv.KernelTimeout(f"device status {code}: {nv._STATUS_NAMES.get(code, 'unknown')} "
                                       f"(gradient all-reduce of the previous step did not complete on every rank)")
        self._status_host.copy_(nv.status_word(self.device), non_blocking=True)
        self._status_event.record()
        self._status_queued = True

    def zero_grad(self, set_to_none: bool = False):
        """Keeps the gradient views alive (zeroing the flat buffer) so that no copy is ever needed."""
        self.flat_grad.zero_()

    def get_sync_stats(self) -> dict:
        return dict(self.stats)


DDP = DistributedDataParallel
