"""Training-step engine: flat mixed-precision parameters, fused optimizer, CUDA-graph replay.

``CausalLMTrainer.step(ids, targets)`` is the call a user makes per step: it copies the batch from
(pinned) host memory to static device buffers, runs forward + backward + fused AdamW, and returns the
loss as a Python float (a device→host read). After a few eager warm-up steps the whole step is
captured into a CUDA graph and replayed, which removes the Python / launch overhead of the ~700
kernels of a GPT-2-medium step. The reference schedules nothing on the device (its training loop is
per-op host code: ``crates/torsh-cli/src/commands/train_real.rs:241-422``); its CUDA-graph wrapper is
``crates/torsh-backend/src/cuda/graph.rs:13-327``.
"""
from __future__ import annotations

import torch

from . import _native as nv
from .optim.flat import FlatAdamW, FlatParameters


def _raise_on_status(code: int, status_dev) -> None:
    """A bounded device-side wait of the step ran out (a peer rank late by more than the limit, a broken pipeline):
    the kernels skipped the work that depended on it, so the optimizer state is intact but the step did not happen
    on every rank. Stop here rather than let the next step run without cross-rank synchronisation."""
    if code != 0:
        if status_dev is not None:
            status_dev.zero_()
        exc = nv.KernelCheckFailed if code in (107, 108) else nv.KernelTimeout
        raise exc(f"device status {code}: {nv._STATUS_NAMES.get(code, 'unknown')} (training step aborted)")


class PendingLoss:
    """The loss of a step that may still be running: :meth:`value` waits for that step's device→host copy only and
    raises :class:`KernelTimeout` if a kernel of that step recorded an error in the device status word."""

    def __init__(self, buf: torch.Tensor, event, status_host=None, status_dev=None):
        self._buf, self._event, self._status_host, self._status_dev = buf, event, status_host, status_dev

    def value(self) -> float:
        if self._event is not None:
            self._event.synchronize()
        if self._status_host is not None:
            _raise_on_status(int(self._status_host[0]), self._status_dev)
        return float(self._buf)


class CausalLMTrainer:
    PIPELINE_SLOTS = 4

    def __init__(self, model, *, lr: float = 3e-4, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 batch_size: int, seq_len: int, use_graph: bool = True, warmup_eager: int = 2, grad_accum: int = 1,
                 parallel=None):
        self.model = model
        self.device = next(model.parameters()).device
        self.parallel = parallel
        if parallel is not None:
            self.flat = parallel.flatten(model)
            self.opt = parallel.optimizer(self.flat, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        else:
            self.flat = FlatParameters(model.parameters())
            self.opt = FlatAdamW(self.flat, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.batch_size, self.seq_len, self.grad_accum = batch_size, seq_len, grad_accum
        self.use_graph = use_graph and self.device.type == "cuda"
        self.warmup_eager = warmup_eager
        self.static_ids = torch.zeros(batch_size, seq_len, dtype=torch.int64, device=self.device)
        self.static_targets = torch.zeros(batch_size, seq_len, dtype=torch.int64, device=self.device)
        self.static_loss = torch.zeros((), dtype=torch.float32, device=self.device)
        self.loss_host = torch.zeros((), dtype=torch.float32).pin_memory() if self.device.type == "cuda" else torch.zeros(())
        cuda = self.device.type == "cuda"
        self._loss_ring = [torch.zeros((), dtype=torch.float32).pin_memory() if cuda else torch.zeros(())
                           for _ in range(self.PIPELINE_SLOTS)]
        self._loss_events = [torch.cuda.Event() if cuda else None for _ in range(self.PIPELINE_SLOTS)]
        # the device status word travels to the host next to the loss of every step (4 more bytes)
        self._status_dev = nv.status_word(self.device) if cuda else None
        self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory() if cuda else None
        self._status_ring = [torch.zeros(4, dtype=torch.int32).pin_memory() if cuda else None
                             for _ in range(self.PIPELINE_SLOTS)]
        self.graph = None
        self.steps_done = 0
        self.launches_per_step = 0
        self.h2d_bytes_per_step = 2 * batch_size * seq_len * 8
        self.d2h_bytes_per_step = 4 + (16 if cuda else 0)

    # ---- the device work of one step ------------------------------------------------------------
    def _device_step(self):
        if self.parallel is not None and hasattr(self.parallel, "begin_step"):
            self.parallel.begin_step()
        loss = self.model(self.static_ids, self.static_targets, loss_scale=1.0 / self.grad_accum)
        loss.backward()
        self.static_loss.copy_(loss.detach())
        if self.parallel is not None:
            self.parallel.reduce_and_step(self.flat, self.opt)
        else:
            self.opt.launch()

    def _capture(self):
        # lr and the Adam bias corrections are read from a device buffer that prepare_step()
        # refreshes before every replay, so the captured step keeps advancing correctly.
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._device_step()

    def step_device_only(self):
        """Run one step on whatever is in the static buffers (no host transfers)."""
        self.opt.prepare_step()
        if self.use_graph and self.steps_done >= self.warmup_eager:
            if self.graph is None:
                torch.cuda.synchronize()
                n0 = nv.launch_count
                self._capture()
                self.launches_per_step = nv.launch_count - n0
            self.graph.replay()
        else:
            n0 = nv.launch_count
            self._device_step()
            self.launches_per_step = nv.launch_count - n0
        self.steps_done += 1

    def step(self, ids: torch.Tensor, targets: torch.Tensor) -> float:
        """One training step from host tensors; returns the loss value."""
        self.static_ids.copy_(ids, non_blocking=True)
        self.static_targets.copy_(targets, non_blocking=True)
        self.step_device_only()
        if self.device.type == "cuda":
            self.loss_host.copy_(self.static_loss, non_blocking=True)
            self._status_host.copy_(self._status_dev, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            _raise_on_status(int(self._status_host[0]), self._status_dev)
            return float(self.loss_host)
        return float(self.static_loss)

    def step_async(self, ids: torch.Tensor, targets: torch.Tensor) -> PendingLoss:
        """Like :meth:`step`, but returns at once with a handle on the loss, so the host can stage and launch the next
        step while this one runs (read the handle one step late and the device never idles between steps). ``ids`` and
        ``targets`` must stay untouched until the step has run; at most ``PIPELINE_SLOTS`` handles may be unread."""
        self.static_ids.copy_(ids, non_blocking=True)
        self.static_targets.copy_(targets, non_blocking=True)
        self.step_device_only()
        slot = self.steps_done % self.PIPELINE_SLOTS
        buf, ev = self._loss_ring[slot], self._loss_events[slot]
        buf.copy_(self.static_loss, non_blocking=True)
        sh = self._status_ring[slot]
        if sh is not None:
            sh.copy_(self._status_dev, non_blocking=True)
        if ev is not None:
            ev.record()
        return PendingLoss(buf, ev, sh, self._status_dev)


class GraphedStep:
    """Any training step as one CUDA graph: ``fn(*static_inputs)`` is run eagerly ``warmup`` times on a side stream
    (so lazily created state exists), captured once, and replayed by every later call after its inputs have been copied
    into the static buffers. The step's side-stream work (gradient-bucket all-reduces launched from autograd hooks)
    is captured with it as long as those streams fork from and join the capturing stream; this package's collectives
    keep their barrier epoch on the device for exactly that reason. ``outputs`` are the tensors ``fn`` returned at
    capture time and are overwritten by every replay. If the capture fails the step stays eager and ``error`` says why.

    The reference's counterpart is its CUDA-graph layer (crates/torsh-backend/src/cuda/graph/mod.rs), which records
    kernel nodes by hand; here stream capture records whatever the step launches."""

    def __init__(self, fn, static_inputs, warmup: int = 2, enabled: bool = True):
        self.fn, self.static_inputs = fn, list(static_inputs)
        self.graph, self.outputs, self.error = None, None, None
        self.launches_per_step = 0
        self._left = max(int(warmup), 1)
        self.enabled = enabled and torch.cuda.is_available()
        self._side = torch.cuda.Stream() if self.enabled else None

    def __call__(self, *inputs):
        for dst, src in zip(self.static_inputs, inputs):
            if dst is not src:
                dst.copy_(src, non_blocking=True)
        if not self.enabled or self.error is not None:
            return self.fn(*self.static_inputs)
        if self.graph is not None:
            self.graph.replay()
            return self.outputs
        if self._left > 0:
            # warm-up on a side stream, as stream capture later runs on one: autograd remembers the stream a gradient
            # was first accumulated on and would otherwise tie the legacy default stream into the capture
            self._left -= 1
            n0 = nv.launch_count
            cur = torch.cuda.current_stream()
            self._side.wait_stream(cur)
            with torch.cuda.stream(self._side):
                out = self.fn(*self.static_inputs)
            cur.wait_stream(self._side)
            self.launches_per_step = nv.launch_count - n0
            return out
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(graph):
                out = self.fn(*self.static_inputs)
        except Exception as e:                      # a step that cannot be captured keeps running eagerly
            import traceback
            self.error = f"{type(e).__name__}: {e}"
            self.error_detail = traceback.format_exc()
            torch.cuda.synchronize()
            return self.fn(*self.static_inputs)
        self.graph, self.outputs = graph, out
        self.graph.replay()
        return self.outputs
