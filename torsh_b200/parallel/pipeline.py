"""Pipeline parallelism: GPipe and 1F1B over point-to-point sends (NCCL p2p on GPUs, gloo on CPU).

Reference (``crates/torsh-distributed/src/pipeline.rs``): schedules ``GPipe / OneFOneBInterleaved /
InterleavedOneFOneB`` (``:18-25``), ``PipelineConfig`` with ``num_micro_batches 4``, ``base_tag 1000``, timeout 30 s
(``:29-55``), stage = prev/next rank (``:58-116``), GPipe forward (``:206-251``), 1F1B warm-up / steady / cool-down
(``:254-340``), micro-batch split along dim 0 (``:410-429``), tags ``base + mb`` forward and ``base + 10000 + mb``
backward (``:350-384``). There send/recv are no-ops and the backward uses mock gradients.

Here the per-stage action list comes from the native planner; every forward stashes its input and output
so the matching backward can run ``torch.autograd.backward`` with the received gradient. Receives for the
next action are posted before computing (on NCCL they run on the p2p stream, overlapping compute).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import torch
import torch.distributed as dist

from . import planner


class ScheduleType(Enum):
    GPIPE = "gpipe"
    ONE_F_ONE_B = "1f1b"
    INTERLEAVED_ONE_F_ONE_B = "interleaved"  # executed as plain 1F1B, as in the reference (pipeline.rs:343-347)


@dataclass
class PipelineConfig:
    num_micro_batches: int = 4
    schedule: ScheduleType = ScheduleType.ONE_F_ONE_B
    base_tag: int = 1000
    timeout_s: float = 30.0


class PipelineParallel:
    """One pipeline stage. ``stage_module`` maps the previous stage's activation (or the raw input on stage 0)
    to this stage's activation; on the last stage ``loss_fn(output, target)`` produces the micro-batch loss."""

    def __init__(self, stage_module: torch.nn.Module, group=None, config: PipelineConfig | None = None,
                 activation_shape=None, activation_dtype=torch.float32, prev_rank: int | None = None,
                 next_rank: int | None = None):
        self.module, self.group, self.cfg = stage_module, group, config or PipelineConfig()
        g = group if group is not None else dist.group.WORLD
        self.stage, self.num_stages = dist.get_rank(g), dist.get_world_size(g)
        ranks = dist.get_process_group_ranks(g)
        self.prev = prev_rank if prev_rank is not None else (ranks[self.stage - 1] if self.stage > 0 else None)
        self.next = next_rank if next_rank is not None else (ranks[self.stage + 1] if self.stage + 1 < self.num_stages else None)
        self.act_shape, self.act_dtype = activation_shape, activation_dtype
        self.device = next(stage_module.parameters()).device
        self.stats = {"sends": 0, "recvs": 0, "bubbles": 0}
        # called as hook(micro_batch_index, in_flight_slot) before each forward: lets layers that keep per-micro-batch
        # buffers (the fused tensor-parallel layers) switch to the slot of this micro-batch
        self.micro_batch_hook = None

    @property
    def is_first(self):
        return self.prev is None

    @property
    def is_last(self):
        return self.next is None

    @staticmethod
    def split_micro_batches(t: torch.Tensor, n: int) -> list[torch.Tensor]:
        return list(t.chunk(n, 0))

    def _exchange(self, sends: list, recv_from: int | None, recv_tag: int = 0):
        """Posts the pending sends and (optionally) one receive as ONE batch, so that a send and the receive
        it is paired with on the peer can never wait on each other (on NCCL they become one grouped kernel).
        Returns the received tensor."""
        ops, buf = [], None
        for t, dst, tag in sends:
            ops.append(dist.P2POp(dist.isend, t, dst, tag=tag))
            self.stats["sends"] += 1
        if recv_from is not None:
            buf = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, buf, recv_from, tag=recv_tag))
            self.stats["recvs"] += 1
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        sends.clear()
        return buf

    def train_step(self, inputs: torch.Tensor | None, targets: torch.Tensor | None, loss_fn=None) -> torch.Tensor | None:
        """Runs all micro-batches through this stage; gradients accumulate in the parameters.
        Returns the mean micro-batch loss on the last stage, ``None`` elsewhere."""
        M = self.cfg.num_micro_batches
        sched = "gpipe" if self.cfg.schedule is ScheduleType.GPIPE else "1f1b"
        actions = planner.pipeline_schedule(sched, self.stage, self.num_stages, M)
        xs = self.split_micro_batches(inputs, M) if self.is_first else None
        ys = self.split_micro_batches(targets, M) if (self.is_last and targets is not None) else None
        stash: dict[int, tuple] = {}
        losses = []
        pending: list = []  # sends not yet posted: (tensor, dst, tag)

        def needs_recv(action):
            kind, _ = action
            return (kind == "F" and not self.is_first) or (kind == "B" and not self.is_last)

        for i, (kind, mb) in enumerate(actions):
            if kind == "F":
                if self.is_first:
                    x = xs[mb]
                else:
                    x = self._exchange(pending, self.prev, self.cfg.base_tag + mb).requires_grad_(True)
                if self.micro_batch_hook is not None:
                    self.micro_batch_hook(mb, mb % max(self.num_stages, 1))
                out = self.module(x)
                if self.is_last:
                    loss = loss_fn(out, ys[mb]) / M if loss_fn is not None else out.mean() / M
                    losses.append(loss.detach() * M)
                    stash[mb] = (x, loss)
                else:
                    pending.append((out.detach().contiguous(), self.next, self.cfg.base_tag + mb))
                    stash[mb] = (x, out)
            else:
                x, out = stash.pop(mb)
                if self.is_last:
                    out.backward()
                else:
                    g = self._exchange(pending, self.next, self.cfg.base_tag + 10000 + mb)
                    torch.autograd.backward(out, g)
                if not self.is_first:
                    pending.append((x.grad.contiguous(), self.prev, self.cfg.base_tag + 10000 + mb))
            # a send waits for the next action's receive (they travel as one batch); if the next action
            # receives nothing, post it now
            if pending and (i + 1 == len(actions) or not needs_recv(actions[i + 1])):
                self._exchange(pending, None)
        return torch.stack(losses).mean() if losses else None


def create_pipeline_stages(layers: list[torch.nn.Module], num_stages: int) -> list[torch.nn.Sequential]:
    """Contiguous equal split of ``layers`` (``crates/torsh-distributed/src/pipeline.rs:552-591``)."""
    per, rem = divmod(len(layers), num_stages)
    out, i = [], 0
    for s in range(num_stages):
        n = per + (1 if s < rem else 0)
        out.append(torch.nn.Sequential(*layers[i:i + n]))
        i += n
    return out
