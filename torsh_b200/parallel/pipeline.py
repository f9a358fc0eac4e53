"""Pipeline parallelism: GPipe and 1F1B over point-to-point sends (NCCL p2p on GPUs, gloo on CPU).

Reference (``crates/torsh-distributed/src/pipeline.rs``): schedules ``GPipe / OneFOneBInterleaved /
InterleavedOneFOneB`` (``:18-25``), ``PipelineConfig`` with ``num_micro_batches 4``, ``base_tag 1000``, timeout 30 s
(``:29-55``), stage = prev/next rank (``:58-116``), GPipe forward (``:206-251``), 1F1B warm-up / steady / cool-down
(``:254-340``), micro-batch split along dim 0 (``:410-429``), tags ``base + mb`` forward and ``base + 10000 + mb``
backward (``:350-384``). There send/recv are no-ops and the backward uses mock gradients.

Here the per-stage action list comes from the native planner (GPipe, 1F1B and the real interleaved 1F1B over virtual
stages); every forward stashes its input and output so the matching backward can run ``torch.autograd.backward`` with
the received gradient. Every directed link has its own two-rank process group (on NCCL: its own communicator and
stream), receives are posted ahead of the action that consumes them and waited for only there, and sends are never
waited for inside the step, so the transfers overlap this stage's compute.
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
    # every rank holds several model chunks (virtual stages); the reference names this schedule and executes plain
    # 1F1B for it (pipeline.rs:343-347), here it is the real interleaved schedule
    INTERLEAVED_ONE_F_ONE_B = "interleaved"


@dataclass
class PipelineConfig:
    num_micro_batches: int = 4
    schedule: ScheduleType = ScheduleType.ONE_F_ONE_B
    base_tag: int = 1000
    timeout_s: float = 30.0
    # overlap=True: every directed link (activations to the next stage, gradients to the previous one) gets its own
    # two-rank process group, receives are posted `recv_lookahead` actions ahead of their use and sends are not waited
    # for until the end of the step, so transfers run on the link's own stream under this stage's compute.
    # overlap=False: sends and the receive they are paired with travel as one blocking batch.
    overlap: bool = True
    # How many actions ahead of its use a receive may be posted. A receive is never posted before every action of THIS
    # rank that the incoming tensor depends on has been issued (the forward of the same micro-batch for a gradient, the
    # previous chunk's forward for a wrapped-around activation). On CUDA the default is 0 (post where the tensor is
    # consumed): an NCCL receive is a kernel that holds SMs while it waits, and the persistent GEMMs of the action that
    # runs meanwhile deal their tiles statically to one CTA per SM, so a parked receive stalls them until the sender
    # delivers (and deadlocks when the sender is waiting for this rank's output). None = 2 on CPU, 0 on CUDA.
    recv_lookahead: int | None = None
    measure_idle: bool = False   # record events around every action; idle_ms() then gives the device idle time of the last step


class PipelineParallel:
    """One pipeline rank. ``stage_module`` maps the previous stage's activation (or the raw input on the first virtual
    stage) to this stage's activation; on the last virtual stage ``loss_fn(output, target)`` produces the micro-batch
    loss. A list of modules makes the rank hold several chunks (virtual stages ``chunk * num_stages + stage``) for the
    interleaved schedule."""

    def __init__(self, stage_module, group=None, config: PipelineConfig | None = None,
                 activation_shape=None, activation_dtype=torch.float32, prev_rank: int | None = None,
                 next_rank: int | None = None):
        self.cfg = config or PipelineConfig()
        self.group = group
        g = group if group is not None else dist.group.WORLD
        self.stage, self.num_stages = dist.get_rank(g), dist.get_world_size(g)
        self.chunks = list(stage_module) if isinstance(stage_module, (list, tuple, torch.nn.ModuleList)) else [stage_module]
        self.module = self.chunks[0]
        self.num_chunks = len(self.chunks)
        if self.num_chunks > 1 and self.cfg.schedule is not ScheduleType.INTERLEAVED_ONE_F_ONE_B:
            raise ValueError("several model chunks per rank need ScheduleType.INTERLEAVED_ONE_F_ONE_B")
        ranks = dist.get_process_group_ranks(g)
        P = self.num_stages
        wrap = self.num_chunks > 1
        self.prev = prev_rank if prev_rank is not None else (ranks[(self.stage - 1) % P] if (self.stage > 0 or wrap) else None)
        self.next = next_rank if next_rank is not None else (ranks[(self.stage + 1) % P] if (self.stage + 1 < P or wrap) else None)
        self.act_shape, self.act_dtype = activation_shape, activation_dtype
        self.device = next(self.chunks[0].parameters()).device
        self.stats = {"sends": 0, "recvs": 0, "bubbles": 0}
        # called as hook(micro_batch_index, in_flight_slot) before each forward: lets layers that keep per-micro-batch
        # buffers (the fused tensor-parallel layers) switch to the slot of this micro-batch
        self.micro_batch_hook = None
        self._links: dict = {}
        self._marks: list = []
        if self.cfg.overlap and P > 1:
            self._make_links(dist.get_rank())

    # ---- topology -------------------------------------------------------------------------------------
    @property
    def total_virtual(self) -> int:
        return self.num_stages * self.num_chunks

    def _vs(self, chunk: int) -> int:
        return chunk * self.num_stages + self.stage

    @property
    def is_first(self):
        return self.stage == 0

    @property
    def is_last(self):
        return self.stage == self.num_stages - 1

    def _make_links(self, me: int):
        """One two-rank group per directed link this rank takes part in: ("act", src, dst) carries activations,
        ("grad", src, dst) gradients. Both ends create their common groups in the same (sorted) order."""
        keys = set()
        for a, b in ((self.prev, me), (me, self.next)):
            if a is None or b is None or a == b:
                continue
            keys.add(("act", a, b))
            keys.add(("grad", b, a))
        for key in sorted(keys):
            _, a, b = key
            try:
                self._links[key] = dist.new_group(sorted((a, b)), use_local_synchronization=True)
            except Exception:
                self._links = {}
                self.cfg.overlap = False   # fall back to the blocking paired exchange
                return

    @staticmethod
    def split_micro_batches(t: torch.Tensor, n: int) -> list[torch.Tensor]:
        return list(t.chunk(n, 0))

    # ---- blocking exchange (overlap=False) -------------------------------------------------------------
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

    # ---- schedule -------------------------------------------------------------------------------------
    def actions(self) -> list[tuple[str, int, int]]:
        M = self.cfg.num_micro_batches
        if self.cfg.schedule is ScheduleType.INTERLEAVED_ONE_F_ONE_B and self.num_chunks > 1:
            return planner.pipeline_schedule_interleaved(self.stage, self.num_stages, M, self.num_chunks)
        sched = "gpipe" if self.cfg.schedule is ScheduleType.GPIPE else "1f1b"
        return [(k, mb, 0) for k, mb in planner.pipeline_schedule(sched, self.stage, self.num_stages, M)]

    def _recv_spec(self, action):
        """(kind, source rank, tag) of the tensor an action needs from a neighbour, or None."""
        kind, mb, c = action
        vs, T = self._vs(c), self.total_virtual
        if kind == "F" and vs > 0:
            return ("act", self.prev, self.cfg.base_tag + mb * T + vs)
        if kind == "B" and vs < T - 1:
            return ("grad", self.next, self.cfg.base_tag + 10000 + mb * T + vs)
        return None

    def train_step(self, inputs: torch.Tensor | None, targets: torch.Tensor | None, loss_fn=None) -> torch.Tensor | None:
        """Runs all micro-batches through this rank's chunks; gradients accumulate in the parameters.
        Returns the mean micro-batch loss on the rank that holds the last virtual stage, ``None`` elsewhere."""
        if self.cfg.overlap and self._links:
            return self._train_step_overlapped(inputs, targets, loss_fn)
        if self.num_chunks > 1:
            raise RuntimeError("the interleaved schedule needs PipelineConfig.overlap=True (per-link process groups)")
        return self._train_step_blocking(inputs, targets, loss_fn)

    def _train_step_overlapped(self, inputs, targets, loss_fn):
        M, T, me = self.cfg.num_micro_batches, self.total_virtual, dist.get_rank()
        acts = self.actions()
        holds_first = self.stage == 0
        holds_last = self.stage == self.num_stages - 1
        xs = self.split_micro_batches(inputs, M) if (holds_first and inputs is not None) else None
        ys = self.split_micro_batches(targets, M) if (holds_last and targets is not None) else None
        stash: dict[tuple[int, int], tuple] = {}
        losses, posted, sends = [], {}, []
        timing = self.cfg.measure_idle and self.device.type == "cuda"
        marks = []

        index_of = {a: j for j, a in enumerate(acts)}
        lookahead = self.cfg.recv_lookahead
        if lookahead is None:
            lookahead = 0 if self.device.type == "cuda" else 2

        def own_dependency(j):
            """Index of the last action of this rank that the tensor received for action j depends on (-1: none)."""
            kind, mb, c = acts[j]
            if kind == "B":
                return index_of[("F", mb, c)]
            return index_of[("F", mb, c - 1)] if c > 0 else -1

        def post_recv(i, issued=-1):
            spec = self._recv_spec(acts[i])
            if spec is None or i in posted or own_dependency(i) > issued:
                return
            kind, src, tag = spec
            buf = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
            grp = self._links[(kind, src, me)]
            posted[i] = (dist.irecv(buf, src, group=grp, tag=tag), buf)
            self.stats["recvs"] += 1

        def send(kind, t, dst, tag):
            grp = self._links[(kind, me, dst)]
            sends.append((dist.isend(t, dst, group=grp, tag=tag), t))   # the tensor stays referenced until the send is done
            self.stats["sends"] += 1

        for i, (kind, mb, c) in enumerate(acts):
            # actions 0 .. i-1 have been issued: post what may be posted up to `lookahead` actions ahead
            for j in range(i, min(i + lookahead, len(acts) - 1) + 1):
                post_recv(j, issued=i - 1)
            got = None
            if i in posted:
                w, got = posted.pop(i)
                w.wait()
            vs = self._vs(c)
            if timing:
                e0 = torch.cuda.Event(enable_timing=True); e0.record()
            if kind == "F":
                x = xs[mb] if vs == 0 else got.requires_grad_(True)
                if self.micro_batch_hook is not None:
                    self.micro_batch_hook(mb, mb % max(self.num_stages, 1))
                out = self.chunks[c](x)
                if vs == T - 1:
                    loss = loss_fn(out, ys[mb]) / M if loss_fn is not None else out.mean() / M
                    losses.append(loss.detach() * M)
                    stash[(mb, c)] = (x, loss)
                else:
                    send("act", out.detach().contiguous(), self.next, self.cfg.base_tag + mb * T + vs + 1)
                    stash[(mb, c)] = (x, out)
            else:
                x, out = stash.pop((mb, c))
                if vs == T - 1:
                    out.backward()
                else:
                    torch.autograd.backward(out, got)
                if vs > 0:
                    send("grad", x.grad.contiguous(), self.prev, self.cfg.base_tag + 10000 + mb * T + vs - 1)
            if timing:
                e1 = torch.cuda.Event(enable_timing=True); e1.record()
                marks.append((e0, e1))
            if len(sends) > 16:
                sends[:] = [(w, t) for w, t in sends if not w.is_completed()]
        for w, _ in sends:
            w.wait()
        self._marks = marks
        return torch.stack(losses).mean() if losses else None

    def idle_ms(self) -> float | None:
        """Device time between the first action's start and the last action's end of the last step that no action
        covered (the pipeline bubble plus exposed transfers), with ``measure_idle`` on. Synchronises."""
        if not self._marks:
            return None
        torch.cuda.synchronize()
        span = self._marks[0][0].elapsed_time(self._marks[-1][1])
        busy = sum(a.elapsed_time(b) for a, b in self._marks)
        return max(span - busy, 0.0)

    def _train_step_blocking(self, inputs, targets, loss_fn):
        M = self.cfg.num_micro_batches
        actions = [(k, mb) for k, mb, _ in self.actions()]
        first, last = self.stage == 0, self.stage == self.num_stages - 1
        xs = self.split_micro_batches(inputs, M) if first else None
        ys = self.split_micro_batches(targets, M) if (last and targets is not None) else None
        stash: dict[int, tuple] = {}
        losses = []
        pending: list = []  # sends not yet posted: (tensor, dst, tag)
        timing = self.cfg.measure_idle and self.device.type == "cuda"
        marks = []

        def mark():
            if timing:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                return e

        def needs_recv(action):
            kind, _ = action
            return (kind == "F" and not first) or (kind == "B" and not last)

        for i, (kind, mb) in enumerate(actions):
            if kind == "F":
                if first:
                    x = xs[mb]
                else:
                    x = self._exchange(pending, self.prev, self.cfg.base_tag + mb).requires_grad_(True)
                if self.micro_batch_hook is not None:
                    self.micro_batch_hook(mb, mb % max(self.num_stages, 1))
                e0 = mark()
                out = self.module(x)
                if last:
                    loss = loss_fn(out, ys[mb]) / M if loss_fn is not None else out.mean() / M
                    losses.append(loss.detach() * M)
                    stash[mb] = (x, loss)
                else:
                    pending.append((out.detach().contiguous(), self.next, self.cfg.base_tag + mb))
                    stash[mb] = (x, out)
                e1 = mark()
            else:
                x, out = stash.pop(mb)
                if last:
                    e0 = mark()
                    out.backward()
                else:
                    g = self._exchange(pending, self.next, self.cfg.base_tag + 10000 + mb)
                    e0 = mark()
                    torch.autograd.backward(out, g)
                if not first:
                    pending.append((x.grad.contiguous(), self.prev, self.cfg.base_tag + 10000 + mb))
                e1 = mark()
            if timing:
                marks.append((e0, e1))
            # a send waits for the next action's receive (they travel as one batch); if the next action
            # receives nothing, post it now
            if pending and (i + 1 == len(actions) or not needs_recv(actions[i + 1])):
                self._exchange(pending, None)
        self._marks = marks
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
