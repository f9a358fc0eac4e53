"""Fully-sharded data parallel on flat units with fused NVSwitch kernels.

Reference surface (``crates/torsh-distributed/src/fsdp.rs``): ``FsdpConfig`` (``min_num_params`` 1000,
auto-wrap policy, sharding strategy, mixed precision, ``cpu_offload``, ``BackwardPrefetch``: ``:24-55``),
``ShardingStrategy {FullShard, ShardGradOp, NoShard, HybridShard}`` (``:72-81``), ``MixedPrecisionConfig``
(``:85-94``), shard arithmetic ``base + (rank < rem)`` (``:239-303``), ``fsdp_wrap`` (``:565-587``). The
reference shards each parameter separately and never un-shards; its "reduce-scatter" is
``all_reduce`` + slice followed by ``shard -= grad`` (``:373-419``).

Here a *unit* (one transformer block by default) is a contiguous range of a flat parameter space:

* the bf16 parameters and the fp32 gradient accumulator of the whole model live in symmetric memory
  (every rank maps every other rank's copy; NVLS multicast addresses when the switch offers them);
* fp32 master weights and both Adam moments exist only for the rank's own 1/world shard of each unit;
* after a unit's backward, ONE kernel (``csrc/kernels/fsdp_fused_sm100.cu``) reduce-scatters the unit's
  gradient in the switch, applies AdamW to the local shard and all-gathers the refreshed bf16
  parameters by multicast stores; it runs on a side stream under the rest of the backward pass.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from enum import Enum

import torch
import torch.distributed as dist

from ..core.error import TorshDistributedError

from .. import _native as nv
from ..ops._dispatch import call
from .symm import CommContext, SymmetricBuffer

ALIGN = 128


class ShardingStrategy(Enum):
    FULL_SHARD = "full_shard"
    SHARD_GRAD_OP = "shard_grad_op"
    NO_SHARD = "no_shard"
    HYBRID_SHARD = "hybrid_shard"


class BackwardPrefetch(Enum):
    BACKWARD_PRE = "backward_pre"
    BACKWARD_POST = "backward_post"
    NONE = "none"


@dataclass
class MixedPrecisionConfig:
    param_dtype: torch.dtype = torch.bfloat16
    reduce_dtype: torch.dtype = torch.float32
    buffer_dtype: torch.dtype = torch.float32
    keep_low_precision_grads: bool = False


@dataclass
class FsdpConfig:
    min_num_params: int = 1000
    auto_wrap_policy: str = "module_list"
    sharding_strategy: ShardingStrategy = ShardingStrategy.FULL_SHARD
    mixed_precision: MixedPrecisionConfig = field(default_factory=MixedPrecisionConfig)
    cpu_offload: bool = False
    backward_prefetch: BackwardPrefetch = BackwardPrefetch.BACKWARD_PRE
    # overlap=True hands each block's fused reduce-scatter + AdamW + all-gather kernel to a side stream from a backward
    # hook; overlap=False runs the whole model as one fused launch after backward. Measured on GPT-2-medium, 2 B200s:
    # 30.8 ms per step with overlap (the 64 co-resident CTAs slow the statically scheduled GEMM tiles of the SMs they
    # share, and 25 barrier-separated launches cost 1.2 ms even with a single rank), 30.0 ms without.
    overlap: bool = False
    coarse_units: int = 0      # with overlap: merge the per-block units into this many groups (0 = one unit per block)
    comm_blocks: int = 64      # CTAs while overlapping backward (measured on 2 B200s: 16 -> 32.1 ms, 32 -> 31.0, 64 -> 30.1 per step)
    tail_blocks: int = 296     # CTAs of the units that are reduced after backward has finished
    use_nvls: bool | None = None


def shard_range(numel: int, world: int, rank: int) -> tuple[int, int]:
    """The reference's per-parameter split: ``base + (rank < rem)`` elements for rank ``rank``
    (``crates/torsh-distributed/src/fsdp.rs:239-303``)."""
    base, rem = divmod(numel, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def default_units(model: torch.nn.Module, min_num_params: int = 1000) -> list[list[torch.nn.Parameter]]:
    """Unit 0 = everything outside ``ModuleList`` children (embeddings, final norm, head); then one unit per
    element of every ``ModuleList`` whose parameter count reaches ``min_num_params``."""
    in_list: set[int] = set()
    units: list[list[torch.nn.Parameter]] = []
    for m in model.modules():
        if isinstance(m, torch.nn.ModuleList):
            for child in m:
                ps = [p for p in child.parameters() if id(p) not in in_list]
                if sum(p.numel() for p in ps) >= min_num_params:
                    units.append(ps)
                    in_list.update(id(p) for p in ps)
    rest, seen = [], set()
    for p in model.parameters():
        if id(p) not in in_list and id(p) not in seen:
            rest.append(p)
            seen.add(id(p))
    return [rest] + units


class ShardedFlatParameters:
    def __init__(self, units: list[list[torch.nn.Parameter]], group, broadcast_from: int | None = 0):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.params = [p for u in units for p in u]
        self.device = self.params[0].device
        unit_align = ALIGN * self.world
        self.unit_ranges: list[tuple[int, int]] = []
        self.offsets: list[int] = []
        off = 0
        for u in units:
            start = off
            for p in u:
                self.offsets.append(off)
                off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            off = (off + unit_align - 1) // unit_align * unit_align
            self.unit_ranges.append((start, off - start))
        self.total = off
        self.lowp_buf = SymmetricBuffer(self.total, torch.bfloat16, group)
        self.grad_buf = SymmetricBuffer(self.total, torch.float32, group)
        self.lowp, self.grad = self.lowp_buf.tensor, self.grad_buf.tensor
        self.shard_total = self.total // self.world
        self.master = torch.zeros(self.shard_total, dtype=torch.float32, device=self.device)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        with torch.no_grad():
            full = torch.zeros(self.total, dtype=torch.float32, device=self.device)
            for p, o in zip(self.params, self.offsets):
                full[o:o + p.numel()].copy_(p.detach().reshape(-1).float())
            if broadcast_from is not None:
                dist.broadcast(full, broadcast_from, group=group)
            self.lowp.copy_(full)
            for (uo, ul) in self.unit_ranges:
                sh = ul // self.world
                so = uo // self.world
                self.master[so:so + sh].copy_(full[uo + self.rank * sh: uo + (self.rank + 1) * sh])
            for p, o in zip(self.params, self.offsets):
                p.data = self.lowp[o:o + p.numel()].view(p.shape)
                p.main_grad = self.grad[o:o + p.numel()].view(p.shape)
                p.grad = None
        torch.cuda.synchronize()
        dist.barrier(group)

    def zero_grad(self):
        self.grad.zero_()

    def numel(self):
        return sum(p.numel() for p in self.params)


class ShardedAdamW:
    """Hyper-parameters and step counter of the fused FSDP step (the state lives in the flat shards)."""

    def __init__(self, flat: ShardedFlatParameters, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01):
        self.flat, self.betas, self.eps, self.weight_decay = flat, betas, eps, weight_decay
        self.param_groups = [{"lr": lr, "params": flat.params}]
        self.step_count = 0
        self.dyn = torch.zeros(3, dtype=torch.float32, device=flat.device)
        self._dyn_host = torch.zeros(8, 3, dtype=torch.float32).pin_memory()

    def get_lr(self):
        return [self.param_groups[0]["lr"]]

    def set_lr(self, lr):
        self.param_groups[0]["lr"] = lr

    def prepare_step(self):
        self.step_count += 1
        # one pinned row per step in flight: the asynchronous upload of an earlier step may not have run yet
        row = self._dyn_host[self.step_count % self._dyn_host.shape[0]]
        row[0] = self.param_groups[0]["lr"]
        row[1] = 1.0 - self.betas[0] ** self.step_count
        row[2] = 1.0 - self.betas[1] ** self.step_count
        self.dyn.copy_(row, non_blocking=True)

    def zero_grad(self, set_to_none: bool = False):
        self.flat.zero_grad()


_SIG = [ctypes.c_void_p] * 8 + [ctypes.c_int64] * 3 + [ctypes.c_int] * 2 + [ctypes.c_void_p] + [ctypes.c_float] * 8 + [
    ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]


class FlatFSDP:
    """The FSDP engine used by :class:`torsh_b200.engine.CausalLMTrainer` (and usable on its own)."""

    def __init__(self, group=None, config: FsdpConfig | None = None):
        self.group = group if group is not None else dist.group.WORLD
        self.cfg = config or FsdpConfig()
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.ctx = CommContext(self.group)
        self.comm_stream = torch.cuda.Stream()
        self._pending: list[int] = []
        self._launched: set[int] = set()
        self._flat = None
        self._opt = None

    # ---- construction -----------------------------------------------------------------------------
    def flatten(self, model: torch.nn.Module, units=None) -> ShardedFlatParameters:
        st = self.cfg.sharding_strategy
        if st is not ShardingStrategy.FULL_SHARD:
            # This engine keeps a replicated bf16 copy of the parameters and shards fp32 masters, moments and the
            # reduction work, which is what SHARD_GRAD_OP describes; FULL_SHARD differs only in when the bf16 copy is
            # refreshed (here: by the optimizer kernel itself), so both run the same kernel. NO_SHARD is plain data
            # parallelism (use DistributedDataParallel) and HYBRID_SHARD needs a second, inter-node group.
            if st is ShardingStrategy.NO_SHARD:
                raise TorshDistributedError.configuration_error("NO_SHARD: use parallel.DistributedDataParallel")
            if st is ShardingStrategy.HYBRID_SHARD and dist.get_world_size(self.group) > 8:
                raise TorshDistributedError.feature_not_available(
                    "HYBRID_SHARD across nodes: shard inside one NVSwitch group and wrap it in DDP across groups")
        units = units or default_units(model, self.cfg.min_num_params)
        if not self.cfg.overlap:
            # nothing runs before backward has finished, so the whole model is ONE unit: one launch, one pair of
            # cross-rank barriers and one pass at full width instead of a barrier-separated kernel per block
            units = [[p for u in units for p in u]]
        elif self.cfg.coarse_units and len(units) > 2:
            # merge the per-block units (units[1:], in depth order) into a few contiguous groups: the deepest group is
            # handed to the comm stream when backward has passed its first block and overlaps the rest of backward
            k = min(self.cfg.coarse_units, len(units) - 1)
            blocks = units[1:]
            per = (len(blocks) + k - 1) // k
            units = [units[0]] + [[p for u in blocks[i:i + per] for p in u] for i in range(0, len(blocks), per)]
        flat = ShardedFlatParameters(units, self.group)
        self._flat = flat
        if self.cfg.overlap:
            self._install_hooks(model, units)
        return flat

    def optimizer(self, flat, **kw) -> ShardedAdamW:
        self._opt = ShardedAdamW(flat, **kw)
        return self._opt

    def _install_hooks(self, model, units):
        """When the gradient w.r.t. a unit's input exists, every parameter gradient of that unit has been
        launched: hand the unit to the comm stream at that point."""
        # with coarse groups the shallowest one finishes with backward itself: it runs afterwards at full width
        first = 2 if self.cfg.coarse_units else 1
        first_param_to_unit = {id(u[0]): i for i, u in enumerate(units) if i >= first and u}
        for m in model.modules():
            if isinstance(m, torch.nn.ModuleList):
                for child in m:
                    ps = list(child.parameters())
                    if ps and id(ps[0]) in first_param_to_unit:
                        ui = first_param_to_unit[id(ps[0])]
                        child.register_forward_pre_hook(self._make_pre_hook(ui))

    def _make_pre_hook(self, ui: int):
        def pre_hook(module, args):
            for a in args:
                if isinstance(a, torch.Tensor) and a.requires_grad and torch.is_grad_enabled():
                    a.register_hook(lambda g, ui=ui: self._unit_backward_done(ui))
                    break
        return pre_hook

    # ---- per-unit fused step --------------------------------------------------------------------------
    def _launch_unit(self, ui: int, stream, blocks: int | None = None):
        f, o = self._flat, self._opt
        uo, ul = f.unit_ranges[ui]
        # in-switch reduction / multicast by default only beyond two ranks (with two, plain peer loads and stores move
        # half the bytes over each link: a multicast store also returns the sender's own copy)
        have_mc = f.grad_buf.has_multicast and f.lowp_buf.has_multicast
        nvls = (have_mc and self.world > 2) if self.cfg.use_nvls is None else (self.cfg.use_nvls and have_mc)
        st = nv.status_word(f.device)
        call("tb_fsdp_rs_adamw_ag", _SIG, f.grad_buf.ptr_array, f.lowp_buf.ptr_array, self.ctx.flags.ptr_array,
             f.grad_buf.mc(nvls), f.lowp_buf.mc(nvls), f.master.data_ptr(), f.exp_avg.data_ptr(), f.exp_avg_sq.data_ptr(),
             uo, ul, uo // self.world, self.rank, self.world, self.ctx.epoch.data_ptr(), o.param_groups[0]["lr"],
             o.betas[0], o.betas[1], o.eps, o.weight_decay, 1.0, 1.0, 1.0 / self.world, o.dyn.data_ptr(),
             blocks or self.cfg.comm_blocks, st.data_ptr(), nv.stream_ptr(stream))

    def _unit_backward_done(self, ui: int):
        if ui in self._launched or self._opt is None:
            return
        self._launched.add(ui)
        cur = torch.cuda.current_stream()
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            self._launch_unit(ui, self.comm_stream)

    def reduce_and_step(self, flat: ShardedFlatParameters, opt: ShardedAdamW):
        """Call after ``backward()``: launches whatever has not been handed to the comm stream yet
        (unit 0 always, every unit when overlap is off) and joins the comm stream."""
        self._flat, self._opt = flat, opt
        cur = torch.cuda.current_stream()
        todo = [u for u in range(len(flat.unit_ranges)) if u not in self._launched]
        # same order on every rank (all ranks share one flag array): descending, as backward visits them
        todo.sort(reverse=True)
        # these units run after the backward pass with nothing left to overlap: give them the whole GPU
        # (two CTAs per SM) instead of the few CTAs that share the SMs with backward kernels
        tail_blocks = self.cfg.tail_blocks
        if self._launched:
            self.comm_stream.wait_stream(cur)
            with torch.cuda.stream(self.comm_stream):
                for u in todo:
                    self._launch_unit(u, self.comm_stream, tail_blocks)
            cur.wait_stream(self.comm_stream)
        else:
            for u in todo:
                self._launch_unit(u, cur, tail_blocks)
        self._launched.clear()


def fsdp_wrap(model: torch.nn.Module, group=None, config: FsdpConfig | None = None):
    """``fsdp_wrap(module, pg, cfg)`` (``crates/torsh-distributed/src/fsdp.rs:565-573``): returns
    ``(engine, flat_parameters)``; parameters of ``model`` become views into the symmetric flat buffers."""
    eng = FlatFSDP(group, config)
    return eng, eng.flatten(model)
