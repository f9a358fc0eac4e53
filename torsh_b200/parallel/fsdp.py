"""Fully-sharded data parallel on flat units with fused NVSwitch kernels.

Reference surface (``crates/torsh-distributed/src/fsdp.rs``): ``FsdpConfig`` (``min_num_params`` 1000,
auto-wrap policy, sharding strategy, mixed precision, ``cpu_offload``, ``BackwardPrefetch``: ``:24-55``),
``ShardingStrategy {FullShard, ShardGradOp, NoShard, HybridShard}`` (``:72-81``), ``MixedPrecisionConfig``
(``:85-94``), shard arithmetic ``base + (rank < rem)`` (``:239-303``), ``fsdp_wrap`` (``:565-587``). The
reference shards each parameter separately and never un-shards; its "reduce-scatter" is
``all_reduce`` + slice followed by ``shard -= grad`` (``:373-419``).

Here a *unit* (one transformer block by default) is a contiguous range of a flat parameter space, and the
sharding strategy decides what of it stays resident on a rank:

``SHARD_GRAD_OP`` (:class:`ShardedFlatParameters`)
  * the bf16 parameters and the fp32 gradient accumulator of the whole model live in symmetric memory
    (every rank maps every other rank's copy; NVLS multicast addresses when the switch offers them);
  * fp32 master weights and both Adam moments exist only for the rank's own 1/world shard of each unit;
  * ONE kernel (``csrc/kernels/fsdp_fused_sm100.cu``) reduce-scatters the gradient in the switch, applies
    AdamW to the local shard and all-gathers the refreshed bf16 parameters by multicast stores.

``FULL_SHARD`` (:class:`FullShardParameters`)
  * only the rank's 1/world shard of every weight matrix is resident: bf16 shard (symmetric memory, so peers
    can read it), fp32 master and both moments;
  * a block is un-sharded into one of two rotating unit buffers right before its forward and again right before
    its backward, INSIDE the first GEMM that reads one of its weights (``tb_fsdp_ag_gemm``: copy CTAs of the
    same launch pull the shards over NVLink and publish per-chunk ready words that the GEMM's TMA producer
    waits on); the root unit (embeddings) is un-sharded once per step by a stand-alone gather;
  * after a block's backward its gradient (one of two rotating fp32 buffers in symmetric memory) is
    reduce-scattered and consumed by AdamW on the shard in one kernel on a side stream, under the backward
    pass of the next block; nothing is all-gathered afterwards;
  * one-dimensional parameters (biases, norm scales: 0.1 % of a transformer) stay replicated, as the reference keeps
    parameters below ``min_num_params`` whole; their gradients are all-reduced in one fused launch per step.

``NO_SHARD``: replicated parameters and optimizer state, one fused gradient all-reduce per step.
``HYBRID_SHARD``: ``FULL_SHARD`` inside ``group`` (one NVSwitch domain); replicas of that group are kept in step by
an NCCL all-reduce of the gradients over ``replica_group`` before the sharded step.
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
from ..optim.flat import FlatAdamW, FlatParameters
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
    # ---- FULL_SHARD only
    # How a block is un-sharded. "copy_engine": the DMA engines pull every rank's shard into the next block's buffer on a
    # side stream while the current block computes (no SM, no cross-rank barrier); "fused": inside the first GEMM that
    # reads the block (a copy warp in every CTA of that GEMM, per-chunk ready words); "kernel": a stand-alone gather
    # kernel right before the block. Measured on GPT-2-medium with 8 ranks the DMA prefetch is the
    # fastest: 32.1 ms per step (reduce-scatter overlapped) against 36.9 ms with the gather fused into the GEMMs.
    gather_mode: str = "copy_engine"
    fuse_gather: bool = True   # gather_mode "fused" (True) / "kernel" (False) when gather_mode is not "copy_engine"
    gather_ctas: int = 16      # copy CTAs inside that GEMM
    root_gather_ctas: int = 96 # copy CTAs of a stand-alone gather
    rs_blocks: int = 32        # CTAs of a block's reduce-scatter + AdamW kernel while it runs under the backward pass
    rs_threads: int = 512      # ... and threads per CTA
    # Each block's reduce-scatter + AdamW: True = on a side stream under the next block's backward, False = on the main
    # stream at full width, None = decide by group size. Measured on GPT-2-medium: with 8 ranks (gradients reduced in the
    # switch, AdamW on 1/8 of the block) 32 side-stream CTAs hide the transfer (32.1 ms against 34.5 ms serial); with 2
    # ranks the kernel is dominated by AdamW's own memory traffic and holding SMs for it costs more than running it
    # alone at full width (31.9 ms serial against 33.1 ms overlapped).
    overlap_rs: bool | None = None
    replica_group: object = None  # HYBRID_SHARD: the group that links the replicas of this rank's shard


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



CHUNK_ELEMS_MAX = 256 * 1024   # 512 KB of bf16 per gather chunk
CHUNK_ELEMS_MIN = 8 * 1024     # one 16 KB copy piece


def gather_chunk_elems(unit_len: int, world: int) -> int:
    """Chunk size (elements, a power of two) of a unit's gather: 512 KB unless that would leave a rank fewer than
    two chunks of a small unit."""
    c = CHUNK_ELEMS_MAX
    while c > CHUNK_ELEMS_MIN and 2 * c * world > unit_len:
        c //= 2
    return c


class _UnitLayout:
    """Offsets of a unit's sharded parameters inside its flat range, padded so that every rank owns whole chunks."""

    def __init__(self, params, world: int, chunk_elems: int | None = None):
        self.params = list(params)
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.chunk = chunk_elems or gather_chunk_elems(max(off, 1), world)
        q = self.chunk * world
        self.length = max(q, (off + q - 1) // q * q)
        self.shard = self.length // world
        self.cpr = self.shard // self.chunk          # chunks per rank


class FullShardParameters:
    """FULL_SHARD storage: resident shards, rotating un-shard / gradient workspaces, replicated small parameters."""

    N_ROT = 2

    def __init__(self, units: list[list[torch.nn.Parameter]], group, min_num_params: int = 1000, broadcast_from: int | None = 0):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        every = [p for u in units for p in u]
        self.params = every
        self.device = every[0].device
        is_small = lambda p: p.dim() < 2 or p.numel() < min_num_params
        self.small_params = [p for p in every if is_small(p)]
        big_units = [[p for p in u if not is_small(p)] for u in units]
        # unit 0 (root) has its own chunk size; the blocks share one so that they can share the rotating buffers
        blocks = big_units[1:]
        blk_chunk = gather_chunk_elems(min((sum((p.numel() + ALIGN - 1) // ALIGN * ALIGN for p in u) for u in blocks if u), default=1), self.world) if blocks else None
        self.layouts = [_UnitLayout(big_units[0], self.world)] + [_UnitLayout(u, self.world, blk_chunk) for u in blocks]
        self.shard_offsets, off = [], 0
        for lay in self.layouts:
            self.shard_offsets.append(off)
            off += lay.shard
        self.shard_total = off
        self.total = sum(lay.length for lay in self.layouts)
        dev = self.device
        # ---- resident: 1 / world of every unit
        self.shard_buf = SymmetricBuffer(self.shard_total, torch.bfloat16, group)
        self.shard_lowp = self.shard_buf.tensor
        self.master = torch.zeros(self.shard_total, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        # ---- workspaces: the root stays un-sharded for the whole step, the blocks rotate through N_ROT buffers
        max_blk = max((lay.length for lay in self.layouts[1:]), default=0)
        self.root_buf = torch.zeros(self.layouts[0].length, dtype=torch.bfloat16, device=dev)
        self.unit_bufs = [torch.zeros(max(max_blk, 8), dtype=torch.bfloat16, device=dev) for _ in range(self.N_ROT)]
        self.root_grad = SymmetricBuffer(self.layouts[0].length, torch.float32, group)
        self.unit_grads = [SymmetricBuffer(max(max_blk, 8), torch.float32, group) for _ in range(self.N_ROT)]
        # ready words + arrival counters of the gathers: one array for the root unit, one shared by the blocks (all
        # blocks have the same chunk count, so a word never changes its role between launches)
        blk_chunks = max((lay.length // lay.chunk for lay in self.layouts[1:]), default=1)
        if any(lay.length // lay.chunk != blk_chunks for lay in self.layouts[1:] if lay.params):
            raise TorshDistributedError.configuration_error("FULL_SHARD units inside a ModuleList must have equal sizes")
        self.ready_root = torch.zeros(2 * (self.layouts[0].length // self.layouts[0].chunk), dtype=torch.int32, device=dev)
        self.ready_blk = torch.zeros(2 * blk_chunks, dtype=torch.int32, device=dev)
        # per-rank pointers of every unit's shard (the gather's sources)
        es = 2
        self.shard_ptrs = []
        for so in self.shard_offsets:
            arr = (ctypes.c_void_p * 8)(*([pp + so * es for pp in self.shard_buf.peer_ptrs] + [0] * (8 - self.world)))
            self.shard_ptrs.append(arr)
        # ---- initial values: rank `broadcast_from`'s, unit by unit (no full-model fp32 copy is ever made)
        with torch.no_grad():
            for ui, lay in enumerate(self.layouts):
                full = torch.zeros(lay.length, dtype=torch.float32, device=dev)
                for p, o in zip(lay.params, lay.offsets):
                    full[o:o + p.numel()].copy_(p.detach().reshape(-1).float())
                if broadcast_from is not None and self.world > 1:
                    dist.broadcast(full, broadcast_from, group=group)
                so = self.shard_offsets[ui]
                mine = full[self.rank * lay.shard:(self.rank + 1) * lay.shard]
                self.master[so:so + lay.shard].copy_(mine)
                self.shard_lowp[so:so + lay.shard].copy_(mine)
                buf, gbuf = self.unit_buffer(ui), self.grad_buffer(ui).tensor
                buf[:lay.length].copy_(full)   # blocks that share a buffer overwrite each other: values come from the gather
                for p, o in zip(lay.params, lay.offsets):
                    p.data = buf[o:o + p.numel()].view(p.shape)
                    p.main_grad = gbuf[o:o + p.numel()].view(p.shape)
                    p.grad = None
                del full
            # ---- replicated small parameters: ordinary flat storage, gradient in symmetric memory for the all-reduce
            self.small = None
            if self.small_params:
                if broadcast_from is not None and self.world > 1:
                    for p in self.small_params:
                        dist.broadcast(p.data, broadcast_from, group=group)
                self.small = FlatParameters(self.small_params)
                self.small_grad_buf = SymmetricBuffer(self.small.total, torch.float32, group)
                self.small.grad = self.small_grad_buf.tensor
                for p, o in zip(self.small.params, self.small.offsets):
                    p.main_grad = self.small.grad[o:o + p.numel()].view(p.shape)
        torch.cuda.synchronize()
        dist.barrier(group)

    def slot(self, ui: int) -> int:
        return (ui - 1) % self.N_ROT

    def unit_buffer(self, ui: int) -> torch.Tensor:
        return self.root_buf if ui == 0 else self.unit_bufs[self.slot(ui)]

    def grad_buffer(self, ui: int) -> SymmetricBuffer:
        return self.root_grad if ui == 0 else self.unit_grads[self.slot(ui)]

    def ready_words(self, ui: int) -> torch.Tensor:
        return self.ready_root if ui == 0 else self.ready_blk

    def zero_grad(self):
        self.root_grad.tensor.zero_()
        for g in self.unit_grads:
            g.tensor.zero_()
        if self.small is not None:
            self.small.grad.zero_()

    def numel(self):
        return sum(p.numel() for p in self.params)

    @torch.no_grad()
    def full_lowp(self) -> torch.Tensor:
        """Every parameter as one bf16 vector (units in order, then the replicated small parameters), assembled with an
        NCCL all-gather of the shards: for checkpoints, evaluation and tests, not for the training step."""
        parts = []
        for ui, lay in enumerate(self.layouts):
            so = self.shard_offsets[ui]
            mine = self.shard_lowp[so:so + lay.shard].contiguous()
            full = torch.empty(lay.length, dtype=torch.bfloat16, device=self.device)
            if self.world > 1:
                dist.all_gather_into_tensor(full, mine, group=self.group)
            else:
                full.copy_(mine)
            parts.append(full)
        if self.small is not None:
            parts.append(self.small.lowp)
        return torch.cat(parts)

    @torch.no_grad()
    def full_state_dict(self, model: torch.nn.Module) -> dict:
        """name -> full bf16 tensor for every parameter of ``model`` (the module's own ``state_dict`` shows whichever
        block last used a rotating buffer)."""
        names = {id(p): n for n, p in model.named_parameters()}
        out = {}
        for ui, lay in enumerate(self.layouts):
            so = self.shard_offsets[ui]
            full = torch.empty(lay.length, dtype=torch.bfloat16, device=self.device)
            mine = self.shard_lowp[so:so + lay.shard].contiguous()
            if self.world > 1:
                dist.all_gather_into_tensor(full, mine, group=self.group)
            else:
                full.copy_(mine)
            for p, o in zip(lay.params, lay.offsets):
                out[names[id(p)]] = full[o:o + p.numel()].view(p.shape).clone()
        for p in self.small_params:
            out[names[id(p)]] = p.detach().clone()
        return out

    def memory_report(self) -> dict:
        """Bytes held on this rank, by role."""
        work = self.layouts[0].length + self.N_ROT * self.unit_bufs[0].numel()
        small = self.small.total if self.small is not None else 0
        return {"strategy": "full_shard", "world": self.world, "parameters": self.numel(),
                "param_shard_bytes": self.shard_total * 2, "optimizer_state_bytes": self.shard_total * 12,
                "unshard_workspace_bytes": work * 2, "grad_workspace_bytes": work * 4,
                "replicated_small_param_bytes": small * 18,
                "full_bf16_param_bytes": self.total * 2}


class FullShardAdamW:
    """Hyper-parameters and step counter of the FULL_SHARD step; the replicated small parameters have an ordinary
    :class:`FlatAdamW` that follows the same learning rate."""

    def __init__(self, flat: FullShardParameters, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01):
        self.flat, self.betas, self.eps, self.weight_decay = flat, betas, eps, weight_decay
        self.param_groups = [{"lr": lr, "params": flat.params}]
        self.step_count = 0
        self.dyn = torch.zeros(3, dtype=torch.float32, device=flat.device)
        self._dyn_host = torch.zeros(8, 3, dtype=torch.float32).pin_memory()
        self.small_opt = FlatAdamW(flat.small, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay) if flat.small is not None else None

    def get_lr(self):
        return [self.param_groups[0]["lr"]]

    def set_lr(self, lr):
        self.param_groups[0]["lr"] = lr

    def prepare_step(self):
        self.step_count += 1
        row = self._dyn_host[self.step_count % self._dyn_host.shape[0]]
        row[0] = self.param_groups[0]["lr"]
        row[1] = 1.0 - self.betas[0] ** self.step_count
        row[2] = 1.0 - self.betas[1] ** self.step_count
        self.dyn.copy_(row, non_blocking=True)
        if self.small_opt is not None:
            self.small_opt.set_lr(self.param_groups[0]["lr"])
            self.small_opt.prepare_step()

    def zero_grad(self, set_to_none: bool = False):
        self.flat.zero_grad()

    def state_dict(self) -> dict:
        """This rank's shard of the optimizer state (fp32 master, both moments) and the step count."""
        f = self.flat
        sd = {"step_count": self.step_count, "lr": self.param_groups[0]["lr"], "rank": f.rank, "world": f.world,
              "master": f.master.detach().cpu().clone(), "exp_avg": f.exp_avg.detach().cpu().clone(),
              "exp_avg_sq": f.exp_avg_sq.detach().cpu().clone()}
        if self.small_opt is not None:
            sd["small"] = self.small_opt.state_dict()
        return sd

    @torch.no_grad()
    def load_state_dict(self, sd: dict):
        f = self.flat
        if sd.get("world", f.world) != f.world or sd.get("rank", f.rank) != f.rank:
            raise TorshDistributedError.checkpoint_error("sharded optimizer state belongs to another rank / world size")
        self.step_count = int(sd["step_count"])
        self.param_groups[0]["lr"] = sd.get("lr", self.param_groups[0]["lr"])
        f.master.copy_(sd["master"]); f.exp_avg.copy_(sd["exp_avg"]); f.exp_avg_sq.copy_(sd["exp_avg_sq"])
        f.shard_lowp.copy_(f.master)      # the bf16 shard always mirrors the master copy
        if self.small_opt is not None and "small" in sd:
            self.small_opt.load_state_dict(sd["small"])


_SIG = [ctypes.c_void_p] * 8 + [ctypes.c_int64] * 3 + [ctypes.c_int] * 2 + [ctypes.c_void_p] + [ctypes.c_float] * 8 + [
    ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]


_SIG_FS = [ctypes.c_void_p] * 7 + [ctypes.c_int64] * 3 + [ctypes.c_int] * 2 + [ctypes.c_void_p] + [ctypes.c_float] * 6 + [
    ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
_SIG_GATHER = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_void_p] * 2


class FlatFSDP:
    """The FSDP engine used by :class:`torsh_b200.engine.CausalLMTrainer` (and usable on its own).

    ``flatten(model)`` moves the parameters into the storage of the configured strategy, ``optimizer(flat)`` returns
    the matching AdamW state holder, ``begin_step()`` opens a step (FULL_SHARD: un-shards the root unit) and
    ``reduce_and_step(flat, opt)`` after ``backward()`` reduces the gradients and applies the optimizer."""

    def __init__(self, group=None, config: FsdpConfig | None = None):
        self.group = group if group is not None else dist.group.WORLD
        self.cfg = config or FsdpConfig()
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.ctx = CommContext(self.group)          # reduce-scatter kernels (side stream)
        self.comm_stream = torch.cuda.Stream()
        self._pending: list[int] = []
        self._launched: set[int] = set()
        self._flat = None
        self._opt = None
        # FULL_SHARD state
        self.ctx_main = None                         # gathers (main stream)
        self.copy_stream = torch.cuda.Stream()       # DMA prefetch of the next block's parameters
        self._prefetched: dict[int, torch.cuda.Event] = {}
        self._resident: dict[int, int] = {}          # rotating buffer -> the block it holds, within one step
        self._direction = 1                          # +1 while the forward pass walks the blocks, -1 in backward
        self._comm_used = False
        self._pending_gather: int | None = None
        self._rs_done: dict[int, torch.cuda.Event] = {}
        self._begun = False
        self._small_coll = None
        mp = self.cfg.mixed_precision
        if mp.param_dtype != torch.bfloat16 or mp.reduce_dtype != torch.float32:
            # gradients are accumulated by the GEMM epilogues in fp32 and reduced in fp32 (in the switch), parameters
            # are bf16 views of fp32 masters; other combinations have no kernel here
            raise TorshDistributedError.feature_not_available(
                "FSDP mixed precision: param_dtype must be bfloat16 and reduce_dtype float32")
        if self.cfg.cpu_offload:
            raise TorshDistributedError.feature_not_available(
                "FsdpConfig.cpu_offload: use parallel.zero_offload.Zero3CpuOffloadManager for host-resident partitions")

    @property
    def strategy(self) -> ShardingStrategy:
        return self.cfg.sharding_strategy

    # ---- construction -----------------------------------------------------------------------------
    def flatten(self, model: torch.nn.Module, units=None):
        st = self.cfg.sharding_strategy
        units = units or default_units(model, self.cfg.min_num_params)
        self._model = model
        if st in (ShardingStrategy.FULL_SHARD, ShardingStrategy.HYBRID_SHARD):
            if st is ShardingStrategy.HYBRID_SHARD and self.cfg.replica_group is None:
                raise TorshDistributedError.configuration_error(
                    "HYBRID_SHARD needs FsdpConfig.replica_group (the ranks that hold the same shard in other groups)")
            flat = FullShardParameters(units, self.group, self.cfg.min_num_params)
            self._flat = flat
            self.ctx_main = CommContext(self.group)
            self._install_full_shard_hooks(model, units)
            return flat
        if st is ShardingStrategy.NO_SHARD:
            flat = ReplicatedFlatParameters([p for u in units for p in u], self.group)
            self._flat = flat
            return flat
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

    def optimizer(self, flat, **kw):
        if isinstance(flat, FullShardParameters):
            self._opt = FullShardAdamW(flat, **kw)
        elif isinstance(flat, ReplicatedFlatParameters):
            self._opt = FlatAdamW(flat, **kw)
        else:
            self._opt = ShardedAdamW(flat, **kw)
        return self._opt

    def memory_report(self) -> dict:
        f = self._flat
        if hasattr(f, "memory_report"):
            return f.memory_report()
        return {"strategy": "shard_grad_op", "world": self.world, "parameters": f.numel(),
                "param_shard_bytes": f.total * 2, "optimizer_state_bytes": f.shard_total * 12,
                "unshard_workspace_bytes": 0, "grad_workspace_bytes": f.total * 4,
                "replicated_small_param_bytes": 0, "full_bf16_param_bytes": f.total * 2}

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

    # ---- FULL_SHARD: hooks ---------------------------------------------------------------------------
    def _install_full_shard_hooks(self, model, units):
        flat = self._flat
        for ui, lay in enumerate(flat.layouts):
            for p in lay.params:
                p._tb_fsdp_unit = (self, ui)
        first_param_to_unit = {id(u[0]): i for i, u in enumerate(units) if i >= 1 and u}
        for m in model.modules():
            if isinstance(m, torch.nn.ModuleList):
                for child in m:
                    ps = list(child.parameters())
                    if ps and id(ps[0]) in first_param_to_unit:
                        ui = first_param_to_unit[id(ps[0])]
                        child.register_forward_pre_hook(self._fs_pre_forward(ui))
                        child.register_forward_hook(self._fs_post_forward(ui))
        # a forward outside the trainer (evaluation, generation) still needs the root unit
        model.register_forward_pre_hook(lambda module, args: self.begin_step())

    def _arm_gather(self, ui: int):
        if self._pending_gather is not None and self._pending_gather != ui:
            raise TorshDistributedError.internal_error(
                f"FSDP unit {self._pending_gather} was never un-sharded: no GEMM read one of its weights first "
                f"(set FsdpConfig.fuse_gather=False)")
        if not self._flat.layouts[ui].params:
            return
        if self.cfg.gather_mode == "copy_engine":
            return self._await_prefetch(ui)
        if self.cfg.fuse_gather:
            self._pending_gather = ui
        else:
            self._gather_unit(ui, self.cfg.root_gather_ctas)

    # ---- FULL_SHARD: DMA prefetch ----------------------------------------------------------------------
    def _prefetch(self, ui: int):
        """Queue the un-shard of block `ui` on the copy stream: one device-to-device copy per rank's shard, executed by
        the copy engines. It may start once the block that used the same rotating buffer last has finished (the copy
        stream waits for everything queued on the compute stream so far). No cross-rank barrier is needed: a rank's
        shard is only rewritten by that block's reduce-scatter + AdamW kernel, whose entry barrier every rank reaches
        after it has consumed this gather."""
        f = self._flat
        if ui < 1 or ui >= len(f.layouts) or not f.layouts[ui].params or ui in self._prefetched:
            return
        lay, so = f.layouts[ui], f.shard_offsets[ui]
        buf = f.unit_buffer(ui)
        cur = torch.cuda.current_stream()
        self.copy_stream.wait_stream(cur)
        with torch.cuda.stream(self.copy_stream):
            for k in range(self.world):
                q = (self.rank + k) % self.world          # own shard first, then the peers in ring order
                src = f.shard_buf.peer_tensor(q)[so:so + lay.shard]
                buf[q * lay.shard:(q + 1) * lay.shard].copy_(src, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        self._prefetched[ui] = ev
        self._resident.pop(f.slot(ui), None)

    def _await_prefetch(self, ui: int):
        slot = self._flat.slot(ui)
        if ui in self._prefetched:
            torch.cuda.current_stream().wait_event(self._prefetched.pop(ui))
        elif self._resident.get(slot) != ui:       # else: still whole from the forward pass (the deepest block)
            self._prefetch(ui)
            torch.cuda.current_stream().wait_event(self._prefetched.pop(ui))
        self._resident[slot] = ui
        # the neighbour in the direction of travel goes to the other rotating buffer while this block computes
        self._prefetch(ui + self._direction)

    def _fs_pre_forward(self, ui: int):
        def hook(module, args):
            self._direction = 1
            self._arm_gather(ui)
            if torch.is_grad_enabled():
                for a in args:
                    if isinstance(a, torch.Tensor) and a.requires_grad:
                        a.register_hook(lambda g, ui=ui: self._fs_backward_done(ui))
                        break
        return hook

    def _fs_post_forward(self, ui: int):
        def hook(module, args, output):
            if self._pending_gather == ui:
                raise TorshDistributedError.internal_error(
                    f"FSDP unit {ui} ran its forward without un-sharding: its first weight was not read by a GEMM "
                    f"(set FsdpConfig.fuse_gather=False)")
            out = output[0] if isinstance(output, (tuple, list)) else output
            if torch.is_grad_enabled() and isinstance(out, torch.Tensor) and out.requires_grad:
                out.register_hook(lambda g, ui=ui: self._fs_pre_backward(ui))
        return hook

    def _fs_pre_backward(self, ui: int):
        """The gradient w.r.t. the unit's output exists: its backward is about to start."""
        ev = self._rs_done.get(self._flat.slot(ui))
        if ev is not None:
            # the unit that used this gradient buffer last (two blocks deeper) must have been reduced and cleared
            torch.cuda.current_stream().wait_event(ev)
        self._direction = -1
        self._arm_gather(ui)

    def take_pending_gather(self, ui: int, weight: torch.Tensor, fusable: bool = True):
        """Called by the GEMM wrapper with the weight it is about to read. While the unit's un-shard is pending this
        returns the launch arguments that fuse it into that GEMM; when the GEMM cannot carry it (split-K, accumulating
        output, weight not a plain view of the unit buffer) the un-shard is launched on its own first. Else None."""
        if self._pending_gather != ui:
            return None
        self._pending_gather = None
        f = self._flat
        lay = f.layouts[ui]
        buf = f.unit_buffer(ui)
        b_off = weight.data_ptr() - buf.data_ptr()
        if not fusable or b_off < 0 or b_off + weight.numel() * 2 > lay.length * 2 or not weight.is_contiguous():
            self._gather_unit(ui, self.cfg.root_gather_ctas)   # not a plain view of the unit buffer: gather first
            return None
        return (f.shard_ptrs[ui], buf.data_ptr(), self.ctx_main.flags.ptr_array, self.ctx_main.epoch.data_ptr(),
                f.ready_words(ui).data_ptr(), lay.chunk * 2, lay.cpr, b_off, self.rank, self.world, self.cfg.gather_ctas)

    def _gather_unit(self, ui: int, ctas: int):
        f = self._flat
        lay = f.layouts[ui]
        if not lay.params:
            return
        st = nv.status_word(f.device)
        call("tb_fsdp_unit_gather", _SIG_GATHER, f.shard_ptrs[ui], f.unit_buffer(ui).data_ptr(),
             self.ctx_main.flags.ptr_array, self.ctx_main.epoch.data_ptr(), f.ready_words(ui).data_ptr(), lay.chunk * 2, lay.cpr,
             self.rank, self.world, ctas, st.data_ptr(), nv.stream_ptr())

    def begin_step(self):
        """Opens a step. FULL_SHARD: un-shards the root unit (embeddings, head) once; it stays whole until the step's
        reduce-scatter. Other strategies: nothing to do."""
        if not isinstance(self._flat, FullShardParameters) or self._begun:
            return
        self._begun = True
        self._gather_unit(0, self.cfg.root_gather_ctas)

    def _rs_unit(self, ui: int, stream, blocks: int, threads: int = 512):
        f, o = self._flat, self._opt
        lay = f.layouts[ui]
        if not lay.params:
            return
        gbuf = f.grad_buffer(ui)
        nvls = (gbuf.has_multicast and self.world > 2) if self.cfg.use_nvls is None else (self.cfg.use_nvls and gbuf.has_multicast)
        st = nv.status_word(f.device)
        call("tb_fsdp_rs_adamw", _SIG_FS, gbuf.ptr_array, self.ctx.flags.ptr_array, gbuf.mc(nvls), f.master.data_ptr(),
             f.exp_avg.data_ptr(), f.exp_avg_sq.data_ptr(), f.shard_lowp.data_ptr(), 0, lay.length, f.shard_offsets[ui],
             self.rank, self.world, self.ctx.epoch.data_ptr(), o.param_groups[0]["lr"], o.betas[0], o.betas[1], o.eps,
             o.weight_decay, 1.0 / self._grad_divisor(), o.dyn.data_ptr(), blocks, threads, st.data_ptr(), nv.stream_ptr(stream))

    def _grad_divisor(self) -> int:
        rg = self.cfg.replica_group
        return self.world * (dist.get_world_size(rg) if rg is not None else 1)

    def _fs_backward_done(self, ui: int):
        """The gradient w.r.t. the unit's input exists: all its parameter gradients have been launched."""
        if ui in self._launched or self._opt is None:
            return
        self._launched.add(ui)
        cur = torch.cuda.current_stream()
        if self.cfg.replica_group is not None:
            dist.all_reduce(self._flat.grad_buffer(ui).tensor[:self._flat.layouts[ui].length], group=self.cfg.replica_group)
        overlap = self.cfg.overlap_rs if self.cfg.overlap_rs is not None else self.world > 2
        if not overlap:
            self._rs_unit(ui, cur, self.cfg.tail_blocks)
            return
        self._comm_used = True
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream):
            self._rs_unit(ui, self.comm_stream, self.cfg.rs_blocks, self.cfg.rs_threads)
            ev = torch.cuda.Event()
            ev.record(self.comm_stream)
        self._rs_done[self._flat.slot(ui)] = ev

    def _full_shard_step(self, flat: FullShardParameters, opt):
        cur = torch.cuda.current_stream()
        todo = sorted((u for u in range(1, len(flat.layouts)) if u not in self._launched), reverse=True)
        if self._comm_used:
            cur.wait_stream(self.comm_stream)
            self._comm_used = False
        for ev in self._prefetched.values():      # a prefetch nobody consumed (e.g. past the first block in backward)
            cur.wait_event(ev)
        self._prefetched.clear()
        self._resident.clear()                    # the shards change below
        rg = self.cfg.replica_group
        for u in todo + [0]:
            if rg is not None:
                dist.all_reduce(flat.grad_buffer(u).tensor[:flat.layouts[u].length], group=rg)
            self._rs_unit(u, cur, self.cfg.tail_blocks)
        if flat.small is not None:
            if self._small_coll is None:
                from .collectives import FusedCollectives
                self._small_coll = FusedCollectives(self.group)
            if rg is not None:
                dist.all_reduce(flat.small.grad, group=rg)
            if self.world > 1:
                self._small_coll.all_reduce_(flat.small_grad_buf, scale=1.0)
            opt.small_opt.launch(grad_scale=1.0 / self._grad_divisor())
        self._launched.clear()
        self._rs_done.clear()
        self._pending_gather = None
        self._begun = False

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

    def reduce_and_step(self, flat, opt):
        """Call after ``backward()``: launches whatever has not been handed to the comm stream yet
        (unit 0 always, every unit when overlap is off) and joins the comm stream."""
        self._flat, self._opt = flat, opt
        if isinstance(flat, FullShardParameters):
            return self._full_shard_step(flat, opt)
        if isinstance(flat, ReplicatedFlatParameters):
            return flat.all_reduce_and_step(opt)
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


class ReplicatedFlatParameters(FlatParameters):
    """NO_SHARD: every rank keeps the whole flat mixed-precision state; the gradient buffer lives in symmetric memory and
    is summed over the ranks by one fused all-reduce launch per step."""

    def __init__(self, params, group):
        from .collectives import FusedCollectives
        params = list(params)
        if dist.get_world_size(group) > 1:
            for p in params:
                dist.broadcast(p.data, 0, group=group)
        super().__init__(params)
        self.group, self.world = group, dist.get_world_size(group)
        self.grad_buf = SymmetricBuffer(self.total, torch.float32, group)
        self.grad = self.grad_buf.tensor
        for p, o in zip(self.params, self.offsets):
            p.main_grad = self.grad[o:o + p.numel()].view(p.shape)
        self._coll = FusedCollectives(group)

    def all_reduce_and_step(self, opt):
        if self.world > 1:
            self._coll.all_reduce_(self.grad_buf, scale=1.0)
        opt.launch(grad_scale=1.0 / self.world)

    def memory_report(self) -> dict:
        return {"strategy": "no_shard", "world": self.world, "parameters": self.numel(), "param_shard_bytes": self.total * 2,
                "optimizer_state_bytes": self.total * 12, "unshard_workspace_bytes": 0, "grad_workspace_bytes": self.total * 4,
                "replicated_small_param_bytes": 0, "full_bf16_param_bytes": self.total * 2}


def fsdp_wrap(model: torch.nn.Module, group=None, config: FsdpConfig | None = None):
    """``fsdp_wrap(module, pg, cfg)`` (``crates/torsh-distributed/src/fsdp.rs:565-573``): returns
    ``(engine, flat_parameters)``; parameters of ``model`` become views into the symmetric flat buffers."""
    eng = FlatFSDP(group, config)
    return eng, eng.flatten(model)
