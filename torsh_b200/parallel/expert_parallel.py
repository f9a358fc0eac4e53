"""Mixture-of-experts routing and expert parallelism.

Router (``crates/torsh-distributed/src/expert_parallelism/router.rs:231-448``): gate linear → softmax → top-k →
capacity ``ceil(tokens·k/E · capacity_factor)`` with dropped tokens, load-balance loss (coefficient of variation of the
expert loads) and z-loss (mean squared probability... the reference's ``mean p²``), defaults 8 experts, top-2,
capacity factor 1.25, aux coefficients 0.01 / 0.001 (``config.rs``). Dispatch/combine (``manager.rs:101-323``) is an
all-to-all of tokens grouped by owning rank.  On GPUs (bf16, more than one rank) dispatch and combine are the
peer-memory kernels of ``csrc/kernels/moe_sm100.cu``: tokens are stored straight into the owning rank's
``[E_local][world][capacity][H]`` buffer and expert outputs are read back with peer loads weighted by the gate, with no
sort, no size exchange and no staging copy (:class:`FusedMoEDispatch`).  Otherwise it is
``torch.distributed.all_to_all_single`` (gloo: emulated), with a dense single-process path when no group is given.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from enum import Enum

import torch
import torch.distributed as dist

from ..nn.module import Module, Parameter


@dataclass
class ExpertParallelismConfig:
    num_experts: int = 8
    top_k: int = 2
    capacity_factor: float = 1.25
    load_balance_coeff: float = 0.01
    z_loss_coeff: float = 0.001
    drop_tokens: bool = True
    enable_load_balancing: bool = False
    rebalancing_threshold: float = 0.3      # (max - min) / mean of the smoothed expert loads that triggers a rebalance
    hierarchical_gate: bool = False         # two-stage gate: expert groups, then experts inside each group


# ------------------------------------------------------------------------------------------ load balancing
class RebalancingStrategy(Enum):
    """``crates/torsh-distributed/src/expert_parallelism/load_balancer.rs:20-75``."""
    ROUTING_ADJUSTMENT = "routing_adjustment"
    EXPERT_MIGRATION = "expert_migration"
    CAPACITY_REALLOCATION = "capacity_reallocation"
    HYBRID_APPROACH = "hybrid_approach"

    def disruption_level(self) -> float:
        return {"routing_adjustment": 0.1, "capacity_reallocation": 0.3, "expert_migration": 0.7, "hybrid_approach": 0.5}[self.value]

    def supports_rollback(self) -> bool:
        return self in (RebalancingStrategy.ROUTING_ADJUSTMENT, RebalancingStrategy.CAPACITY_REALLOCATION)


class MigrationType(Enum):
    LOAD_REDISTRIBUTION = "load_redistribution"
    DEVICE_MIGRATION = "device_migration"
    EXPERT_REPLICATION = "expert_replication"
    EXPERT_CONSOLIDATION = "expert_consolidation"

    def complexity(self) -> int:
        return {"load_redistribution": 1, "expert_replication": 2, "device_migration": 3, "expert_consolidation": 4}[self.value]

    def requires_parameter_copy(self) -> bool:
        return self in (MigrationType.DEVICE_MIGRATION, MigrationType.EXPERT_REPLICATION)


@dataclass
class ExpertMigration:
    source_expert_id: int
    target_expert_id: int
    migration_type: MigrationType
    priority: float
    estimated_duration_s: float
    expected_load_reduction: float = 0.3
    expected_load_increase: float = 0.8

    def is_high_priority(self) -> bool:
        return self.priority > 0.7

    def expected_improvement(self) -> float:
        return self.expected_load_reduction * self.priority


@dataclass
class LoadBalancingStats:
    expert_loads: list
    load_variance: float
    rebalancing_count: int
    pending_migrations: int
    routing_adjustments: list
    strategy_effectiveness: dict

    def load_cv(self) -> float:
        n = len(self.expert_loads)
        mean = sum(self.expert_loads) / n if n else 0.0
        return math.sqrt(self.load_variance) / mean if mean > 0 else 0.0

    def best_strategy(self):
        return max(self.strategy_effectiveness, key=self.strategy_effectiveness.get) if self.strategy_effectiveness else None

    def is_well_balanced(self) -> bool:
        return self.load_cv() < 0.2


class LoadBalancer:
    """Host-side controller that watches the routing decisions and steers them back to balance
    (``load_balancer.rs:174-720``): exponentially smoothed expert loads (alpha 0.1), a rebalance at most every ten
    updates when ``(max - min) / mean`` exceeds the threshold, and four strategies - bias the router (x1.2 for experts
    under 0.8 of the mean load, x0.8 above 1.2, decaying back to 1 by 0.95 per step), re-allocate per-expert capacity from
    the predicted load (load + 0.3 x trend over the last five updates), schedule expert migrations (experts above 1.3 x
    mean paired with experts below 0.7 x mean, at most two at a time, highest load difference first), or the first two
    together. The strategy is the historically most effective one (relative variance reduction, smoothed 0.9 / 0.1)
    when that exceeds 0.3, else chosen from the severity of the imbalance."""

    def __init__(self, cfg: ExpertParallelismConfig):
        E = cfg.num_experts
        self.expert_loads = [0.0] * E
        self.expert_capacities = [1.0] * E
        self.routing_adjustments = [1.0] * E
        self.routing_adjustment_decay = 1.0
        self.rebalancing_threshold = cfg.rebalancing_threshold
        self.last_rebalancing_step = 0
        self.rebalancing_count = 0
        self.load_history: deque = deque(maxlen=100)
        self.load_variance_history: deque = deque(maxlen=50)
        self.pending_migrations: deque = deque()
        self.completed_migrations: list[ExpertMigration] = []
        self.strategy_effectiveness: dict = {}
        self.last_strategy = None

    # ---- observations
    def update_expert_load(self, tokens_per_expert, total_tokens: int):
        if total_tokens == 0:
            return
        alpha = 0.1
        for e, c in enumerate(tokens_per_expert):
            if e < len(self.expert_loads):
                self.expert_loads[e] = alpha * (float(c) / total_tokens) + (1 - alpha) * self.expert_loads[e]
        self.load_history.append(list(self.expert_loads))
        self.load_variance_history.append(self.load_variance())
        if self.should_rebalance():
            self.trigger_rebalancing()
        self.last_rebalancing_step += 1

    def load_variance(self) -> float:
        n = len(self.expert_loads)
        if n == 0:
            return 0.0
        mean = sum(self.expert_loads) / n
        return sum((l - mean) ** 2 for l in self.expert_loads) / n

    def imbalance(self) -> float:
        mean = sum(self.expert_loads) / max(len(self.expert_loads), 1)
        return (max(self.expert_loads) - min(self.expert_loads)) / mean if mean > 0 else 0.0

    def should_rebalance(self) -> bool:
        if not self.expert_loads or self.last_rebalancing_step < 10:
            return False
        return self.imbalance() > self.rebalancing_threshold

    def load_trend(self, e: int) -> float:
        recent = [h[e] for h in list(self.load_history)[-5:]][::-1]
        n = len(recent)
        if n < 2:
            return 0.0
        sx, sy = sum(range(n)), sum(recent)
        sxy, sx2 = sum(i * y for i, y in enumerate(recent)), sum(i * i for i in range(n))
        den = n * sx2 - sx * sx
        return 0.0 if abs(den) < 1e-12 else (n * sxy - sx * sy) / den

    # ---- decisions
    def rebalancing_strategy(self) -> RebalancingStrategy:
        if self.strategy_effectiveness:
            best = max(self.strategy_effectiveness, key=self.strategy_effectiveness.get)
            if self.strategy_effectiveness[best] > 0.3:
                return best
        sev, var = self.imbalance(), self.load_variance()
        if sev > 0.5 and var > 0.1:
            return RebalancingStrategy.HYBRID_APPROACH
        if sev > 0.3:
            return RebalancingStrategy.EXPERT_MIGRATION
        if var > 0.05:
            return RebalancingStrategy.CAPACITY_REALLOCATION
        return RebalancingStrategy.ROUTING_ADJUSTMENT

    def trigger_rebalancing(self, strategy: RebalancingStrategy | None = None):
        strategy = strategy or self.rebalancing_strategy()
        start = self.load_variance()
        if strategy in (RebalancingStrategy.ROUTING_ADJUSTMENT, RebalancingStrategy.HYBRID_APPROACH):
            self.apply_routing_adjustment()
        if strategy in (RebalancingStrategy.CAPACITY_REALLOCATION, RebalancingStrategy.HYBRID_APPROACH):
            self.apply_capacity_reallocation()
        if strategy is RebalancingStrategy.EXPERT_MIGRATION:
            self.apply_expert_migration()
        end = self.load_variance()
        imp = (start - end) / max(start, 1e-12)
        self.strategy_effectiveness[strategy] = 0.9 * self.strategy_effectiveness[strategy] + 0.1 * imp if strategy in self.strategy_effectiveness else imp
        self.last_strategy = strategy
        self.rebalancing_count += 1
        self.last_rebalancing_step = 0

    def apply_routing_adjustment(self):
        mean = sum(self.expert_loads) / len(self.expert_loads)
        for e, load in enumerate(self.expert_loads):
            ratio = load / mean if mean > 0 else 1.0
            self.routing_adjustments[e] = 1.2 if ratio < 0.8 else (0.8 if ratio > 1.2 else 1.0)
        self.routing_adjustment_decay = 0.95

    def apply_capacity_reallocation(self):
        # The reference compares the predicted load FRACTION with a capacity (1.0 per expert), which can only ever shrink
        # capacities (load_balancer.rs:430-457); here the prediction is first put on the capacity scale (load relative
        # to the mean load), so hot experts really gain capacity and cold ones lose it.
        total = sum(self.expert_capacities)
        target = total / len(self.expert_loads)
        mean_load = sum(self.expert_loads) / len(self.expert_loads)
        for e, load in enumerate(self.expert_loads):
            pred = (load + 0.3 * self.load_trend(e)) / mean_load * target if mean_load > 0 else target
            if pred > target * 1.1:
                self.expert_capacities[e] = min(target * 1.25, total * 0.3)
            elif pred < target * 0.8:
                self.expert_capacities[e] = max(target * 0.75, target * 0.5)
            else:
                self.expert_capacities[e] = target

    def migration_candidates(self) -> tuple[list[int], list[int]]:
        mean = sum(self.expert_loads) / len(self.expert_loads)
        over = [e for e, l in enumerate(self.expert_loads) if l > mean * 1.3]
        under = [e for e, l in enumerate(self.expert_loads) if l < mean * 0.7]
        return over, under

    def apply_expert_migration(self):
        over, under = self.migration_candidates()
        if not over or not under:
            return
        plan = []
        for i in range(min(len(over), len(under), 2)):
            src, dst = over[i], under[i % len(under)]
            plan.append(ExpertMigration(src, dst, MigrationType.LOAD_REDISTRIBUTION,
                                        (self.expert_loads[src] - self.expert_loads[dst]) * 10.0,
                                        5.0 * (1.0 + self.expert_loads[src])))
        plan.sort(key=lambda m: -m.priority)
        self.pending_migrations.extend(plan)

    def process_pending_migrations(self) -> ExpertMigration | None:
        """Pops the next scheduled migration and updates the load estimates as the reference does; the caller moves
        the expert (``DistributedExpertManager.execute_migration``)."""
        if not self.pending_migrations:
            return None
        m = self.pending_migrations.popleft()
        self.expert_loads[m.source_expert_id] = max(self.expert_loads[m.source_expert_id] * (1 - m.expected_load_reduction), 0.0)
        self.expert_loads[m.target_expert_id] += m.expected_load_reduction * m.expected_load_increase
        self.completed_migrations.append(m)
        return m

    def get_routing_adjustment(self, e: int) -> float:
        return self.routing_adjustments[e] if 0 <= e < len(self.routing_adjustments) else 1.0

    def decay_routing_adjustments(self):
        d = self.routing_adjustment_decay
        self.routing_adjustments = [a * d + (1 - d) for a in self.routing_adjustments]

    def capacity_scale(self) -> list[float]:
        mean = sum(self.expert_capacities) / len(self.expert_capacities)
        return [c / mean for c in self.expert_capacities]

    def get_stats(self) -> LoadBalancingStats:
        return LoadBalancingStats(list(self.expert_loads), self.load_variance(), self.rebalancing_count, len(self.pending_migrations),
                                  list(self.routing_adjustments), dict(self.strategy_effectiveness))

    def reset(self):
        self.__init__(ExpertParallelismConfig(num_experts=len(self.expert_loads), rebalancing_threshold=self.rebalancing_threshold))


class GateNetwork(Module):
    """Hierarchical gate (``router.rs:497-640``): experts are arranged in ``ceil(sqrt(E))`` groups; a group router gives
    ``p(group | token)``, each group's own router ``p(expert | group, token)``, and the gate probability of an expert is
    their product. Returns ``[..., E]`` probabilities (each token's row sums to 1)."""

    def __init__(self, input_dim: int, num_experts: int):
        super().__init__()
        self.num_experts = num_experts
        self.num_groups = int(math.ceil(math.sqrt(num_experts)))
        self.experts_per_group = -(-num_experts // self.num_groups)
        self.group_router = Parameter(torch.empty(input_dim, self.num_groups).normal_(0, 0.02))
        self.expert_routers = Parameter(torch.empty(self.num_groups, input_dim, self.experts_per_group).normal_(0, 0.02))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape[:-1]
        xf = x.reshape(-1, x.shape[-1]).float()
        gp = torch.softmax(xf @ self.group_router.float(), -1)                                  # [T, G]
        el = torch.einsum("th,ghe->tge", xf, self.expert_routers.float())                       # [T, G, Eg]
        ids = torch.arange(self.num_groups * self.experts_per_group, device=x.device).view(self.num_groups, self.experts_per_group)
        el = el.masked_fill(ids.unsqueeze(0) >= self.num_experts, float("-inf"))                # slots past the last expert
        ep = torch.softmax(el, -1)
        probs = (gp.unsqueeze(-1) * ep).reshape(xf.shape[0], -1)[:, : self.num_experts]
        return probs.reshape(*shape, self.num_experts)

    def get_hierarchy_stats(self) -> dict:
        return {"num_groups": self.num_groups, "experts_per_group": self.experts_per_group, "total_experts": self.num_experts,
                "total_capacity": self.num_groups * self.experts_per_group}


class TopKRouter(Module):
    def __init__(self, hidden: int, cfg: ExpertParallelismConfig | None = None):
        super().__init__()
        self.cfg = cfg or ExpertParallelismConfig()
        if self.cfg.hierarchical_gate:
            self.gate_network = GateNetwork(hidden, self.cfg.num_experts)
            self.gate = None
        else:
            self.gate = Parameter(torch.empty(self.cfg.num_experts, hidden).normal_(0, 0.02))
        self.load_balancer = LoadBalancer(self.cfg) if self.cfg.enable_load_balancing else None

    def capacity(self, tokens: int) -> int:
        c = self.cfg
        return int(math.ceil(tokens * c.top_k / c.num_experts * c.capacity_factor))

    def forward(self, x: torch.Tensor):
        """``x``: ``[T, H]`` → ``(expert_idx [T,k], weights [T,k], keep [T,k], aux_loss)``."""
        c = self.cfg
        if self.gate is None:
            probs = self.gate_network(x)
        else:
            logits = torch.nn.functional.linear(x.float(), self.gate.float())
            probs = torch.softmax(logits, -1)
        lb = self.load_balancer
        sel = probs
        if lb is not None:
            # the balancer biases the SELECTION (which experts a token goes to); the combine weights stay the gate's own
            # probabilities, so the bias never changes what an expert's output is multiplied with
            sel = probs * torch.tensor(lb.routing_adjustments, dtype=probs.dtype, device=probs.device)
        _, idx = sel.topk(c.top_k, -1)
        w = probs.gather(-1, idx)
        w = w / w.sum(-1, keepdim=True)
        T = x.shape[0]
        cap = self.capacity(T)
        onehot = torch.nn.functional.one_hot(idx, c.num_experts)                       # [T,k,E]
        pos = (onehot.reshape(T * c.top_k, c.num_experts).cumsum(0) - 1).reshape(T, c.top_k, c.num_experts)
        slot = (pos * onehot).sum(-1)                                                  # arrival order within its expert
        if lb is not None:
            # per-expert capacities re-allocated by the balancer, never above the buffer capacity `cap`
            caps = torch.tensor([min(cap, max(1, int(cap * s))) for s in lb.capacity_scale()], device=idx.device)
            keep = slot < caps[idx] if c.drop_tokens else torch.ones_like(slot, dtype=torch.bool)
        else:
            keep = slot < cap if c.drop_tokens else torch.ones_like(slot, dtype=torch.bool)
        load = onehot.sum((0, 1)).float()
        if lb is not None and self.training:
            # every rank must take the same balancing decisions (migrations are collective): feed the balancer the
            # routing counts of the whole group
            glob, total = load.detach().clone(), T * c.top_k
            grp = getattr(self, "stats_group", None)
            if grp is not None and dist.is_initialized() and dist.get_world_size(grp) > 1:
                dist.all_reduce(glob, group=grp)
                total *= dist.get_world_size(grp)
            lb.update_expert_load(glob.tolist(), int(total))
            lb.decay_routing_adjustments()
        cv = load.std(unbiased=False) / load.mean().clamp(min=1e-9)
        aux = c.load_balance_coeff * cv * cv + c.z_loss_coeff * probs.pow(2).mean()
        return idx, w, keep, slot, aux


class FusedMoEDispatch:
    """Symmetric buffers + autograd functions of the peer-memory dispatch / combine."""

    def __init__(self, hidden: int, e_local: int, capacity: int, group=None):
        import ctypes

        from .symm import CommContext, SymmetricBuffer
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.H, self.e_local, self.C = hidden, e_local, capacity
        n = e_local * self.world * capacity * hidden
        self.ctx = CommContext(self.group)
        mk = lambda: SymmetricBuffer(n, torch.bfloat16, self.group)
        self.recv, self.out, self.d_out, self.d_recv = mk(), mk(), mk(), mk()
        self.counts = SymmetricBuffer(max(e_local * self.world, 8), torch.int32, self.group, zero=True)
        dev = self.recv.tensor.device
        self._count_ptrs = torch.tensor(self.counts.peer_ptrs, dtype=torch.int64, device=dev)
        self.shape = (e_local, self.world, capacity, hidden)
        self._ct = ctypes

    # -- raw launches ------------------------------------------------------------------------------------
    def barrier(self):
        from .. import _native as nv
        from ..ops._dispatch import I, P, call
        call("tb_comm_barrier", [P, I, I, P, P, P], self.ctx.flags.ptr_array, self.rank, self.world, self.ctx.epoch.data_ptr(),
             nv.status_word().data_ptr(), nv.stream_ptr())

    def scatter(self, src, dst_buf, idx, slot, keep, scale=None, counts=None):
        from .. import _native as nv
        from ..ops._dispatch import I, P, call
        T, K = idx.shape
        call("tb_moe_scatter", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P], src.data_ptr(), dst_buf.ptr_array,
             idx.data_ptr(), slot.data_ptr(), keep.data_ptr(), nv.ptr(scale), nv.ptr(counts),
             self._count_ptrs.data_ptr() if counts is not None else None, T, K, self.H, self.C, self.e_local, self.rank,
             self.world, nv.stream_ptr())

    def gather(self, src_buf, idx, slot, keep, w=None, want_y=True, dy=None):
        from .. import _native as nv
        from ..ops._dispatch import I, P, call
        T, K = idx.shape
        y = torch.empty(T, self.H, dtype=torch.bfloat16, device=idx.device) if want_y else None
        dot = torch.empty(T, K, dtype=torch.float32, device=idx.device) if dy is not None else None
        call("tb_moe_gather", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P], src_buf.ptr_array, idx.data_ptr(),
             slot.data_ptr(), keep.data_ptr(), nv.ptr(w), nv.ptr(y), nv.ptr(dy), nv.ptr(dot), T, K, self.H, self.C,
             self.e_local, self.rank, self.world, nv.stream_ptr())
        return y, dot

    def valid_mask(self) -> torch.Tensor:
        """``[E_local, world, C, 1]`` mask of the slots the peers filled in the last dispatch."""
        c = self.counts.tensor[: self.e_local * self.world].view(self.e_local, self.world, 1)
        return (torch.arange(self.C, device=c.device).view(1, 1, -1) < c).unsqueeze(-1)

    # -- autograd -----------------------------------------------------------------------------------------
    def dispatch(self, x, idx, slot, keep, counts):
        return _MoEDispatchFn.apply(x, self, idx, slot, keep, counts)

    def combine(self, expert_out, gate, idx, slot, keep):
        return _MoECombineFn.apply(expert_out, gate, self, idx, slot, keep)


class _MoEDispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, d: FusedMoEDispatch, idx, slot, keep, counts):
        d.barrier()                                    # everybody is done reading the buffers of the previous step
        d.scatter(x.contiguous(), d.recv, idx, slot, keep, counts=counts)
        d.barrier()                                    # all rows (and counts) have landed
        ctx.d, ctx.meta = d, (idx, slot, keep)
        return d.recv.tensor.view(d.shape) * d.valid_mask()

    @staticmethod
    def backward(ctx, g):
        d = ctx.d
        idx, slot, keep = ctx.meta
        d.d_recv.tensor.view(d.shape).copy_(g)
        d.barrier()
        dx, _ = d.gather(d.d_recv, idx, slot, keep)    # dx[t] = sum over the token's kept choices of the row gradients
        d.barrier()
        return dx, None, None, None, None, None


class _MoECombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, gate, d: FusedMoEDispatch, idx, slot, keep):
        d.out.tensor.view(d.shape).copy_(expert_out)
        d.barrier()
        y, _ = d.gather(d.out, idx, slot, keep, w=gate.float().contiguous())
        ctx.d, ctx.meta = d, (idx, slot, keep)
        ctx.save_for_backward(gate)
        return y

    @staticmethod
    def backward(ctx, dy):
        d = ctx.d
        idx, slot, keep = ctx.meta
        (gate,) = ctx.saved_tensors
        dy = dy.contiguous()
        g32 = gate.float().contiguous()
        _, dgate = d.gather(d.out, idx, slot, keep, want_y=False, dy=dy)       # <dy[t], expert row>, rows still in place
        d.scatter(dy, d.d_out, idx, slot, keep, scale=g32)                      # gate * dy[t] into the owners' buffers
        d.barrier()
        d_expert = d.d_out.tensor.view(d.shape) * d.valid_mask()
        return d_expert, (dgate * keep).to(gate.dtype), None, None, None, None


class MoELayer(Module):
    """Experts are ``[E_local, H, F]`` / ``[E_local, F, H]`` weight stacks; tokens travel to the rank that owns their
    expert (all-to-all), run through the expert MLP, and travel back."""

    def __init__(self, hidden: int, ffn: int, cfg: ExpertParallelismConfig | None = None, group=None):
        super().__init__()
        self.cfg = cfg or ExpertParallelismConfig()
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None or dist.is_initialized()) and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        assert self.cfg.num_experts % self.world == 0
        self.e_local = self.cfg.num_experts // self.world
        self.router = TopKRouter(hidden, self.cfg)
        self.router.stats_group = (group if group is not None else dist.group.WORLD) if self.world > 1 else None
        self.w1 = Parameter(torch.empty(self.e_local, hidden, ffn).normal_(0, 0.02))
        self.w2 = Parameter(torch.empty(self.e_local, ffn, hidden).normal_(0, 0.02))
        # placement[e] = physical slot of logical expert e (slot // e_local is the owning rank, slot % e_local the row of
        # the weight stacks); the identity until experts are migrated
        self.register_buffer("placement", torch.arange(self.cfg.num_experts), persistent=True)

    @torch.no_grad()
    def swap_experts(self, a: int, b: int, extra_stacks=()):
        """Exchanges the physical homes of logical experts ``a`` and ``b`` (an expert migration that moves a hot expert to
        the rank of a cold one and back-fills with the cold one): the two weight rows - and the matching rows of every
        ``[E_local, ...]`` tensor in ``extra_stacks``, e.g. optimizer moments - travel between the owning ranks, and
        the placement table is updated on every rank. Collective: every rank of the group must call it."""
        sa, sb = int(self.placement[a]), int(self.placement[b])
        ra, rb = sa // self.e_local, sb // self.e_local
        la, lb = sa % self.e_local, sb % self.e_local
        stacks = [self.w1.data, self.w2.data, *extra_stacks]
        if ra == rb:
            if self.rank == ra:
                for t in stacks:
                    tmp = t[la].clone(); t[la].copy_(t[lb]); t[lb].copy_(tmp)
        elif self.rank in (ra, rb):
            mine, peer = (la, rb) if self.rank == ra else (lb, ra)
            g = self.group if self.group is not None else dist.group.WORLD
            peer_global = dist.get_global_rank(g, peer)
            for t in stacks:
                send, recv = t[mine].contiguous(), torch.empty_like(t[mine])
                ops = [dist.P2POp(dist.isend, send, peer_global, group=g), dist.P2POp(dist.irecv, recv, peer_global, group=g)]
                for wk in dist.batch_isend_irecv(ops):
                    wk.wait()
                t[mine].copy_(recv)
        self.placement[a], self.placement[b] = sb, sa

    def execute_pending_migration(self, extra_stacks=()) -> ExpertMigration | None:
        """Carries out the next migration the router's load balancer scheduled (every rank holds the same balancer state,
        since the routing statistics it sees are summed over the group): the overloaded expert swaps homes with the
        underloaded one when they live on different ranks."""
        lb = self.router.load_balancer
        if lb is None:
            return None
        m = lb.process_pending_migrations()
        if m is not None:
            self.swap_experts(m.source_expert_id, m.target_expert_id, extra_stacks)
        return m

    def expert_sharding_map(self) -> dict[int, tuple[int, int]]:
        """logical expert -> (owning rank, local row) (``manager.rs:444-751``)."""
        return {e: (int(s) // self.e_local, int(s) % self.e_local) for e, s in enumerate(self.placement.tolist())}

    def _experts(self, xs: torch.Tensor, eid: torch.Tensor) -> torch.Tensor:
        out = torch.zeros_like(xs)
        for e in range(self.e_local):
            m = eid == e
            if m.any():
                out[m] = torch.nn.functional.gelu(xs[m] @ self.w1[e].to(xs.dtype)) @ self.w2[e].to(xs.dtype)
        return out

    def _forward_fused(self, x, idx, w, keep, slot, aux, shape):
        T = x.shape[0]
        cap = self.router.capacity(T)
        d = getattr(self, "_fused", None)
        if d is None or d.C != cap or d.H != x.shape[1]:
            d = self._fused = FusedMoEDispatch(x.shape[1], self.e_local, cap, self.group)
        counts = torch.bincount(idx[keep].reshape(-1), minlength=self.cfg.num_experts).to(torch.int32)
        keep8 = keep.to(torch.uint8).contiguous()
        xs = d.dispatch(x, idx.contiguous(), slot.contiguous(), keep8, counts)          # [E_local, world, C, H]
        h = xs.reshape(self.e_local, -1, x.shape[1])
        out = torch.bmm(torch.nn.functional.gelu(torch.bmm(h, self.w1.to(h.dtype))), self.w2.to(h.dtype))
        y = d.combine(out.view(d.shape), w.to(torch.float32), idx, slot, keep8)
        return y.view(shape), aux

    def forward(self, x: torch.Tensor):
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        idx, w, keep, _, aux = self.router(x)
        idx = self.placement[idx]          # logical expert -> physical slot (slot numbering drives ownership below)
        T, k = idx.shape
        tok = torch.arange(T, device=x.device).repeat_interleave(k)[keep.reshape(-1)]
        exp = idx.reshape(-1)[keep.reshape(-1)]
        wt = w.reshape(-1)[keep.reshape(-1)]
        if self.world > 1 and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and k <= 8:
            return self._forward_fused(x, idx, w, keep, _, aux, shape)
        if self.world == 1:
            y = self._experts(x[tok], exp)
        else:
            owner = exp // self.e_local
            order = torch.argsort(owner, stable=True)
            send = x[tok][order]
            send_e = (exp % self.e_local)[order]
            counts = torch.bincount(owner, minlength=self.world)
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)
            sc, rc = counts.tolist(), recv_counts.tolist()
            recv = x.new_empty(sum(rc), x.shape[1])
            recv_e = send_e.new_empty(sum(rc))
            dist.all_to_all_single(recv, send, rc, sc, group=self.group)
            dist.all_to_all_single(recv_e, send_e, rc, sc, group=self.group)
            out = self._experts(recv, recv_e)
            back = torch.empty_like(send)
            dist.all_to_all_single(back, out, sc, rc, group=self.group)
            y = torch.empty_like(back)
            y[order] = back
        res = torch.zeros_like(x)
        res.index_add_(0, tok, y * wt.unsqueeze(1).to(y.dtype))
        return res.view(shape), aux
