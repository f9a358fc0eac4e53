"""3-D (data × tensor × pipeline) process mesh.

``ThreeDParallelismConfig`` validates ``dp·tp·pp == world`` and ``layers % pp == 0``
(``crates/torsh-distributed/src/three_d_parallelism/config.rs:11-92``). ``RankMapping`` reproduces the
reference rule ``rank = dp·(tp·pp) + tp·pp_size + pp`` with pp fastest (``:195-225``) and offers ``tp_fastest``
so that on one NVSwitch box the TP peers are adjacent ranks; group rank lists and next/prev pipeline ranks follow
``:248-294``. ``DeviceMesh3D`` creates the ``torch.distributed`` sub-groups.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch.distributed as dist

from ..core.error import TorshDistributedError
from . import planner


@dataclass
class ThreeDParallelismConfig:
    dp_size: int = 1
    tp_size: int = 1
    pp_size: int = 1
    num_layers: int = 1
    micro_batch_size: int = 1
    num_micro_batches: int = 1
    sequence_parallel: bool = True
    tp_fastest: bool = True
    schedule: str = "1f1b"

    def validate(self, world_size: int):
        if self.dp_size * self.tp_size * self.pp_size != world_size:
            raise TorshDistributedError.configuration_error(
                f"dp({self.dp_size}) x tp({self.tp_size}) x pp({self.pp_size}) != world size {world_size}")
        if self.num_layers % self.pp_size != 0:
            raise TorshDistributedError.configuration_error(
                f"{self.num_layers} layers are not divisible by {self.pp_size} pipeline stages")
        return self

    @property
    def layers_per_stage(self) -> int:
        return self.num_layers // self.pp_size


class RankMapping:
    def __init__(self, cfg: ThreeDParallelismConfig, rank: int):
        self.cfg, self.rank = cfg, rank
        self.dp_rank, self.tp_rank, self.pp_rank = planner.coords_of(rank, cfg.dp_size, cfg.tp_size, cfg.pp_size, cfg.tp_fastest)

    def _r(self, dp, tp, pp):
        c = self.cfg
        return planner.rank_of(dp, tp, pp, c.dp_size, c.tp_size, c.pp_size, c.tp_fastest)

    def tp_group_ranks(self) -> list[int]:
        return [self._r(self.dp_rank, t, self.pp_rank) for t in range(self.cfg.tp_size)]

    def pp_group_ranks(self) -> list[int]:
        return [self._r(self.dp_rank, self.tp_rank, p) for p in range(self.cfg.pp_size)]

    def dp_group_ranks(self) -> list[int]:
        return [self._r(d, self.tp_rank, self.pp_rank) for d in range(self.cfg.dp_size)]

    def next_pp_rank(self) -> int | None:
        return None if self.pp_rank + 1 >= self.cfg.pp_size else self._r(self.dp_rank, self.tp_rank, self.pp_rank + 1)

    def prev_pp_rank(self) -> int | None:
        return None if self.pp_rank == 0 else self._r(self.dp_rank, self.tp_rank, self.pp_rank - 1)

    def layer_range(self) -> range:
        n = self.cfg.layers_per_stage
        return range(self.pp_rank * n, (self.pp_rank + 1) * n)


class DeviceMesh3D:
    """Creates every TP / PP / DP sub-group (all ranks must construct it) and keeps this rank's three."""

    def __init__(self, cfg: ThreeDParallelismConfig):
        world, rank = dist.get_world_size(), dist.get_rank()
        cfg.validate(world)
        self.cfg, self.mapping = cfg, RankMapping(cfg, rank)
        self.tp_group = self.pp_group = self.dp_group = None
        seen = {"tp": set(), "pp": set(), "dp": set()}
        for r in range(world):
            m = RankMapping(cfg, r)
            for kind, ranks in (("tp", m.tp_group_ranks()), ("pp", m.pp_group_ranks()), ("dp", m.dp_group_ranks())):
                key = tuple(ranks)
                if key in seen[kind]:
                    continue
                seen[kind].add(key)
                g = dist.new_group(list(ranks))
                if rank in ranks:
                    setattr(self, f"{kind}_group", g)

    @property
    def is_first_stage(self):
        return self.mapping.pp_rank == 0

    @property
    def is_last_stage(self):
        return self.mapping.pp_rank == self.cfg.pp_size - 1
