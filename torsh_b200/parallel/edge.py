"""Edge / federated training coordination (``crates/torsh-distributed/src/edge_computing.rs:24-1230``): a device registry
with client selection, bandwidth-adaptive communication parameters, federated aggregation (FedAvg / FedProx / weighted /
median / trimmed mean), differential privacy (clip + Gaussian noise) and tier assignment for hierarchical training.
This is host-side coordination logic; the tensors it aggregates can live on any device."""
from __future__ import annotations

import enum
import math
import random
import time
from collections import defaultdict, deque
from dataclasses import dataclass, field

import torch


class DeviceType(enum.Enum):
    SMARTPHONE = "smartphone"; TABLET = "tablet"; LAPTOP = "laptop"; IOT = "iot"; EDGE_SERVER = "edge_server"; DATACENTER = "datacenter"


class DeviceStatus(enum.Enum):
    AVAILABLE = "available"; TRAINING = "training"; OFFLINE = "offline"; LOW_BATTERY = "low_battery"; THROTTLED = "throttled"


class ClientSelectionStrategy(enum.Enum):
    RANDOM = "random"; RESOURCE_AWARE = "resource_aware"; DATA_SIZE = "data_size"; ROUND_ROBIN = "round_robin"


class FederatedAlgorithm(enum.Enum):
    FED_AVG = "fedavg"; FED_PROX = "fedprox"; FED_NOVA = "fednova"


class AggregationStrategy(enum.Enum):
    WEIGHTED_AVERAGE = "weighted_average"; SIMPLE_AVERAGE = "simple_average"; MEDIAN = "median"; TRIMMED_MEAN = "trimmed_mean"


class TrainingTier(enum.Enum):
    DEVICE = "device"; EDGE = "edge"; CLOUD = "cloud"


@dataclass
class EdgeDevice:
    device_id: str
    device_type: DeviceType = DeviceType.SMARTPHONE
    flops: float = 1e11
    memory_gb: float = 4.0
    bandwidth_mbps: float = 20.0
    battery: float = 1.0
    num_samples: int = 0
    status: DeviceStatus = DeviceStatus.AVAILABLE
    last_seen: float = field(default_factory=time.time)


@dataclass
class FederatedLearningConfig:
    algorithm: FederatedAlgorithm = FederatedAlgorithm.FED_AVG
    clients_per_round: int = 10
    local_epochs: int = 1
    selection: ClientSelectionStrategy = ClientSelectionStrategy.RANDOM
    aggregation: AggregationStrategy = AggregationStrategy.WEIGHTED_AVERAGE
    prox_mu: float = 0.01
    trim_fraction: float = 0.1
    min_battery: float = 0.2


@dataclass
class PrivacyConfig:
    clip_norm: float = 1.0
    noise_multiplier: float = 0.0
    seed: int | None = None


@dataclass
class AdaptiveCommunicationParams:
    compression_ratio: float
    quantization_bits: int
    sync_every: int


class BandwidthMonitor:
    def __init__(self, history: int = 256):
        self._h: dict[str, deque] = defaultdict(lambda: deque(maxlen=history))

    def record_measurement(self, device_id: str, mbps: float, when: float | None = None):
        self._h[device_id].append((when if when is not None else time.time(), mbps))

    def get_average_bandwidth(self, device_id: str, window_minutes: float = 5.0, now: float | None = None) -> float | None:
        now = now if now is not None else time.time()
        xs = [b for t, b in self._h.get(device_id, ()) if now - t <= window_minutes * 60]
        return sum(xs) / len(xs) if xs else None


def adaptive_params(bandwidth_mbps: float) -> AdaptiveCommunicationParams:
    """Slower links get sparser, coarser and rarer updates (``CommunicationManager::get_adaptive_params``)."""
    if bandwidth_mbps >= 100:
        return AdaptiveCommunicationParams(1.0, 16, 1)
    if bandwidth_mbps >= 20:
        return AdaptiveCommunicationParams(0.25, 8, 1)
    if bandwidth_mbps >= 5:
        return AdaptiveCommunicationParams(0.05, 8, 2)
    return AdaptiveCommunicationParams(0.01, 4, 4)


class EdgeComputingManager:
    """Device registry + client selection (``EdgeComputingManager::{register_device, select_clients, update_device_status}``)."""

    def __init__(self, config: FederatedLearningConfig | None = None, seed: int = 0, stale_after_s: float = 300.0):
        self.cfg = config or FederatedLearningConfig()
        self.devices: dict[str, EdgeDevice] = {}
        self.rng = random.Random(seed)
        self.stale_after_s = stale_after_s
        self._rr = 0

    def register_device(self, d: EdgeDevice):
        self.devices[d.device_id] = d

    def get_device(self, device_id: str) -> EdgeDevice | None:
        return self.devices.get(device_id)

    def update_device_status(self, device_id: str, status: DeviceStatus):
        d = self.devices[device_id]
        d.status, d.last_seen = status, time.time()

    def eligible(self, now: float | None = None) -> list[EdgeDevice]:
        now = now if now is not None else time.time()
        return [d for d in self.devices.values() if d.status is DeviceStatus.AVAILABLE and d.battery >= self.cfg.min_battery
                and now - d.last_seen <= self.stale_after_s]

    def select_clients(self, round_index: int) -> list[str]:
        pool = sorted(self.eligible(), key=lambda d: d.device_id)
        k = min(self.cfg.clients_per_round, len(pool))
        s = self.cfg.selection
        if s is ClientSelectionStrategy.RANDOM:
            chosen = self.rng.sample(pool, k)
        elif s is ClientSelectionStrategy.RESOURCE_AWARE:
            chosen = sorted(pool, key=lambda d: -(d.flops * min(d.bandwidth_mbps, 100.0) * d.battery))[:k]
        elif s is ClientSelectionStrategy.DATA_SIZE:
            chosen = sorted(pool, key=lambda d: -d.num_samples)[:k]
        else:
            start = (round_index * k) % max(len(pool), 1)
            chosen = [pool[(start + i) % len(pool)] for i in range(k)]
        return [d.device_id for d in chosen]


class PrivacyManager:
    """Per-client clipping to ``clip_norm`` and Gaussian noise of ``noise_multiplier · clip_norm`` on the aggregate
    (``PrivacyManager::apply_differential_privacy``)."""

    def __init__(self, cfg: PrivacyConfig | None = None):
        self.cfg = cfg or PrivacyConfig()
        self.gen = torch.Generator().manual_seed(self.cfg.seed) if self.cfg.seed is not None else None

    def clip(self, update: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        norm = math.sqrt(sum(float(v.float().pow(2).sum()) for v in update.values()))
        scale = min(1.0, self.cfg.clip_norm / max(norm, 1e-12))
        return {k: v * scale for k, v in update.items()}

    def add_noise(self, agg: dict[str, torch.Tensor], num_clients: int) -> dict[str, torch.Tensor]:
        if self.cfg.noise_multiplier <= 0:
            return agg
        std = self.cfg.noise_multiplier * self.cfg.clip_norm / max(num_clients, 1)
        return {k: v + (torch.randn(v.shape, generator=self.gen) * std).to(v.device, v.dtype) for k, v in agg.items()}


class FederatedLearningCoordinator:
    """``aggregate_updates``: combines client updates (deltas or full states) into the new global state."""

    def __init__(self, cfg: FederatedLearningConfig | None = None, privacy: PrivacyManager | None = None):
        self.cfg, self.privacy, self.round = cfg or FederatedLearningConfig(), privacy, 0

    def aggregate_updates(self, updates: list[dict[str, torch.Tensor]], num_samples: list[int] | None = None,
                          local_steps: list[int] | None = None) -> dict[str, torch.Tensor]:
        if not updates:
            raise ValueError("no client updates to aggregate")
        if self.privacy is not None:
            updates = [self.privacy.clip(u) for u in updates]
        n = len(updates)
        strat = self.cfg.aggregation
        w = [1.0 / n] * n
        if strat is AggregationStrategy.WEIGHTED_AVERAGE and num_samples:
            tot = float(sum(num_samples))
            w = [s / tot for s in num_samples]
        if self.cfg.algorithm is FederatedAlgorithm.FED_NOVA and local_steps:
            # normalise every client's update by its number of local steps, then rescale by the weighted mean step count
            tau = sum(wi * t for wi, t in zip(w, local_steps))
            updates = [{k: v * (tau / t) for k, v in u.items()} for u, t in zip(updates, local_steps)]
        out = {}
        for k in updates[0]:
            stack = torch.stack([u[k].float() for u in updates])
            if strat is AggregationStrategy.MEDIAN:
                agg = stack.median(0).values
            elif strat is AggregationStrategy.TRIMMED_MEAN:
                t = int(n * self.cfg.trim_fraction)
                srt = stack.sort(0).values
                agg = srt[t:n - t].mean(0) if n - 2 * t > 0 else srt.mean(0)
            else:
                agg = (stack * torch.tensor(w, dtype=stack.dtype).view(-1, *[1] * (stack.dim() - 1))).sum(0)
            out[k] = agg.to(updates[0][k].dtype)
        if self.privacy is not None:
            out = self.privacy.add_noise(out, n)
        self.round += 1
        return out

    def proximal_term(self, local: dict[str, torch.Tensor], global_state: dict[str, torch.Tensor]) -> torch.Tensor:
        """FedProx: ``mu/2 · ‖w - w_global‖²`` to add to a client's loss."""
        return 0.5 * self.cfg.prox_mu * sum(((local[k] - global_state[k].detach()) ** 2).sum() for k in local)


class HierarchicalTrainingCoordinator:
    """Assigns devices to tiers by capability (``assign_device_tier``): phones and IoT train on-device models, edge
    servers aggregate their neighbourhood, datacentre nodes aggregate the edge tier."""

    def __init__(self):
        self.tiers: dict[TrainingTier, list[str]] = {t: [] for t in TrainingTier}

    def assign_device_tier(self, d: EdgeDevice) -> TrainingTier:
        if d.device_type is DeviceType.DATACENTER or d.flops >= 1e14:
            tier = TrainingTier.CLOUD
        elif d.device_type is DeviceType.EDGE_SERVER or (d.flops >= 5e12 and d.memory_gb >= 16):
            tier = TrainingTier.EDGE
        else:
            tier = TrainingTier.DEVICE
        for ids in self.tiers.values():
            if d.device_id in ids:
                ids.remove(d.device_id)
        self.tiers[tier].append(d.device_id)
        return tier

    def get_tier_devices(self, tier: TrainingTier) -> list[str]:
        return list(self.tiers[tier])
