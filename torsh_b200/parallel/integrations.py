"""Import of third-party training configurations (``crates/torsh-distributed/src/{deepspeed,fairscale,horovod}_integration.rs``):
DeepSpeed JSON (ZeRO stage, offload, fp16 / bf16, gradient clipping, batch sizes), FairScale (OSS / ShardedDDP / FSDP /
Pipe) and Horovod (fusion threshold, cycle time, compression) settings are mapped onto this framework's own
``FsdpConfig`` / ``BucketConfig`` / ``PipelineConfig`` / optimizer options."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path


@dataclass
class TrainingPlan:
    strategy: str = "ddp"                  # ddp | fsdp | zero_offload | pipeline
    sharding: str = "no_shard"             # no_shard | shard_grad_op | full_shard
    cpu_offload: bool = False
    param_dtype: str = "fp32"
    loss_scale: float | None = None
    bucket_mb: float = 25.0
    grad_clip: float | None = None
    micro_batch: int | None = None
    grad_accum: int = 1
    optimizer: dict = field(default_factory=dict)
    pipeline_stages: int = 1
    micro_batches: int = 1
    compression: str | None = None
    notes: list = field(default_factory=list)

    def fsdp_config(self):
        from .fsdp import FsdpConfig, ShardingStrategy
        m = {"full_shard": ShardingStrategy.FULL_SHARD, "shard_grad_op": ShardingStrategy.SHARD_GRAD_OP, "no_shard": ShardingStrategy.NO_SHARD}
        return FsdpConfig(sharding_strategy=m[self.sharding], cpu_offload=self.cpu_offload)

    def bucket_config(self):
        from .ddp import BucketConfig
        return BucketConfig(max_bucket_size_mb=self.bucket_mb)


def _load(cfg):
    if isinstance(cfg, (str, Path)):
        return json.loads(Path(cfg).read_text())
    return dict(cfg)


def from_deepspeed(cfg) -> TrainingPlan:
    c = _load(cfg)
    z = c.get("zero_optimization", {})
    stage = int(z.get("stage", 0))
    plan = TrainingPlan()
    plan.sharding = {0: "no_shard", 1: "shard_grad_op", 2: "shard_grad_op", 3: "full_shard"}[stage]
    plan.strategy = "ddp" if stage == 0 else "fsdp"
    if stage == 1:
        plan.notes.append("ZeRO-1 (optimizer-state sharding only): DDP + optim.distributed.ZeroRedundancyOptimizer")
    off = (z.get("offload_optimizer", {}).get("device", "none") != "none") or (z.get("offload_param", {}).get("device", "none") != "none")
    plan.cpu_offload = off
    if off:
        plan.strategy = "zero_offload"
    if c.get("bf16", {}).get("enabled"):
        plan.param_dtype = "bf16"
    elif c.get("fp16", {}).get("enabled"):
        plan.param_dtype = "fp16"
        ls = c["fp16"].get("loss_scale", 0)
        plan.loss_scale = float(ls) if ls else 2.0 ** c["fp16"].get("initial_scale_power", 16)
    if "reduce_bucket_size" in z:
        plan.bucket_mb = float(z["reduce_bucket_size"]) * 4 / 2**20 if z["reduce_bucket_size"] < 1e9 else 25.0
    plan.grad_clip = c.get("gradient_clipping")
    plan.micro_batch = c.get("train_micro_batch_size_per_gpu")
    plan.grad_accum = int(c.get("gradient_accumulation_steps", 1))
    opt = c.get("optimizer", {})
    if opt:
        plan.optimizer = {"type": opt.get("type", "AdamW"), **opt.get("params", {})}
    return plan


def from_fairscale(cfg) -> TrainingPlan:
    c = _load(cfg)
    plan = TrainingPlan()
    kind = c.get("wrapper", "ddp").lower()
    if kind in ("oss", "sharded_ddp", "shardedddp"):
        plan.strategy, plan.sharding = "fsdp", "shard_grad_op"
    elif kind == "fsdp":
        plan.strategy = "fsdp"
        plan.sharding = "full_shard" if c.get("reshard_after_forward", True) else "shard_grad_op"
        plan.cpu_offload = bool(c.get("move_params_to_cpu") or c.get("cpu_offload"))
        if c.get("mixed_precision"):
            plan.param_dtype = "bf16" if c.get("compute_dtype", "bf16") in ("bf16", "bfloat16") else "fp16"
    elif kind == "pipe":
        plan.strategy = "pipeline"
        plan.pipeline_stages = len(c.get("balance", [1]))
        plan.micro_batches = int(c.get("chunks", 1))
    plan.bucket_mb = float(c.get("bucket_cap_mb", 25.0))
    return plan


def from_horovod(cfg) -> TrainingPlan:
    c = _load(cfg)
    plan = TrainingPlan(strategy="ddp")
    plan.bucket_mb = float(c.get("fusion_threshold_mb", c.get("HOROVOD_FUSION_THRESHOLD", 64 * 2**20) / 2**20 if "HOROVOD_FUSION_THRESHOLD" in c else 64.0))
    comp = str(c.get("compression", "none")).lower()
    plan.compression = None if comp == "none" else comp
    if comp == "fp16":
        plan.notes.append("fp16 gradient compression maps to bf16 bucket all-reduce with fp32 accumulation")
    plan.grad_accum = int(c.get("backward_passes_per_step", 1))
    return plan


def from_ray(cfg) -> TrainingPlan:
    """Ray Train ``ScalingConfig`` / ``TorchConfig`` (``crates/torsh-distributed/src/ray_integration.rs``): workers map to
    ranks, ``use_gpu`` and ``resources_per_worker`` to one process per GPU; elastic / fault-tolerance settings become notes
    for ``parallel.fault_tolerance``."""
    c = _load(cfg)
    sc = c.get("scaling_config", c)
    plan = TrainingPlan(strategy="ddp")
    workers = int(sc.get("num_workers", 1))
    plan.notes.append(f"world size {workers} (one process per GPU)")
    if not sc.get("use_gpu", True):
        plan.notes.append("CPU workers requested: gloo backend")
    tc = c.get("torch_config", {})
    if str(tc.get("backend", "nccl")).lower() != "nccl":
        plan.notes.append(f"backend {tc.get('backend')} requested; NCCL / fused NVSwitch kernels are used on GPUs")
    fc = c.get("failure_config", {})
    if fc.get("max_failures"):
        plan.notes.append(f"max_failures {fc['max_failures']}: use fault_tolerance.ElasticTrainingManager with checkpoint restarts")
    strat = str(c.get("strategy", "ddp")).lower()
    if strat in ("fsdp", "zero3", "deepspeed"):
        plan.strategy, plan.sharding = "fsdp", "full_shard"
    return plan


def from_dask(cfg) -> TrainingPlan:
    """Dask cluster description (``crates/torsh-distributed/src/dask_integration.rs``): ``n_workers`` ×
    ``threads_per_worker`` with a GPU per worker (dask-cuda); data-parallel with the batch split over workers."""
    c = _load(cfg)
    plan = TrainingPlan(strategy="ddp")
    plan.notes.append(f"world size {int(c.get('n_workers', 1))}")
    if int(c.get("threads_per_worker", 1)) > 1:
        plan.notes.append("threads_per_worker > 1: one training process per GPU is used; extra threads serve the data loader")
    if c.get("memory_limit"):
        plan.notes.append(f"host memory limit {c['memory_limit']} applies to the pinned staging pools")
    chunk = c.get("chunk_size")
    if chunk:
        plan.micro_batches = max(1, int(c.get("batch_size", chunk)) // int(chunk))
    return plan
