"""Distributed training: process groups, stores, collectives (NCCL / gloo and hand-written NVSwitch kernels),
DDP, FSDP, tensor + sequence parallelism, pipeline parallelism, 3-D mesh, expert parallelism, ZeRO offload,
gradient compression, fault tolerance. Mirrors the re-export list of ``crates/torsh-distributed/src/lib.rs:355-537``."""
from . import collectives, compression, planner
from .collectives import (ReduceOp, all_gather, all_gather_into_tensor, all_reduce, all_to_all, barrier, broadcast,
                          bucket_all_reduce, fused_all_reduce, gather, irecv, isend, recv, reduce, reduce_scatter,
                          ring_all_reduce_host, scatter, send, CollectiveBatch, CommunicationGroup, GroupManager, NcclBatch,
                          double_buffered_all_reduce, hierarchical_all_reduce, pipelined_all_reduce, ring_all_reduce,
                          tree_broadcast)
from .connection import ConnectionPool, RetryPolicy, retry
from .context_parallel import ContextParallelAttention, ring_attention, ulysses_attention
from .ddp import DDP, BucketConfig, DistributedDataParallel, OverlapConfig
from .expert_parallel import ExpertParallelismConfig, MoELayer, TopKRouter
from .fault_tolerance import (CircuitBreaker, CircuitState, ElasticConfig, ElasticTrainingManager, FailureDetector,
                              FaultInjector, FaultKind, HealthChecker, HeartbeatPublisher, RetryConfig, RetryExecutor)
from .fsdp import (BackwardPrefetch, FlatFSDP, FsdpConfig, MixedPrecisionConfig, ShardingStrategy, fsdp_wrap, shard_range)
from .mesh import DeviceMesh3D, RankMapping, ThreeDParallelismConfig
from .pipeline import PipelineConfig, PipelineParallel, ScheduleType, create_pipeline_stages
from .process_group import (BackendConfig, BackendType, ProcessGroup, destroy_process_group, get_rank, get_world_size,
                            init_process_group, is_available, is_initialized)
from .store import FileStore, MemoryStore, RedisStore, Store, TCPStore, create_store
from .tensor_parallel import (ColumnParallelLinear, ParallelAttention, ParallelEmbedding, RowParallelLinear, TensorParallelConfig, TPContext,
                              gather_tensor_from_tp, split_tensor_for_tp, vocab_parallel_cross_entropy)
from .zero_offload import OffloadedAdamW, Zero3OffloadConfig
