"""``rstorch.distributed``: ProcessGroup, DistributedDataParallel (DDP), init/destroy_process_group, get_rank,
get_world_size, is_initialized, is_available, barrier, all_reduce, all_gather, broadcast, reduce, scatter, gather."""
from torsh_b200.parallel import (DDP, DistributedDataParallel, ProcessGroup, ReduceOp, all_gather, all_reduce, barrier,  # noqa: F401
                                 broadcast, destroy_process_group, gather, get_rank, get_world_size, init_process_group,
                                 is_available, is_initialized, reduce, scatter)
