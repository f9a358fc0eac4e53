"""Collective micro-benchmark (role of ``examples/distributed_nccl.rs``: env ``WORLD_SIZE`` / ``RANK`` / ``BENCHMARK``,
times all-reduce and broadcast). With GPUs the fused NVSwitch kernels are compared with NCCL; on CPU it runs over gloo.

  BENCHMARK=1 python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
      --master-port 29563 examples/distributed_nccl.py"""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

from torsh_b200.parallel import collectives as C


def main(argv=None):
    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29563"), ("RANK", "0"), ("WORLD_SIZE", "1")):
        os.environ.setdefault(k, v)
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    rank, world = dist.get_rank(), dist.get_world_size()
    bench = os.environ.get("BENCHMARK", "0") == "1"
    sizes = [1 << 12, 1 << 16, 1 << 20] + ([1 << 24] if bench else [])
    rows = []
    for n in sizes:
        t = torch.full((n,), float(rank + 1), device=dev)
        C.all_reduce(t)
        assert float(t[0]) == world * (world + 1) / 2
        b = torch.full((n,), float(rank), device=dev)
        C.broadcast(b, src=0)
        assert float(b[-1]) == 0.0
        iters = 10 if bench else 2
        if cuda:
            torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(iters):
            C.all_reduce(t)
        if cuda:
            torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / iters
        rows.append((n * 4, dt * 1e6, 2 * (world - 1) / max(world, 1) * n * 4 / dt / 1e9))
    if cuda and world > 1:
        fc = C.FusedCollectives()
        from torsh_b200.parallel.symm import SymmetricBuffer
        buf = SymmetricBuffer(1 << 20, torch.float32)
        buf.tensor.fill_(rank + 1)
        fc.all_reduce_(buf, numel=1 << 20, scale=1.0)
        torch.cuda.synchronize()
        assert float(buf.tensor[0]) == world * (world + 1) / 2
    if rank == 0:
        for nbytes, us, bw in rows:
            print(f"all_reduce {nbytes:>10d} B: {us:9.1f} us, bus bandwidth {bw:7.2f} GB/s")
    dist.barrier()
    dist.destroy_process_group()
    return rows


if __name__ == "__main__":
    main()
