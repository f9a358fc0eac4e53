#!/usr/bin/env python
"""Collective sweep: in-kernel all-reduce / all-gather / reduce-scatter over NVSwitch peer memory (NVLS multimem when
available) against NCCL, bf16, 1 KB - 1 GB, device-timed with CUDA events, max over ranks.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29551 \
      bench/collectives.py [--max-mb 1024] [--json out.json]

Bus bandwidth follows the usual convention: all-reduce 2(n-1)/n x bytes / time, all-gather and reduce-scatter
(n-1)/n x total bytes / time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json")
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from torsh_b200 import _native as nv
    from torsh_b200.parallel.collectives import FusedCollectives
    from torsh_b200.parallel.symm import SymmetricBuffer
    rank, world = dist.get_rank(), dist.get_world_size()
    fc = FusedCollectives()
    sizes = [1 << k for k in range(10, 31, 2) if (1 << k) <= args.max_mb << 20]
    buf = SymmetricBuffer(max(sizes) // 2, torch.bfloat16)
    x = torch.randn(max(sizes) // 2, device=dev, dtype=torch.bfloat16)
    y = torch.empty_like(x)

    def timeit(fn):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier(); torch.cuda.synchronize()
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() * 1e3  # us

    rows = []
    for nbytes in sizes:
        n = nbytes // 2
        chunk = max(8, n // world // 8 * 8)
        cases = {
            "all_reduce": (lambda: fc.all_reduce_(buf, numel=n), lambda: dist.all_reduce(x[:n]), 2 * (world - 1) / world * nbytes),
            "all_gather": (lambda: fc.all_gather_(buf, chunk), lambda: dist.all_gather_into_tensor(y[:chunk * world], x[:chunk]),
                           (world - 1) / world * chunk * world * 2),
            "reduce_scatter": (lambda: fc.reduce_scatter(buf, chunk, out=y[:chunk]),
                               lambda: dist.reduce_scatter_tensor(y[:chunk], x[:chunk * world]), (world - 1) / world * chunk * world * 2),
        }
        for name, (fused, nccl, bus_bytes) in cases.items():
            tf, tn = timeit(fused), timeit(nccl)
            rows.append({"op": name, "bytes": nbytes, "fused_us": round(tf, 1), "nccl_us": round(tn, 1),
                         "fused_busbw_gbs": round(bus_bytes / tf / 1e3, 1), "nccl_busbw_gbs": round(bus_bytes / tn / 1e3, 1)})
            if rank == 0:
                r = rows[-1]
                print(f"{name:15s} {nbytes:>11d} B  fused {r['fused_us']:9.1f} us ({r['fused_busbw_gbs']:6.1f} GB/s)   "
                      f"nccl {r['nccl_us']:9.1f} us ({r['nccl_busbw_gbs']:6.1f} GB/s)   {tn / tf:.2f}x", flush=True)
        nv.check_status()
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump({"world": world, "nvls": buf.has_multicast, "rows": rows}, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
