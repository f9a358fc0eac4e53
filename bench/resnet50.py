#!/usr/bin/env python
"""ResNet-50 data-parallel training throughput (images/s): bf16 activations, fp32 parameters, SGD momentum 0.9,
25 MB gradient buckets, batch 256 per GPU, 224x224x3 inputs with N(0,1) pixels, uniform labels over 1000 classes,
Kaiming-normal init, BatchNorm not synchronised.

  python bench/resnet50.py --steps 10 --warmup 3                       # this framework, one GPU
  python bench/resnet50.py --impl torch                                # stock PyTorch (cuDNN, autocast, torch SGD)
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
      bench/resnet50.py --gpus 2

``--impl ours`` runs the channels-last kernel path of ``torsh_b200.models.ResNet`` (tcgen05 GEMM convolutions, fused
BatchNorm/ReLU/residual), the fused multi-tensor SGD kernel and, for N > 1, ``parallel.DistributedDataParallel`` whose
bucket all-reduce + 1/world scale is one NVSwitch kernel launched from autograd hooks.  ``--impl torch`` is the
constructed baseline: the same architecture on PyTorch's layers in channels_last under bf16 autocast, torch SGD and
``torch.nn.parallel.DistributedDataParallel`` (NCCL).  One JSON line on rank 0; device-timed with CUDA events, max over
ranks; the end-to-end figure copies each batch from pinned host memory and reads the loss back every step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--image", type=int, default=224)
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    ap.add_argument("--model", default="resnet50")
    ap.add_argument("--no-graph", action="store_true", help="issue every launch of the step from Python instead of replaying one CUDA graph")
    ap.add_argument("--ddp-no-overlap", action="store_true", help="reduce all gradient buckets after backward instead of from hooks")
    ap.add_argument("--ddp-comm-blocks", type=int, default=64, help="CTAs of the fused bucket all-reduce kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.graph = not args.no_graph and args.impl == "ours"

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from bench import ClockSampler  # repo-root bench.py
    from torsh_b200 import _native as nv
    from torsh_b200.models import create_model

    torch.manual_seed(1234)
    model = create_model(args.model).to(dev)
    model.train()
    B = args.batch
    if args.impl == "ours":
        from torsh_b200.optim.fused import SGD
        model.use_kernels = True
        net = model
        if world > 1:
            from torsh_b200.parallel.ddp import DistributedDataParallel, OverlapConfig
            net = DistributedDataParallel(model, bucket_cap_mb=25.0, comm_blocks=args.ddp_comm_blocks,
                                          overlap_config=OverlapConfig(enabled=not args.ddp_no_overlap))
        # under a graph the gradients must keep their addresses: the SGD kernel clears them in the pass that reads them
        opt = SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4, zero_grad_in_step=args.graph and world == 1)

        def step(x, y):
            logits = net(x)
            loss = torch.nn.functional.cross_entropy(logits, y)
            loss.backward()
            if world > 1:
                net.sync_gradients()
            opt.step()
            if world > 1:
                net.zero_grad()
            elif not args.graph:
                opt.zero_grad(set_to_none=True)
            return loss
    else:
        model.use_kernels = False
        model = model.to(memory_format=torch.channels_last)
        net = model
        if world > 1:
            net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], bucket_cap_mb=25, gradient_as_bucket_view=True)
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)

        def step(x, y):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                logits = net(x.contiguous(memory_format=torch.channels_last))
            loss = torch.nn.functional.cross_entropy(logits.float(), y)
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            return loss

    g = torch.Generator().manual_seed(1000 + rank)
    nb = 4
    x_host = torch.randn(nb, B, 3, args.image, args.image, generator=g).to(torch.bfloat16).pin_memory()
    y_host = torch.randint(0, 1000, (nb, B), generator=g).pin_memory()
    x_dev, y_dev = x_host[0].to(dev), y_host[0].to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    graphed = None
    launches0 = nv.launch_count
    if args.impl == "ours" and args.graph:
        # the whole step (forward, backward with its hook-launched bucket all-reduces, SGD) as one CUDA graph
        from torsh_b200.engine import GraphedStep
        eager_step = step
        graphed = GraphedStep(eager_step, [torch.empty_like(x_dev), torch.empty_like(y_dev)], warmup=2)
        step = lambda x, y: graphed(x, y)
        args.warmup = max(args.warmup, 4)
    for i in range(args.warmup):
        loss = step(x_dev, y_dev)
    first = loss.item()
    per_step_launches = graphed.launches_per_step if graphed is not None else (nv.launch_count - launches0) // args.warmup
    if args.impl == "ours":
        nv.check_status()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step(x_dev, y_dev)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    # Python time to queue ONE step on an idle device (with steps queued back to back the launch queue fills up and
    # the host is held to the device's pace, whatever it could do alone)
    t_issue = time.perf_counter()
    loss = step(x_dev, y_dev)
    host_issue_ms = (time.perf_counter() - t_issue) * 1e3
    barrier()
    # end to end: batch i + 1 is copied from pinned memory on a side stream while step i runs; the loss of step i is
    # copied to pinned memory behind the step and read after step i + 1 has been launched (every loss is read)
    copy_stream = torch.cuda.Stream()
    main = torch.cuda.current_stream()
    xbuf = [torch.empty_like(x_dev) for _ in range(2)]
    ybuf = [torch.empty_like(y_dev) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    loss_host = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_done = [torch.cuda.Event() for _ in range(2)]

    def stage(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])
            xbuf[i % 2].copy_(x_host[i % nb], non_blocking=True)
            ybuf[i % 2].copy_(y_host[i % nb], non_blocking=True)
            ready[i % 2].record()

    for ev in consumed:
        ev.record()
    t0 = time.perf_counter()
    stage(0)
    last = None
    for i in range(args.steps):
        if i + 1 < args.steps:
            stage(i + 1)
        main.wait_event(ready[i % 2])
        loss = step(xbuf[i % 2], ybuf[i % 2])
        consumed[i % 2].record()
        loss_host[i % 2].copy_(loss.detach().float(), non_blocking=True)
        loss_done[i % 2].record()
        if i > 0:
            loss_done[(i - 1) % 2].synchronize()
            last = float(loss_host[(i - 1) % 2])
    loss_done[(args.steps - 1) % 2].synchronize()
    last = float(loss_host[(args.steps - 1) % 2])
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    if args.impl == "ours":
        nv.check_status()
    t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    images = world * B * args.steps
    if rank == 0:
        print(json.dumps({
            "metric": "images/sec (ResNet-50 training step, device-timed, max over ranks)", "impl": args.impl,
            "value": images / (dev_ms / 1e3), "unit": "images/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "dtype": "bf16", "data": "synthetic (N(0,1) pixels, uniform labels, Kaiming-normal init)",
            "config": {"model": args.model, "global_batch": world * B, "batch_per_gpu": B, "image": args.image,
                       "optimizer": "SGD momentum 0.9, wd 1e-4", "bucket_mb": 25, "parallelism": f"ddp{world}" if world > 1 else "single",
                       "l2": "activations per step (>10 GB) far exceed the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": images / (e2e_ms / 1e3), "unit": "images/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": x_host[0].numel() * 2 + y_host[0].numel() * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": per_step_launches * args.steps, "launches_per_step": per_step_launches,
            "cuda_graph": bool(graphed is not None and graphed.graph is not None),
            "cuda_graph_error": graphed.error if graphed is not None else None,
            "host_issue_ms_per_step": host_issue_ms,
            "loss_first": first, "loss_last": last}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
