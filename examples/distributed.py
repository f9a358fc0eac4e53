"""Data-parallel and fully-sharded training on one node (roles of ``examples/distributed.rs``,
``distributed_fsdp.rs``, ``distributed_gradient_sync.rs``).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29561 \
      examples/distributed.py --mode ddp          # or --mode fsdp (GPUs only)
With GPUs the backend is NCCL and gradients go through the fused bucket all-reduce kernel; without, gloo."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

import torsh_b200 as tb


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="ddp", choices=["ddp", "fsdp"])
    ap.add_argument("--steps", type=int, default=5)
    a = ap.parse_args(argv)
    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29561")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    losses = []
    if a.mode == "ddp":
        model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.Linear(256, 10)).to(dev)
        ddp = tb.parallel.DistributedDataParallel(model, bucket_cap_mb=1.0)
        opt = torch.optim.SGD(model.parameters(), lr=0.1)
        for s in range(a.steps):
            g = torch.Generator().manual_seed(100 * s + rank)
            x, y = torch.randn(32, 64, generator=g).to(dev), torch.randint(0, 10, (32,), generator=g).to(dev)
            loss = torch.nn.functional.cross_entropy(ddp(x), y)
            loss.backward()
            ddp.sync_gradients()
            opt.step()
            ddp.zero_grad()
            losses.append(loss.item())
        if rank == 0:
            print("ddp", ddp.get_sync_stats(), "losses", [round(v, 3) for v in losses])
    else:
        assert cuda, "the fused FSDP step needs GPUs"
        from torsh_b200.parallel.fsdp import FlatFSDP
        model = tb.models.create_model("gpt2-tiny").to(dev)
        trainer = tb.engine.CausalLMTrainer(model, lr=3e-4, batch_size=4, seq_len=64,
                                            parallel=FlatFSDP(dist.group.WORLD) if world > 1 else None)
        for s in range(a.steps):
            g = torch.Generator().manual_seed(100 * s + rank)
            ids = torch.randint(0, model.config.vocab_size, (4, 65), generator=g)
            losses.append(trainer.step(ids[:, :-1].contiguous(), ids[:, 1:].contiguous()))
        if rank == 0:
            print("fsdp losses", [round(v, 3) for v in losses])
    dist.barrier()
    dist.destroy_process_group()
    return losses


if __name__ == "__main__":
    main()
