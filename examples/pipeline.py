"""Pipeline-parallel training with the 1F1B schedule (role of ``examples/distributed_pipeline.rs``).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29562 \
      examples/pipeline.py
Each rank owns one stage; activations and their gradients travel over ``torch.distributed`` point-to-point
(NCCL between GPUs, gloo on CPU)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

from torsh_b200.parallel.pipeline import PipelineConfig, PipelineParallel, ScheduleType, create_pipeline_stages


def main(argv=None):
    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29562"), ("RANK", "0"), ("WORLD_SIZE", "1")):
        os.environ.setdefault(k, v)
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    layers = [torch.nn.Sequential(torch.nn.Linear(32, 32), torch.nn.Tanh()) for _ in range(4 * world)]
    stage = create_pipeline_stages(layers, world)[rank].to(dev)
    pipe = PipelineParallel(stage, config=PipelineConfig(num_micro_batches=4, schedule=ScheduleType.ONE_F_ONE_B),
                            activation_shape=(8, 32), activation_dtype=torch.float32)
    opt = torch.optim.SGD(stage.parameters(), lr=0.05)
    x, y = torch.randn(32, 32, device=dev), torch.randn(32, 32, device=dev)
    losses = []
    for step in range(5):
        loss = pipe.train_step(x if pipe.is_first else None, y if pipe.is_last else None, torch.nn.functional.mse_loss)
        opt.step(); opt.zero_grad()
        if loss is not None:
            losses.append(loss.item())
            print(f"step {step}  loss {loss.item():.4f}  sends {pipe.stats['sends']} recvs {pipe.stats['recvs']}")
    dist.barrier()
    dist.destroy_process_group()
    return losses


if __name__ == "__main__":
    main()
