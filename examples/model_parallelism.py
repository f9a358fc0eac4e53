"""Tensor, sequence and context parallelism on one node (roles of ``examples/advanced_model_parallelism.rs`` and
``advanced_multi_gpu_training.rs``): a Llama-style block stack whose projections are column / row parallel with the
activations sharded along tokens between them, a vocabulary-parallel head, and attention over a sequence that is
sharded across ranks (Ulysses all-to-all and ring attention).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29564 \
      examples/model_parallelism.py
With GPUs (NCCL) the parallel linears run the fused all-gather→GEMM and GEMM→reduce-scatter kernels; on CPU, gloo."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist

from torsh_b200.models.llama import LlamaConfig, LlamaModel
from torsh_b200.parallel.context_parallel import ring_attention, ulysses_attention
from torsh_b200.parallel.tensor_parallel import TensorParallelConfig, TPContext


def main(argv=None):
    cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29564"), ("RANK", "0"), ("WORLD_SIZE", "1")):
        os.environ.setdefault(k, v)
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    rank, world = dist.get_rank(), dist.get_world_size()

    # ---- tensor + sequence parallel language model with a vocabulary-parallel head
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_layers=2, num_heads=4, max_seq_len=64)
    tp = TPContext(dist.group.WORLD, TensorParallelConfig(tp_size=world, fused=cuda)) if world > 1 else None
    torch.manual_seed(1234 + rank)
    with torch.device(dev):
        model = LlamaModel(cfg, tp=tp, vocab_parallel=True)
    if cuda:
        model = model.to(torch.bfloat16)
    if tp is not None:
        for p in model.replicated_parameters():
            dist.broadcast(p.data, src=0)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    ids = torch.randint(0, cfg.vocab_size, (2, 65), generator=torch.Generator().manual_seed(7)).to(dev)
    losses = []
    for _ in range(5):
        loss = model(ids[:, :-1].contiguous(), targets=ids[:, 1:].contiguous())
        loss.backward()
        if tp is not None:
            for p in model.replicated_parameters():
                dist.all_reduce(p.grad)
        opt.step()
        opt.zero_grad(set_to_none=True)
        losses.append(loss.item())

    # ---- context parallelism: each rank holds S / world tokens of q, k, v
    B, S, H, D = 1, 16 * world, 4 * world, 16
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(B, S, H, D, generator=g).to(dev) for _ in range(3))
    n = S // world
    mine = slice(rank * n, (rank + 1) * n)
    full = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                           is_causal=True).transpose(1, 2)
    errs = {}
    for name, fn in (("ulysses", ulysses_attention), ("ring", ring_attention)):
        out = fn(q[:, mine].contiguous(), k[:, mine].contiguous(), v[:, mine].contiguous(), causal=True)
        errs[name] = float((out.float() - full[:, mine].float()).abs().max())
    if rank == 0:
        print(f"tp{world} loss {losses[0]:.3f} -> {losses[-1]:.3f}; context-parallel max error {errs}")
    dist.barrier()
    dist.destroy_process_group()
    return losses, errs


if __name__ == "__main__":
    main()
