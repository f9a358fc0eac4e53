#!/usr/bin/env python
"""Llama-style 7B training throughput (tokens/s) under 3-D parallelism: tensor parallel with sequence parallelism x
pipeline parallel (1F1B) x data parallel, bf16 with fp32 master weights and AdamW.

Named configuration: 32 layers, d_model 4096, 32 heads, SwiGLU FFN 11008, RMSNorm, RoPE theta 1e4, vocab 32000,
sequence 4096, TP 4 x PP 2 x DP 1 on 8 GPUs, 8 micro-batches of 1 x 4096 per step:

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29544 \
      bench/llama_3d.py --tp 4 --pp 2

``--impl fused`` (default): column- / row-parallel linears run the all-gather->GEMM and GEMM->reduce-scatter kernels
over NVSwitch peer memory; ``--impl nccl``: the same model with NCCL all-gather / reduce-scatter around library GEMMs
(the constructed baseline).  Pipeline activations travel over NCCL p2p in both.  ``--layers`` / ``--hidden`` shrink the
model for runs on fewer GPUs.  One JSON line on rank 0, device-timed, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=4)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micro-batches", type=int, default=8)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--pp-overlap", action="store_true",
                    help="pipeline transfers on per-link process groups with sends not waited for (default: blocking paired "
                         "exchanges on the pipeline group, which measured the same step time: 275.6 against 275.4 ms on two ranks)")
    ap.add_argument("--dense-head", action="store_true",
                    help="every TP rank computes all logits (default: vocabulary-parallel head and loss)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    assert world % (args.tp * args.pp) == 0, "world size must be a multiple of tp * pp"
    dp = world // (args.tp * args.pp)

    from bench import ClockSampler
    from torsh_b200 import _native as nv
    from torsh_b200.models.llama import LlamaConfig, LlamaModel
    from torsh_b200.ops import elementwise as ew
    from torsh_b200.optim.fused import AdamW
    from torsh_b200.parallel.mesh import DeviceMesh3D, ThreeDParallelismConfig
    from torsh_b200.parallel.pipeline import PipelineConfig, PipelineParallel, ScheduleType
    from torsh_b200.parallel.tensor_parallel import TensorParallelConfig, TPContext

    mesh = DeviceMesh3D(ThreeDParallelismConfig(dp_size=dp, tp_size=args.tp, pp_size=args.pp, num_layers=args.layers,
                                                micro_batch_size=1, num_micro_batches=args.micro_batches))
    mp = mesh.mapping
    cfg = LlamaConfig(vocab_size=args.vocab, hidden_size=args.hidden, intermediate_size=args.ffn, num_layers=args.layers,
                      num_heads=args.heads, max_seq_len=args.seq)
    tpc = TPContext(mesh.tp_group, TensorParallelConfig(tp_size=args.tp, fused=args.impl == "fused")) if args.tp > 1 else None
    torch.manual_seed(1234 + mp.pp_rank * 100 + mp.tp_rank)
    with torch.device(dev):
        model = LlamaModel(cfg, tp=tpc, layer_range=mp.layer_range(), first_stage=mesh.is_first_stage,
                           last_stage=mesh.is_last_stage, vocab_parallel=not args.dense_head)
    model = model.to(torch.bfloat16)
    if tpc is not None:
        # parameters that every tensor-parallel rank holds in full start from rank 0's values
        src = dist.get_global_rank(mesh.tp_group, 0)
        for p in model.replicated_parameters() + ([model.lm_head] if hasattr(model, "lm_head") else []):
            dist.broadcast(p.data, src=src, group=mesh.tp_group)
    opt = AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    B, S, M = 1, args.seq, args.micro_batches

    class Stage(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, x):
            if self.m.first_stage:
                x = self.m._shard_tokens(ew.embedding(x, self.m.embed).reshape(B * S, -1))
            for blk in self.m.layers:
                x = blk(x, B, S)
            return x

    stage = Stage(model)
    rows = B * S // args.tp if args.tp > 1 else B * S
    pipe = PipelineParallel(stage, group=mesh.pp_group,
                            config=PipelineConfig(num_micro_batches=M, schedule=ScheduleType.ONE_F_ONE_B,
                                                  overlap=args.pp_overlap, measure_idle=True),
                            activation_shape=(rows, args.hidden), activation_dtype=torch.bfloat16) if args.pp > 1 else None
    if pipe is not None and tpc is not None:
        pipe.micro_batch_hook = lambda mb, slot: setattr(tpc, "slot", slot)
    loss_fn = lambda h, y: model.head(h, B, S, y)
    replicated = model.replicated_parameters() if args.tp > 1 else []

    # a fresh batch of M micro-batches for every step (warm-up, device-timed and end-to-end steps all differ), generated
    # once in pinned host memory; the device-timed region reads resident copies, the end-to-end region copies each
    # step's batch from the host and reads the loss back
    import time
    g = torch.Generator().manual_seed(99 + mp.dp_rank)
    nb = args.warmup + 2 * args.steps
    ids_host = torch.randint(0, args.vocab, (nb, M, S + 1), generator=g).pin_memory()
    ids_dev = ids_host.to(dev)
    inp_buf = torch.empty(M, S, dtype=torch.int64, device=dev)
    tgt_buf = torch.empty(M, S, dtype=torch.int64, device=dev)

    def step(i, from_host=False):
        src = ids_host[i] if from_host else ids_dev[i]
        inp_buf.copy_(src[:, :-1], non_blocking=True)
        tgt_buf.copy_(src[:, 1:], non_blocking=True)
        inp, tgt = inp_buf, tgt_buf
        if pipe is not None:
            loss = pipe.train_step(inp if mesh.is_first_stage else None, tgt if mesh.is_last_stage else None, loss_fn)
        else:
            losses = []
            for mb in range(M):
                l = loss_fn(stage(inp[mb:mb + 1]), tgt[mb:mb + 1]) / M
                l.backward()
                losses.append(l.detach() * M)
            loss = torch.stack(losses).mean()
        for p in replicated:
            if p.grad is not None:
                dist.all_reduce(p.grad, group=mesh.tp_group)
        if dp > 1:
            for p in model.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.AVG, group=mesh.dp_group)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    launches0 = nv.launch_count
    for i in range(args.warmup):
        loss = step(i)
    per_step = (nv.launch_count - launches0) // args.warmup
    first = loss.item() if loss is not None else None
    nv.check_status()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step(args.warmup + i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # end to end: every step copies its batch from pinned host memory and the last stage reads the loss back
    t0 = time.perf_counter()
    for i in range(args.steps):
        loss = step(args.warmup + args.steps + i, from_host=True)
        if loss is not None:
            loss_value = loss.item()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    nv.check_status()
    # Python time to queue ONE step on an idle device (back to back the launch queue fills and hides it)
    t1 = time.perf_counter()
    step(args.warmup)
    host_issue_ms = (time.perf_counter() - t1) * 1e3
    barrier()
    # device time of the last step that no forward / backward action covered: the pipeline bubble plus exposed transfers
    idle = torch.tensor([pipe.idle_ms() or 0.0 if pipe is not None else 0.0], dtype=torch.float64, device=dev)
    dist.all_reduce(idle, op=dist.ReduceOp.MAX)
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    last = torch.tensor([loss.item() if loss is not None else 0.0, first if first is not None else 0.0], device=dev)
    dist.all_reduce(last, op=dist.ReduceOp.MAX)
    last, first_all = last[0], last[1].item()
    tokens = dp * M * B * S * args.steps
    n_params = args.layers * (4 * args.hidden ** 2 + 3 * args.hidden * args.ffn) + 2 * args.vocab * args.hidden
    if rank == 0:
        print(json.dumps({
            "metric": "tokens/sec (Llama-style training step, device-timed, max over ranks)", "impl": args.impl,
            "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "dtype": "bf16",
            "model_tflops_per_gpu": 6 * n_params * tokens / (ms / 1e3) / world / 1e12,
            "data": "synthetic (uniform random token ids, N(0,0.02) init)",
            "config": {"layers": args.layers, "d_model": args.hidden, "heads": args.heads, "ffn": args.ffn, "vocab": args.vocab,
                       "seq_len": S, "micro_batches": M, "head": "dense" if args.dense_head else "vocab-parallel", "parallelism": f"tp{args.tp}(sp) x pp{args.pp}(1f1b) x dp{dp}",
                       "params_b": round(n_params / 1e9, 2)},
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": M * (S + 1) * 8, "d2h_bytes_per_step": 4},
            "pipeline": {"transfers": "per-link groups, asynchronous sends" if args.pp_overlap else "blocking pairs",
                         "idle_ms_last_step_max_over_ranks": idle.item()},
            "clocks": clocks, "gpu_launches": per_step * args.steps, "launches_per_step": per_step,
            "host_issue_ms_per_step": host_issue_ms,
            "loss_after_warmup": first_all, "loss_last": last.item()}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
