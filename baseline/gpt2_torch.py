#!/usr/bin/env python
"""Constructed baseline: GPT-2-medium training step with stock PyTorch only (cuBLAS GEMMs, SDPA flash
attention, fused AdamW, FSDP2 `fully_shard` + NCCL when launched on more than one GPU).

Same shapes, synthetic data, dtype policy (bf16 compute, fp32 master weights) and timing rules as the
repository's bench.py; none of this package's kernels or engine are imported. The logits reach the loss in bf16
(no fp32 copy of the [tokens, vocab] matrix). `--compile` wraps the model in `torch.compile`; bench.py runs both
variants and keeps the faster one.

  python baseline/gpt2_torch.py --steps 20 --warmup 4 [--compile]
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 baseline/gpt2_torch.py --gpus 8
"""
import argparse
import json
import math
import os
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, E, H):
        super().__init__()
        self.ln_1, self.ln_2 = nn.LayerNorm(E), nn.LayerNorm(E)
        self.c_attn, self.c_proj = nn.Linear(E, 3 * E), nn.Linear(E, E)
        self.c_fc, self.c_proj2 = nn.Linear(E, 4 * E), nn.Linear(4 * E, E)
        self.H = H

    def forward(self, x):
        B, S, E = x.shape
        q, k, v = self.c_attn(self.ln_1(x)).split(E, dim=2)
        sp = lambda t: t.view(B, S, self.H, E // self.H).transpose(1, 2)
        a = F.scaled_dot_product_attention(sp(q), sp(k), sp(v), is_causal=True)
        x = x + self.c_proj(a.transpose(1, 2).reshape(B, S, E))
        return x + self.c_proj2(F.gelu(self.c_fc(self.ln_2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, V=50257, P=1024, E=1024, L=24, H=16):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(V, E), nn.Embedding(P, E)
        self.h = nn.ModuleList([Block(E, H) for _ in range(L)])
        self.ln_f = nn.LayerNorm(E)
        self.apply(lambda m: nn.init.normal_(m.weight, std=0.02) if isinstance(m, (nn.Linear, nn.Embedding)) else None)

    def forward(self, ids, targets):
        S = ids.shape[1]
        x = self.wte(ids) + self.wpe(torch.arange(S, device=ids.device))
        for b in self.h:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)
        with torch.autocast("cuda", enabled=False):   # autocast would widen the [tokens, vocab] logits to fp32
            return F.cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--compile", action="store_true")
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)
    B, S = 8, 1024
    model = GPT2().to(dev)
    if world > 1:
        # FSDP2 with its defaults (full shard, reshard after forward, prefetching), one unit per block + the root;
        # fp32 parameters are the master weights, compute and all-gathers in bf16, gradient reduction in fp32
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for blk in model.h:
            fully_shard(blk, mp_policy=mp)
        fully_shard(model, mp_policy=mp)
        ctx = torch.autocast("cuda", enabled=False)
    else:
        ctx = torch.autocast("cuda", dtype=torch.bfloat16)
    if a.compile:
        model = torch.compile(model)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.01, fused=True)
    g = torch.Generator().manual_seed(1000 + rank)
    nb = a.steps + a.warmup
    data = torch.randint(0, 50257, (nb, B, S + 1), generator=g)
    ids_h, tgt_h = data[:, :, :-1].contiguous().pin_memory(), data[:, :, 1:].contiguous().pin_memory()
    ids_d, tgt_d = ids_h[0].to(dev), tgt_h[0].to(dev)

    def step(ids, tgt):
        with ctx:
            loss = model(ids, tgt)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(a.warmup):
        step(ids_h[i].to(dev, non_blocking=True), tgt_h[i].to(dev, non_blocking=True)).item()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        step(ids_d, tgt_d)
    e1.record()
    sync()
    dev_ms = e0.elapsed_time(e1)
    t0 = time.perf_counter()
    for i in range(a.steps):
        last = step(ids_h[a.warmup + i].to(dev, non_blocking=True), tgt_h[a.warmup + i].to(dev, non_blocking=True)).item()
    sync()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    tokens = world * B * S * a.steps
    if rank == 0:
        print(json.dumps({"impl": "baseline-pytorch" + ("-compile" if a.compile else ""), "metric": "tokens/sec",
                          "value": tokens / dev_ms * 1e3, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
                          "warmup": a.warmup, "ms_per_step": dev_ms / a.steps, "dtype": "bf16",
                          "e2e": {"value": tokens / e2e_ms * 1e3, "ms_per_step": e2e_ms / a.steps}, "loss_last": last,
                          "config": {"model": "gpt2-medium", "global_batch": world * B, "seq_len": S,
                                     "parallelism": f"fsdp{world}" if world > 1 else "single"}}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
