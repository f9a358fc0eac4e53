#!/usr/bin/env python
"""Headline benchmark: GPT-2-medium causal-LM training throughput (tokens/s) on N B200 GPUs.

Config (fixed by the baseline definition): 24 layers, d_model 1024, 16 heads, FFN 4096 GELU, vocab
50 257, sequence 1024, micro-batch 8 per GPU, bf16 parameters/activations with fp32 master weights
and AdamW, FSDP full-shard across the GPUs (N = 1 degenerates to the unsharded flat buffers).
Synthetic uniform-random token ids, random-init N(0, 0.02) weights.

  python bench.py --gpus 1 --steps 20 --warmup 5
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5

Prints ONE JSON line on rank 0. `value` is device-timed (CUDA events, max over ranks) over exactly K
steps; `e2e` times the same K steps through `CausalLMTrainer.step_async` (one step in flight), including the
pinned-host → device copy of every batch and the device → host read of every step's loss.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.lines, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for ln in self.proc.stdout:
            self.lines.append((time.perf_counter(), ln.strip()))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        return self.window(float("-inf"), float("inf"))

    def window(self, t0: float, t1: float) -> dict:
        """Statistics of the samples that arrived between two ``time.perf_counter()`` instants."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm, mx, reasons = [], None, set()
        for ts, ln in list(self.lines):
            if not (t0 <= ts <= t1 + 0.05):
                continue
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def reference_arm(args):
    # The reference (cool-japan/torsh) is a Rust workspace whose Python package builds with maturin;
    # `pip install --no-index --no-build-isolation` fails here with "No module named 'maturin'", there is
    # no Rust toolchain, and its NCCL backend is a mock, so no reference number can be produced.
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference cannot be installed offline: build backend maturin and a Rust toolchain are "
                      "missing (pip: ModuleNotFoundError: No module named 'maturin')"}))
    return 0


def _child_env(port_offset: int) -> dict:
    """Environment of a child benchmark process of this rank: same RANK / WORLD_SIZE / LOCAL_RANK, its own rendezvous
    port, and none of the launcher's agent-store settings (the child ranks form their own process group)."""
    env = {k: v for k, v in os.environ.items() if not k.startswith("TORCHELASTIC_")}
    env["MASTER_ADDR"] = "127.0.0.1"
    env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29517")) + port_offset)
    env.setdefault("RANK", "0"); env.setdefault("WORLD_SIZE", "1"); env.setdefault("LOCAL_RANK", "0")
    return env


def run_child(argv: list[str], port_offset: int, timeout_s: float) -> dict:
    """Runs one benchmark script as a child of EVERY rank (the children rendezvous among themselves) and returns the
    JSON line its rank 0 printed, or ``{"failed": reason}``. Never raises: a broken extra arm must not cost the
    headline number."""
    t0 = time.perf_counter()
    try:
        r = subprocess.run([sys.executable] + argv, env=_child_env(port_offset), capture_output=True, text=True,
                           timeout=timeout_s, cwd=REPO)
    except subprocess.TimeoutExpired:
        return {"failed": f"timed out after {timeout_s:.0f} s"}
    except OSError as e:
        return {"failed": str(e)}
    out = None
    for ln in r.stdout.splitlines():
        ln = ln.strip()
        if ln.startswith("{") and ln.endswith("}"):
            try:
                out = json.loads(ln)
            except json.JSONDecodeError:
                pass
    if r.returncode != 0:
        return {"failed": f"exit code {r.returncode}: {r.stderr.strip().splitlines()[-1][:200] if r.stderr.strip() else ''}"}
    out = out or {}
    out["wall_s"] = round(time.perf_counter() - t0, 1)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="run every step eagerly (no CUDA-graph replay)")
    ap.add_argument("--model", default="gpt2-medium", choices=["gpt2-medium", "gpt2-small", "gpt2-tiny"])
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--fsdp-comm-blocks", type=int, default=0, help="CTAs of the fused FSDP kernel while it overlaps backward")
    ap.add_argument("--fsdp-no-overlap", action="store_true", help="one fused FSDP launch after backward (the default)")
    ap.add_argument("--fsdp-overlap", action="store_true", help="launch each block's FSDP kernel from a backward hook on a side stream")
    ap.add_argument("--fsdp-nvls", type=int, default=None, help="1 / 0: force NVLS multimem on / off in the fused FSDP kernel")
    ap.add_argument("--fsdp-coarse", type=int, default=0, help="with --fsdp-overlap: merge the per-block units into this many groups")
    ap.add_argument("--fsdp-strategy", default="full_shard", choices=["full_shard", "shard_grad_op", "no_shard"],
                    help="full_shard: 1/N of every weight resident, un-shard fused into each block's first GEMM, "
                         "reduce-scatter + AdamW per block under backward; shard_grad_op: replicated bf16 parameters and "
                         "gradients, sharded optimizer, one fused reduce-scatter + AdamW + all-gather launch")
    ap.add_argument("--fsdp-gather", default="copy_engine", choices=["copy_engine", "fused", "kernel"],
                    help="full_shard: how blocks are un-sharded (DMA prefetch on a side stream / inside the first GEMM / stand-alone kernel)")
    ap.add_argument("--fsdp-no-fuse-gather", action="store_true", help="same as --fsdp-gather kernel")
    ap.add_argument("--fsdp-overlap-rs", action="store_true", help="full_shard: per-block reduce-scatter + AdamW on a side stream")
    ap.add_argument("--fsdp-gather-ctas", type=int, default=0)
    ap.add_argument("--fsdp-rs-blocks", type=int, default=0)
    ap.add_argument("--fsdp-rs-threads", type=int, default=0)
    ap.add_argument("--fsdp-no-overlap-rs", action="store_true", help="full_shard: each block's reduce-scatter + AdamW on the main stream at full width")
    ap.add_argument("--fsdp-single", action="store_true",
                    help="diagnostic: run the FSDP engine in a one-rank group on one GPU (its kernels without any peer)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the constructed PyTorch baseline arm (child processes)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the ResNet-50 DDP and Llama 3-D secondary benchmarks")
    ap.add_argument("--budget-s", type=float, default=float(os.environ.get("TORSH_BENCH_BUDGET_S", "700")),
                    help="wall-clock budget of the whole invocation; extra arms that no longer fit are skipped")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)
    t_start = time.perf_counter()
    headline = args.model == "gpt2-medium" and not args.fsdp_single and not args.no_graph
    left = lambda: args.budget_s - (time.perf_counter() - t_start)

    # ---- constructed baseline (stock PyTorch: cuBLAS, SDPA, fused AdamW, FSDP2 over NCCL) as child processes on the
    #      same GPUs, BEFORE this process creates its CUDA context; eager and torch.compile variants, the faster wins
    baseline = None
    if headline and not args.no_baseline:
        base_cmd = [os.path.join(REPO, "baseline", "gpt2_torch.py"), "--gpus", str(args.gpus), "--steps",
                    str(max(args.steps, 20)), "--warmup", "4"]
        arms = {"eager": run_child(base_cmd, 11, min(300.0, max(left() - 200, 60)))}
        if left() > 420:
            arms["compile"] = run_child(base_cmd + ["--compile"], 12, min(330.0, left() - 200))
        ok = {k: v for k, v in arms.items() if "value" in v}
        if ok:
            best = max(ok, key=lambda k: ok[k]["value"])
            baseline = {"variant": best, "value": ok[best]["value"], "ms_per_step": ok[best]["ms_per_step"],
                        "e2e_value": ok[best]["e2e"]["value"], "arms": {k: (v.get("value") or v.get("failed")) for k, v in arms.items()}}
        else:
            baseline = {"variant": None, "arms": {k: v.get("failed") for k, v in arms.items()}}

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be launched with torch.distributed.run", file=sys.stderr)
            return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 or args.fsdp_single:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group("nccl", device_id=dev)

    from torsh_b200 import _native as nv
    from torsh_b200.engine import CausalLMTrainer
    from torsh_b200.models import GPT2Config, GPTForCausalLM

    cfg = {"gpt2-medium": GPT2Config.medium, "gpt2-small": GPT2Config.small, "gpt2-tiny": GPT2Config.tiny}[args.model](
        embd_pdrop=0.0, attn_pdrop=0.0, resid_pdrop=0.0)
    B, S = args.micro_batch, min(args.seq_len, cfg.n_positions)
    torch.manual_seed(1234)
    model = GPTForCausalLM(cfg).to(dev)
    parallel = None
    if world > 1 or args.fsdp_single:
        from torsh_b200.parallel.fsdp import FlatFSDP, FsdpConfig, ShardingStrategy
        fc = FsdpConfig(sharding_strategy=ShardingStrategy(args.fsdp_strategy))
        fc.gather_mode = "kernel" if args.fsdp_no_fuse_gather else args.fsdp_gather
        fc.fuse_gather = fc.gather_mode == "fused"
        if args.fsdp_gather_ctas:
            fc.gather_ctas = args.fsdp_gather_ctas
        if args.fsdp_rs_blocks:
            fc.rs_blocks = args.fsdp_rs_blocks
        if args.fsdp_rs_threads:
            fc.rs_threads = args.fsdp_rs_threads
        fc.overlap_rs = True if args.fsdp_overlap_rs else (False if args.fsdp_no_overlap_rs else None)
        if args.fsdp_comm_blocks:
            fc.comm_blocks = args.fsdp_comm_blocks
        fc.overlap = bool(args.fsdp_overlap) and not args.fsdp_no_overlap
        fc.coarse_units = args.fsdp_coarse
        if args.fsdp_nvls is not None:
            fc.use_nvls = bool(args.fsdp_nvls)
        parallel = FlatFSDP(dist.group.WORLD, fc)
    trainer = CausalLMTrainer(model, lr=3e-4, weight_decay=0.01, batch_size=B, seq_len=S,
                              use_graph=not args.no_graph, parallel=parallel)

    # synthetic data: one pinned host batch per step (uniform random ids, targets = next ids)
    g = torch.Generator().manual_seed(1000 + rank)
    nb = args.steps + args.warmup
    data = torch.randint(0, cfg.vocab_size, (nb, B, S + 1), generator=g, dtype=torch.int64)
    ids_host = data[:, :, :-1].contiguous().pin_memory()
    tgt_host = data[:, :, 1:].contiguous().pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (eager steps, graph capture, first replays) through the public step() call
    sampler = ClockSampler(local_rank)      # one nvidia-smi process for the whole run; the regions pick their samples
    sampler.start()
    losses = []
    for i in range(args.warmup):
        losses.append(trainer.step(ids_host[i], tgt_host[i]))
    nv.check_status()

    # ---- end-to-end region (first: it is the headline): K steps through step_async(), H2D of the batch + D2H of the
    #      loss every step
    barrier()
    t0 = time.perf_counter()
    pending = None
    marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for i in range(args.steps):
        # one step in flight: step i is staged and launched, then the loss of step i - 1 is read
        marks[i][0].record()
        nxt = trainer.step_async(ids_host[args.warmup + i], tgt_host[args.warmup + i])
        marks[i][1].record()
        if pending is not None:
            losses.append(pending.value())
        pending = nxt
    losses.append(pending.value())
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    # how long the device sat idle between consecutive steps of the end-to-end region
    idle_ms = sum(marks[i][1].elapsed_time(marks[i + 1][0]) for i in range(args.steps - 1)) / max(1, args.steps - 1)
    busy_ms = sum(a.elapsed_time(b) for a, b in marks) / args.steps
    e2e_clocks = sampler.window(t0, time.perf_counter())

    # ---- device-timed region: K steps on resident batches (kernel-only number)
    barrier()
    t_dev0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        trainer.step_device_only()
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    clocks = sampler.window(t_dev0, time.perf_counter())
    sampler.stop()

    nv.check_status()
    h2d_bytes, d2h_bytes = trainer.h2d_bytes_per_step, trainer.d2h_bytes_per_step

    t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    tokens = world * B * S * args.steps
    value = tokens / (dev_ms / 1e3)
    e2e = tokens / (e2e_ms / 1e3)

    # ---- multi-GPU correctness evidence taken after the timed steps
    checks = None
    if parallel is not None and world > 1:
        checks = {"status_word": 0}   # nv.check_status() above would have raised otherwise
        from torsh_b200.parallel.fsdp import FullShardParameters
        flat = trainer.flat
        vec = flat.full_lowp().float() if isinstance(flat, FullShardParameters) else flat.lowp.float()
        # (full shard: the gathered weights are the same bytes on every rank by construction; the test bites on the
        # replicated small parameters and, for the other strategies, on every rank's copy of every parameter)
        mx, mn = vec.clone(), vec.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX); dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        checks["params_identical_across_ranks"] = bool(torch.equal(mx, mn))
        # loss of the first timed step against a one-GPU evaluation is not repeated here (it needs the global batch on
        # one device); the per-rank losses of step 0 are identical functions of the same weights:
        l0 = torch.tensor([losses[0]], dtype=torch.float64, device=dev)
        l0max, l0min = l0.clone(), l0.clone()
        dist.all_reduce(l0max, op=dist.ReduceOp.MAX); dist.all_reduce(l0min, op=dist.ReduceOp.MIN)
        checks["step0_loss_min_max_over_ranks"] = [l0min.item(), l0max.item()]
        checks["step0_loss_expected_ln_vocab"] = round(float(__import__("math").log(cfg.vocab_size)), 4)
        ll = torch.tensor([losses[-1]], dtype=torch.float64, device=dev)
        dist.all_reduce(ll)
        checks["last_loss_mean_over_ranks"] = ll.item() / world
        del vec, mx, mn

    # ---- secondary benchmarks (child processes on the same GPUs, after this process has released its memory)
    secondary = None
    if headline and not args.no_secondary:
        launches_per_step, strategy = trainer.launches_per_step, (parallel.strategy.value if parallel is not None else "none")
        mem_report = parallel.memory_report() if parallel is not None else None
        graph_on = trainer.graph is not None
        del trainer, model, parallel
        if dist.is_initialized():
            dist.barrier()
        import gc
        gc.collect(); torch.cuda.empty_cache()
        secondary = {}
        rn = os.path.join(REPO, "bench", "resnet50.py")
        if left() > 150:
            ours = run_child([rn, "--gpus", str(world), "--steps", "10", "--warmup", "3"], 21, min(200.0, left() - 60))
            base = run_child([rn, "--gpus", str(world), "--steps", "10", "--warmup", "3", "--impl", "torch"], 22, min(200.0, max(left() - 40, 30))) if left() > 90 else {"failed": "no time left"}
            secondary["resnet50_ddp"] = {
                "metric": "images/s (ResNet-50, batch 256/GPU, bf16, SGD 0.9, DDP 25 MB buckets)",
                "value": ours.get("value"), "e2e_value": (ours.get("e2e") or {}).get("value"), "ms_per_step": ours.get("ms_per_step"),
                "baseline_value": base.get("value"), "ratio": (ours["value"] / base["value"]) if ours.get("value") and base.get("value") else None,
                "failed": ours.get("failed") or base.get("failed")}
        if world == 8 and left() > 260:
            ll3 = os.path.join(REPO, "bench", "llama_3d.py")
            ours = run_child([ll3, "--tp", "4", "--pp", "2", "--steps", "10", "--warmup", "3"], 23, min(240.0, left() - 130))
            base = run_child([ll3, "--tp", "4", "--pp", "2", "--steps", "10", "--warmup", "3", "--impl", "nccl"], 24, min(240.0, max(left() - 20, 30))) if left() > 120 else {"failed": "no time left"}
            secondary["llama7b_tp4_pp2"] = {
                "metric": "tokens/s (Llama-style 7B, seq 4096, TP4(+SP) x PP2 1F1B, 8 micro-batches)",
                "value": ours.get("value"), "e2e_value": (ours.get("e2e") or {}).get("value"), "ms_per_step": ours.get("ms_per_step"),
                "baseline_value": base.get("value"), "ratio": (ours["value"] / base["value"]) if ours.get("value") and base.get("value") else None,
                "failed": ours.get("failed") or base.get("failed")}
    else:
        launches_per_step, strategy = trainer.launches_per_step, (parallel.strategy.value if parallel is not None else "none")
        mem_report = parallel.memory_report() if parallel is not None else None
        graph_on = trainer.graph is not None
    if rank == 0:
        out = {
            "metric": "tokens/sec (GPT-2-medium training step, device-timed, max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "config": {"model": args.model, "layers": cfg.n_layer, "d_model": cfg.n_embd, "heads": cfg.n_head,
                       "ffn": cfg.inner, "vocab": cfg.vocab_size, "global_batch": world * B, "micro_batch_per_gpu": B,
                       "seq_len": S, "optimizer": "AdamW fp32 master weights", "dropout": 0.0,
                       "parallelism": f"fsdp{world}" if strategy != "none" else "single",
                       "sharding": strategy,
                       "memory_per_rank": mem_report,
                       "cuda_graph": graph_on,
                       "l2": "working set per step (>10 GB) far exceeds the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "device_busy_ms_per_step": busy_ms, "device_idle_ms_between_steps": idle_ms,
                    "clocks": e2e_clocks,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "loss_first": losses[0], "loss_last": losses[-1],
            # the constructed baseline of this very invocation (same GPUs, child processes, run first)
            "vs_constructed_baseline": None if baseline is None else {
                **baseline,
                "value_ratio": (value / baseline["value"]) if baseline.get("value") else None,
                "e2e_ratio": (e2e / baseline["e2e_value"]) if baseline.get("e2e_value") else None},
            "checks": checks, "secondary": secondary,
        }
        print(json.dumps(out))
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
