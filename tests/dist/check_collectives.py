"""Multi-rank checks run under torch.distributed.run (one process per GPU).

  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29531 \
      tests/dist/check_collectives.py [collectives] [fsdp] [bench]
Exit code 0 means every selected check passed on every rank.
"""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist


def log(*a):
    if dist.get_rank() == 0:
        print(*a, flush=True)


def check_collectives(dev):
    from torsh_b200 import _native as nv
    from torsh_b200.parallel.collectives import FusedCollectives
    from torsh_b200.parallel.symm import SymmetricBuffer
    rank, world = dist.get_rank(), dist.get_world_size()
    fc = FusedCollectives(nblocks=32)
    ok = True
    for dtype in (torch.float32, torch.bfloat16):
        n = 1 << 20
        buf = SymmetricBuffer(n, dtype)
        log(f"multicast available: {buf.has_multicast}")
        modes = ["one_shot", "two_shot"]
        for use_nvls in ([True, False] if buf.has_multicast else [False]):
            fc.use_nvls = use_nvls
            for mode in modes:
                numel = 4096 * 8 if mode == "one_shot" else n
                g = torch.Generator(device=dev).manual_seed(100 + rank)
                x = torch.randn(numel, device=dev, dtype=dtype, generator=g)
                ref = x.float().clone()
                dist.all_reduce(ref)
                buf.tensor[:numel].copy_(x)
                fc.all_reduce_(buf, numel=numel, scale=0.5, mode=mode)
                torch.cuda.synchronize()
                nv.check_status()
                err = (buf.tensor[:numel].float() - 0.5 * ref).abs().max().item()
                tol = 0.05 if dtype == torch.bfloat16 else 1e-4
                # every rank must hold the same bits: replicated parameters are stepped with these sums
                got = buf.tensor[:numel].float().clone()
                hi, lo = got.clone(), got.clone()
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                same = torch.equal(hi, lo)
                log(f"all_reduce {dtype} {mode} nvls={use_nvls}: max err {err:.5f}, identical on all ranks: {same}")
                ok &= err < tol and same
            # all-gather
            chunk = n // world
            buf.tensor.zero_()
            buf.tensor[rank * chunk:(rank + 1) * chunk] = rank + 1
            fc.all_gather_(buf, chunk)
            torch.cuda.synchronize()
            nv.check_status()
            exp = torch.arange(1, world + 1, device=dev).repeat_interleave(chunk).to(dtype)
            ok &= torch.equal(buf.tensor, exp)
            log(f"all_gather {dtype} nvls={use_nvls}: {'ok' if torch.equal(buf.tensor, exp) else 'MISMATCH'}")
            # reduce-scatter
            g = torch.Generator(device=dev).manual_seed(200 + rank)
            x = torch.randn(n, device=dev, dtype=dtype, generator=g)
            ref = x.float().clone()
            dist.all_reduce(ref)
            buf.tensor.copy_(x)
            out = fc.reduce_scatter(buf, chunk, scale=1.0 / world)
            torch.cuda.synchronize()
            nv.check_status()
            err = (out.float() - ref[rank * chunk:(rank + 1) * chunk] / world).abs().max().item()
            log(f"reduce_scatter {dtype} nvls={use_nvls}: max err {err:.5f}")
            ok &= err < (0.05 if dtype == torch.bfloat16 else 1e-4)
    # bandwidth of the two-shot all-reduce vs NCCL (device-timed, max over ranks)
    fc.use_nvls = None
    for nbytes in (1 << 20, 1 << 24, 1 << 28):
        n = nbytes // 2
        buf = SymmetricBuffer(n, torch.bfloat16)
        x = torch.randn(n, device=dev, dtype=torch.bfloat16)
        for name, fn in (("fused", lambda: fc.all_reduce_(buf, mode="two_shot")), ("nccl", lambda: dist.all_reduce(x))):
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier(); torch.cuda.synchronize()
            e0.record()
            for _ in range(10):
                fn()
            e1.record(); torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 10], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            busbw = nbytes * 2 * (world - 1) / world / (t.item() * 1e-3) / 1e9
            log(f"all_reduce {nbytes >> 20} MiB {name}: {t.item() * 1e3:.1f} us, bus bw {busbw:.0f} GB/s")
        nv.check_status()
    return ok


def check_fsdp(dev):
    """2+ ranks of every FSDP strategy must reproduce a single-process AdamW run on the global batch: the loss of every
    step within 0.2 % of the oracle's, parameters bit-identical on every rank, and after six steps every weight matrix
    within 1 % (relative L2) of the oracle's. Element-wise equality with the oracle is not expected: the gradient sums
    are formed in a different order, and AdamW turns the rounding noise of gradients that are zero in exact arithmetic
    (the key bias of an attention layer) into full-size steps."""
    from torsh_b200 import _native as nv
    from torsh_b200.engine import CausalLMTrainer
    from torsh_b200.models import GPT2Config, GPTForCausalLM
    from torsh_b200.parallel.fsdp import FlatFSDP, FsdpConfig, ShardingStrategy
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = GPT2Config.tiny()
    B, S, steps = 4, 128, 6
    data = torch.randint(0, cfg.vocab_size, (world * B, S + 1), generator=torch.Generator().manual_seed(7))
    ok = True
    # single-process oracle on the global batch (this rank's GPU, plain flat AdamW)
    torch.manual_seed(0)
    m1 = GPTForCausalLM(cfg).to(dev)
    t1 = CausalLMTrainer(m1, lr=1e-3, weight_decay=0.01, batch_size=world * B, seq_len=S, use_graph=False)
    gx, gy = data[:, :-1].contiguous().pin_memory(), data[:, 1:].contiguous().pin_memory()
    ref_losses = [t1.step(gx, gy) for _ in range(steps)]
    ref_params = {n: p.detach().float().clone() for n, p in m1.named_parameters()}
    log(f"single-process oracle: {[round(v, 4) for v in ref_losses]}")
    FS, SGO, NS = ShardingStrategy.FULL_SHARD, ShardingStrategy.SHARD_GRAD_OP, ShardingStrategy.NO_SHARD
    cases = [(SGO, dict(overlap=False), False), (SGO, dict(overlap=False), True), (SGO, dict(overlap=True), False),
             (SGO, dict(overlap=True), True), (FS, dict(), False), (FS, dict(), True), (FS, dict(overlap_rs=True), True),
             (FS, dict(gather_mode="fused", fuse_gather=True), False), (FS, dict(gather_mode="fused", fuse_gather=True), True),
             (FS, dict(gather_mode="kernel", fuse_gather=False, overlap_rs=True), True), (NS, dict(), True)]
    for strategy, kw, use_graph in cases:
        torch.manual_seed(0)
        model = GPTForCausalLM(cfg).to(dev)
        eng = FlatFSDP(config=FsdpConfig(sharding_strategy=strategy, **kw))
        tr = CausalLMTrainer(model, lr=1e-3, weight_decay=0.01, batch_size=B, seq_len=S, use_graph=use_graph,
                             warmup_eager=2, parallel=eng)
        mine = data[rank * B:(rank + 1) * B]
        x, y = mine[:, :-1].contiguous().pin_memory(), mine[:, 1:].contiguous().pin_memory()
        losses = []
        for _ in range(steps):
            l = torch.tensor([tr.step(x, y)], device=dev)
            dist.all_reduce(l)
            losses.append(l.item() / world)
        torch.cuda.synchronize()
        nv.check_status()
        if strategy is FS:
            got = {n: v.float() for n, v in tr.flat.full_state_dict(model).items()}
            flat = torch.cat([v.reshape(-1) for v in got.values()])
        else:
            got = {n: p.detach().float() for n, p in model.named_parameters()}
            flat = tr.flat.lowp.float()
        mx = flat.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        mn = flat.clone(); dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        same = torch.equal(mx, mn)
        worst = 0.0
        for n, v in got.items():
            r = ref_params[n]
            if r.dim() >= 2:
                worst = max(worst, ((v - r).norm() / r.norm().clamp(min=1e-12)).item())
        tag = f"{strategy.value} {kw} graph={use_graph}"
        log(f"fsdp {tag}: losses {[round(v, 4) for v in losses]} identical across ranks={same} "
            f"max relative L2 distance of a weight from the oracle {worst:.5f}; memory {eng.memory_report()}")
        ok &= same and losses[-1] < losses[0] - 0.5 and worst <= 1e-2
        for a_, b_ in zip(losses, ref_losses):
            ok &= abs(a_ - b_) < 2e-3 * abs(b_)
        del tr, eng, model
    return ok


def check_tp(dev):
    """Fused AG->GEMM / GEMM->RS layers against the same algebra on NCCL collectives + cuBLAS."""
    from torsh_b200 import _native as nv
    from torsh_b200.parallel.tensor_parallel import (ColumnParallelLinear, RowParallelLinear, TensorParallelConfig,
                                                     TPContext, _ag_gemm, _gemm_rs)
    rank, world = dist.get_rank(), dist.get_world_size()
    ok = True
    for rs_fp32 in (False, True):
        tpc = TPContext(config=TensorParallelConfig(tp_size=world, rs_fp32=rs_fp32))
        M, H, Fh = 1024 * world, 1024, 4096
        torch.manual_seed(100 + rank)
        col = ColumnParallelLinear(H, Fh, tp=tpc, device=dev, dtype=torch.bfloat16)
        row = RowParallelLinear(Fh, H, tp=tpc, device=dev, dtype=torch.bfloat16)
        x = torch.randn(M // world, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
        res = torch.randn(M // world, H, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(M // world, H, device=dev, dtype=torch.bfloat16)
        y = row(torch.nn.functional.gelu(col(x), approximate="tanh"), residual=res)
        y.backward(dy)
        torch.cuda.synchronize()
        nv.check_status()
        got = [y.detach().float(), x.grad.float(), col.weight.grad.float(), row.weight.grad.float(), row.bias.grad.float()]
        # oracle: same modules, unfused path (tp=None -> torch.distributed collectives), fp32 math
        col.tp = row.tp = None
        for p in list(col.parameters()) + list(row.parameters()):
            p.grad = None
            p.data = p.data.float()
        xf = x.detach().float().requires_grad_(True)
        yr = row(torch.nn.functional.gelu(col(xf), approximate="tanh"), residual=res.float())
        yr.backward(dy.float())
        ref = [yr.detach(), xf.grad, col.weight.grad, row.weight.grad, row.bias.grad]
        for name, a, b in zip(("y", "dx", "dW_col", "dW_row", "db_row"), got, ref):
            rel = ((a - b).abs().max() / b.abs().max().clamp(min=1e-6)).item()
            log(f"tp rs_fp32={rs_fp32} {name}: rel err {rel:.4f}")
            ok &= rel < 0.05
    # timing sweep: fused kernels vs NCCL collective + cuBLAS GEMM (device-timed, max over ranks)
    tpc = TPContext(config=TensorParallelConfig(tp_size=world))

    def timeit(fn, iters=10):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier(); torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for M in (4096, 16384, 32768):
        for NK in (4096, 8192):
            rows = M // world
            xs = torch.randn(rows, NK, device=dev, dtype=torch.bfloat16)
            w_col = torch.randn(NK // world, NK, device=dev, dtype=torch.bfloat16) * 0.02
            xf = torch.empty(M, NK, device=dev, dtype=torch.bfloat16)
            t_f = timeit(lambda: _ag_gemm(tpc, f"bench_ag{M}_{NK}", xs, w_col, 0))
            t_b = timeit(lambda: (dist.all_gather_into_tensor(xf, xs), torch.matmul(xf, w_col.t())))
            fl = 2.0 * M * NK * (NK // world)
            log(f"AG->GEMM M={M} N=K={NK}: fused {t_f*1e3:.0f} us ({fl/t_f/1e9:.0f} TF) | nccl+cublas {t_b*1e3:.0f} us")
            xk = torch.randn(M, NK // world, device=dev, dtype=torch.bfloat16)
            w_row = torch.randn(NK, NK // world, device=dev, dtype=torch.bfloat16) * 0.02
            out = torch.empty(rows, NK, device=dev, dtype=torch.bfloat16)
            t_f = timeit(lambda: _gemm_rs(tpc, f"bench_rs{M}_{NK}", xk, w_row, 0))
            t_b = timeit(lambda: dist.reduce_scatter_tensor(out, torch.matmul(xk, w_row.t())))
            log(f"GEMM->RS M={M} N=K={NK}: fused {t_f*1e3:.0f} us ({fl/t_f/1e9:.0f} TF) | cublas+nccl {t_b*1e3:.0f} us")
            nv.check_status()
    return ok


def check_ddp(dev):
    """Fused bucket all-reduce (x 1/world) launched from autograd hooks: every rank's gradients must equal the
    average, over ranks, of the gradients a plain copy of the model produces on each rank's own batch."""
    from torsh_b200 import _native as nv
    from torsh_b200.parallel.ddp import DistributedDataParallel
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(7)
    make = lambda: torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 512), torch.nn.GELU(),
                                       torch.nn.Linear(512, 64)).to(dev)
    model, ref = make(), make()
    ref.load_state_dict(model.state_dict())
    ddp = DistributedDataParallel(model, bucket_cap_mb=0.6)          # several buckets
    ok = len(ddp.buckets) >= 2
    for step in range(3):
        torch.manual_seed(100 + step)
        xs = torch.randn(world, 32, 256, device=dev)
        ys = torch.randn(world, 32, 64, device=dev)
        loss = torch.nn.functional.mse_loss(ddp(xs[rank]), ys[rank])
        loss.backward()
        ddp.sync_gradients()
        ref.zero_grad()
        for r in range(world):
            (torch.nn.functional.mse_loss(ref(xs[r]), ys[r]) / world).backward()
        for (n, p), q in zip(model.named_parameters(), ref.parameters()):
            err = (p.grad - q.grad).abs().max().item() / (q.grad.abs().max().item() + 1e-12)
            if err > 1e-4:
                ok = False
                log(f"ddp step {step} {n}: rel err {err:.2e}")
        with torch.no_grad():
            for p, q in zip(model.parameters(), ref.parameters()):
                p.add_(p.grad, alpha=-0.1)
                q.add_(q.grad, alpha=-0.1)
        ddp.zero_grad()
    nv.check_status()
    log(f"ddp: {len(ddp.buckets)} buckets, stats {ddp.get_sync_stats()} -> {'ok' if ok else 'FAILED'}")
    return ok


def check_moe(dev):
    """Peer-memory MoE dispatch / combine against a dense evaluation of the same routing with all experts local."""
    from torsh_b200 import _native as nv
    from torsh_b200.parallel.expert_parallel import ExpertParallelismConfig, MoELayer
    rank, world = dist.get_rank(), dist.get_world_size()
    H, Fh, E, T = 256, 512, 4 * world, 192
    cfg = ExpertParallelismConfig(num_experts=E, top_k=2, capacity_factor=float(E))      # no token is dropped
    torch.manual_seed(5)
    layer = MoELayer(H, Fh, cfg, group=dist.group.WORLD).to(dev).to(torch.bfloat16)
    with torch.no_grad():                                  # same router everywhere, experts differ per rank
        torch.manual_seed(50 + rank)
        layer.w1.normal_(0, 0.05); layer.w2.normal_(0, 0.05)
    torch.manual_seed(500 + rank)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    y, aux = layer(x)
    (y.float() * dy.float()).sum().backward()
    torch.cuda.synchronize()
    nv.check_status()
    got = [y.detach().float(), x.grad.float(), layer.router.gate.grad.float(), layer.w1.grad.float(), layer.w2.grad.float()]
    # dense oracle in fp32 with every expert's weights gathered
    w1 = [torch.empty_like(layer.w1.data) for _ in range(world)]; w2 = [torch.empty_like(layer.w2.data) for _ in range(world)]
    dist.all_gather(w1, layer.w1.data); dist.all_gather(w2, layer.w2.data)
    W1 = torch.cat(w1).float().requires_grad_(); W2 = torch.cat(w2).float().requires_grad_()
    xr = x.detach().float().requires_grad_()
    gate = layer.router.gate.detach().float().requires_grad_()
    probs = torch.softmax(xr.to(torch.bfloat16).float() @ gate.t(), -1)
    wts, idx = probs.topk(2, -1)
    wts = wts / wts.sum(-1, keepdim=True)
    ref = torch.zeros(T, H, device=dev)
    for k in range(2):
        for e in range(E):
            m = idx[:, k] == e
            if m.any():
                h = torch.nn.functional.gelu(xr[m] @ W1[e]) @ W2[e]
                ref = ref.index_add(0, m.nonzero().flatten(), wts[m, k, None] * h)
    (ref * dy.float()).sum().backward()
    dW1, dW2 = W1.grad.clone(), W2.grad.clone()
    dist.all_reduce(dW1); dist.all_reduce(dW2)
    el = E // world
    want = [ref.detach(), xr.grad, gate.grad, dW1[rank * el:(rank + 1) * el], dW2[rank * el:(rank + 1) * el]]
    ok = True
    for name, a, b in zip(("y", "dx", "dgate", "dW1", "dW2"), got, want):
        rel = ((a - b).abs().max() / b.abs().max().clamp(min=1e-6)).item()
        log(f"moe {name}: rel err {rel:.4f}")
        ok &= rel < 0.06
    return ok


def check_canaries(dev):
    """Run with TORSH_SYMM_CANARIES=1: every symmetric buffer carries guard bytes; after the fused collectives have run
    over the whole payload on every rank the guards must be untouched."""
    from torsh_b200 import _native as nv
    from torsh_b200.parallel.collectives import FusedCollectives
    from torsh_b200.parallel.symm import SymmetricBuffer
    rank, world = dist.get_rank(), dist.get_world_size()
    fc = FusedCollectives(nblocks=32)
    n = 1 << 18
    ok = True
    for dtype in (torch.float32, torch.bfloat16):
        buf = SymmetricBuffer(n, dtype)
        ok &= buf.guard_bytes == 256
        for use_nvls in ([True, False] if buf.has_multicast else [False]):
            fc.use_nvls = use_nvls
            x = torch.full((n,), float(rank + 1), device=dev, dtype=dtype)
            buf.tensor.copy_(x)
            fc.all_reduce_(buf, numel=n, scale=1.0, mode="two_shot")
            torch.cuda.synchronize()
            ok &= bool((buf.tensor.float() == world * (world + 1) / 2).all())
            chunk = n // world
            fc.all_gather_(buf, chunk)
            fc.reduce_scatter(buf, chunk, scale=1.0)
            torch.cuda.synchronize()
            nv.check_status()
            dist.barrier()
            good = buf.check_canaries() and fc.ctx.flags.check_canaries()
            log(f"canaries {dtype} nvls={use_nvls}: {'intact' if good else 'OVERWRITTEN'}")
            ok &= good
    return ok


def check_native_heap(dev):
    """The package's own symmetric heap (cuMemCreate blocks exchanged as file descriptors, cuMemMap of every peer, one
    multicast object): peers see each other's writes, the fused collectives run on its blocks through peer loads and
    through the multicast address, blocks are released collectively."""
    from torsh_b200 import _native as nv
    from torsh_b200.parallel.collectives import FusedCollectives
    from torsh_b200.parallel.symm import SymmetricBuffer
    rank, world = dist.get_rank(), dist.get_world_size()
    os.environ["TORSH_SYMM_BACKEND"] = "native"
    ok = True
    try:
        n = 1 << 20
        buf = SymmetricBuffer(n, torch.float32)
        ok &= buf.native and bool((buf.tensor == 0).all())
        buf.tensor.fill_(float(rank + 1))
        torch.cuda.synchronize()
        dist.barrier()
        for q in range(world):
            got = buf.peer_tensor(q)
            ok &= bool((got == float(q + 1)).all())
        dist.barrier()
        fc = FusedCollectives(nblocks=32)          # its flag buffer comes from the native heap too
        for use_nvls in ([False, True] if buf.has_multicast else [False]):
            fc.use_nvls = use_nvls
            buf.tensor.fill_(float(rank + 1))
            torch.cuda.synchronize()
            dist.barrier()
            fc.all_reduce_(buf, numel=n, scale=1.0, mode="two_shot")
            torch.cuda.synchronize()
            nv.check_status()
            good = bool((buf.tensor == world * (world + 1) / 2).all())
            log(f"native heap all-reduce nvls={use_nvls}: {'ok' if good else 'WRONG'} (multicast address {'yes' if buf.has_multicast else 'no'})")
            ok &= good
            dist.barrier()
        torch.cuda.synchronize()
        dist.barrier()
        buf.release()
        ok &= buf.tensor is None
    finally:
        os.environ["TORSH_SYMM_BACKEND"] = "torch"
    return ok


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    what = sys.argv[1:] or ["collectives", "fsdp"]
    ok = True
    if "collectives" in what:
        ok &= check_collectives(dev)
    if "fsdp" in what:
        ok &= check_fsdp(dev)
    if "tp" in what:
        ok &= check_tp(dev)
    if "ddp" in what:
        ok &= check_ddp(dev)
    if "moe" in what:
        ok &= check_moe(dev)
    if "canaries" in what:
        ok &= check_canaries(dev)
    if "native_heap" in what:
        ok &= check_native_heap(dev)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    log("ALL CHECKS PASSED" if flag.item() == 1 else "CHECKS FAILED")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
