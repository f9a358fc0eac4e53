"""CPU tests of the host-side parallel logic: planner arithmetic, stores, gloo ranks running DDP."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_bucket_assignment_largest_first():
    from torsh_b200.parallel import planner
    mb = 1024 * 1024
    sizes = [1 * mb, 20 * mb, 3 * mb, 10 * mb, 10 * mb, 4 * mb]
    got = planner.assign_buckets(sizes, 25 * mb)
    # sorted desc: 20,10,10,4,3,1 -> [20] | [10,10,4] | [3,1]
    assert got == [2, 0, 2, 1, 1, 1]
    assert planner.assign_buckets([], 25 * mb) == []


def test_shard_ranges_cover_everything():
    from torsh_b200.parallel import planner
    from torsh_b200.parallel.fsdp import shard_range
    for numel, world in ((10, 4), (1000, 8), (7, 8), (64, 2)):
        prev = 0
        for r in range(world):
            s, e = planner.shard_range(numel, world, r)
            assert (s, e) == shard_range(numel, world, r) and s == prev
            base, rem = divmod(numel, world)
            assert e - s == base + (1 if r < rem else 0)
            prev = e
        assert prev == numel


def test_rank_mapping_reference_and_tp_fastest():
    from torsh_b200.parallel import planner
    dp, tp, pp = 1, 4, 2
    # reference rule: rank = dp*(tp*pp) + tp*pp_size + pp (pp fastest)
    assert planner.rank_of(0, 1, 1, dp, tp, pp) == 3
    assert planner.rank_of(0, 1, 1, dp, tp, pp, tp_fastest=True) == 5
    for order in (False, True):
        seen = set()
        for r in range(dp * tp * pp):
            c = planner.coords_of(r, dp, tp, pp, order)
            assert planner.rank_of(*c, dp, tp, pp, order) == r
            seen.add(c)
        assert len(seen) == 8


def test_pipeline_schedules():
    from torsh_b200.parallel import planner
    S, M = 4, 8
    for stage in range(S):
        a = planner.pipeline_schedule("1f1b", stage, S, M)
        assert [m for k, m in a if k == "F"] == list(range(M)) and [m for k, m in a if k == "B"] == list(range(M))
        warm = min(S - stage - 1, M)
        assert all(k == "F" for k, _ in a[:warm]) and planner.pipeline_peak_inflight("1f1b", stage, S, M) == warm + 1
        done_f = set()
        for k, m in a:
            if k == "F":
                done_f.add(m)
            else:
                assert m in done_f
    g = planner.pipeline_schedule("gpipe", 0, S, M)
    assert g[:M] == [("F", i) for i in range(M)] and planner.pipeline_peak_inflight("gpipe", 0, S, M) == M


def test_memory_and_file_store(tmp_path):
    from torsh_b200.parallel.store import FileStore, MemoryStore
    for st in (MemoryStore(), FileStore(tmp_path / "kv")):
        st.set("a", b"1")
        assert st.get("a") == b"1" and st.contains("a") and st.num_keys() == 1
        assert st.add("n", 2) == 2 and st.add("n", 3) == 5
        assert st.compare_and_swap("a", b"0", b"2") is False and st.compare_and_swap("a", b"1", b"2") is True
        st.wait(["a"], 1.0)
        with pytest.raises(Exception):
            st.wait(["zz"], 0.05)
        st.delete("a")
        assert st.get("a") is None


def _ddp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.parallel.ddp import BucketConfig, DistributedDataParallel
        torch.manual_seed(0)
        net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4), torch.nn.Linear(4, 4))
        for p in net[3].parameters():  # unused branch: parameters that never receive a gradient
            pass
        ddp = DistributedDataParallel(net, bucket_config=BucketConfig(max_bucket_size_mb=0.002))
        g = torch.Generator().manual_seed(10 + rank)
        x = torch.randn(8, 16, generator=g)
        y = net[2](net[1](net[0](x))).pow(2).mean()   # skips net[3]
        y.backward()
        ddp.sync_gradients()
        # oracle: average of per-rank gradients computed independently
        grads = []
        for r in range(world):
            torch.manual_seed(0)
            ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4), torch.nn.Linear(4, 4))
            xr = torch.randn(8, 16, generator=torch.Generator().manual_seed(10 + r))
            ref[2](ref[1](ref[0](xr))).pow(2).mean().backward()
            grads.append([p.grad.clone() if p.grad is not None else torch.zeros_like(p) for p in ref.parameters()])
        ok = True
        for i, p in enumerate(net.parameters()):
            exp = sum(gr[i] for gr in grads) / world
            ok &= torch.allclose(p.grad, exp, atol=1e-6)
        st = ddp.get_sync_stats()
        ok &= st["unused_parameters"] == 2 and len(ddp.buckets) >= 2 and st["buckets_reduced"] == len(ddp.buckets)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _ddp_accum_worker(rank, world, port, q):
    """Two micro-batches per step: the first under no_sync(), the second synchronising; the result must be the
    rank-average of the per-rank sums. A second synchronising backward without sync_gradients() must raise."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.parallel.ddp import BucketConfig, DistributedDataParallel
        torch.manual_seed(0)
        net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
        ddp = DistributedDataParallel(net, bucket_config=BucketConfig(max_bucket_size_mb=0.002))
        xs = [torch.randn(8, 16, generator=torch.Generator().manual_seed(100 * r + m)) for r in range(world) for m in range(2)]
        mine = xs[2 * rank:2 * rank + 2]
        with ddp.no_sync():
            ddp(mine[0]).pow(2).mean().backward()
        ddp(mine[1]).pow(2).mean().backward()
        ddp.sync_gradients()
        torch.manual_seed(0)
        ref = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
        for x in xs:
            ref(x).pow(2).mean().backward()
        ok = all(torch.allclose(p.grad, pr.grad / world, atol=1e-6) for p, pr in zip(net.parameters(), ref.parameters()))
        # misuse: two synchronising backward passes in one step
        ddp.zero_grad()
        ddp(mine[0]).pow(2).mean().backward()
        raised = False
        try:
            ddp(mine[1]).pow(2).mean().backward()
        except RuntimeError as e:
            raised = "no_sync" in str(e)
        ddp.sync_gradients()
        q.put((rank, bool(ok and raised)))
    finally:
        dist.destroy_process_group()


def test_ddp_gradient_accumulation_with_no_sync():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ddp_accum_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, True), (1, True)]


def test_ddp_two_gloo_ranks_average_gradients():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ddp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, True), (1, True)]


def _pp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.parallel.pipeline import PipelineConfig, PipelineParallel, ScheduleType, create_pipeline_stages
        torch.manual_seed(0)
        layers = [torch.nn.Linear(8, 8), torch.nn.Tanh(), torch.nn.Linear(8, 8), torch.nn.Tanh(), torch.nn.Linear(8, 4)]
        full = torch.nn.Sequential(*layers)
        x = torch.randn(8, 8, generator=torch.Generator().manual_seed(1))
        y = torch.randn(8, 4, generator=torch.Generator().manual_seed(2))
        # oracle on the un-split model: mean over 4 micro-batches of the micro-batch MSE
        ref = torch.nn.Sequential(*[torch.nn.Linear(8, 8), torch.nn.Tanh(), torch.nn.Linear(8, 8), torch.nn.Tanh(), torch.nn.Linear(8, 4)])
        ref.load_state_dict(full.state_dict())
        loss_ref = sum(torch.nn.functional.mse_loss(ref(a), b) for a, b in zip(x.chunk(4), y.chunk(4))) / 4
        loss_ref.backward()
        ok = True
        for sched, overlap in ((ScheduleType.ONE_F_ONE_B, True), (ScheduleType.GPIPE, True), (ScheduleType.ONE_F_ONE_B, False)):
            full.zero_grad()
            stages = create_pipeline_stages(list(full), world)
            shape = (2, 8)
            pp = PipelineParallel(stages[rank], config=PipelineConfig(num_micro_batches=4, schedule=sched, overlap=overlap),
                                  activation_shape=shape)
            ok &= (len(pp._links) == 2) == overlap
            loss = pp.train_step(x if rank == 0 else None, y if rank == world - 1 else None, torch.nn.functional.mse_loss)
            if rank == world - 1:
                ok &= abs(loss.item() - loss_ref.item()) < 1e-5
            mine = dict(stages[rank].named_parameters())
            refp = dict(ref.named_parameters())
            offset = sum(len(s) for s in stages[:rank])
            for name, p in mine.items():
                idx, leaf = name.split(".")
                ok &= torch.allclose(p.grad, refp[f"{int(idx) + offset}.{leaf}"].grad, atol=1e-5)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_pipeline_two_gloo_ranks_match_unsplit_model():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, True), (1, True)]


def test_interleaved_schedule_covers_every_virtual_stage_in_dependency_order():
    from torsh_b200.parallel import planner
    P, M, V = 4, 8, 2
    per_rank = [planner.pipeline_schedule_interleaved(r, P, M, V) for r in range(P)]
    for r, acts in enumerate(per_rank):
        assert len(acts) == 2 * M * V
        assert sorted((mb, c) for k, mb, c in acts if k == "F") == sorted((mb, c) for mb in range(M) for c in range(V))
        assert sorted((mb, c) for k, mb, c in acts if k == "B") == sorted((mb, c) for mb in range(M) for c in range(V))
        warm = min((P - r - 1) * 2 + (V - 1) * P, M * V)
        assert all(k == "F" for k, _, _ in acts[:warm]) and acts[warm + 1][0] == "B"
        seen = set()
        for k, mb, c in acts:
            if k == "F":
                assert c == 0 or (mb, c - 1) in seen      # a chunk runs after the rank's previous chunk of that micro-batch
                seen.add((mb, c))
            else:
                assert (mb, c) in seen
    # executing the four ranks in lock step never blocks: every receive has its matching send earlier in global order
    pos = [0] * P
    done = set()
    progressed = True
    while progressed:
        progressed = False
        for r in range(P):
            while pos[r] < len(per_rank[r]):
                k, mb, c = per_rank[r][pos[r]]
                vs = c * P + r
                need = ("F", mb, vs - 1) if (k == "F" and vs > 0) else (("B", mb, vs + 1) if (k == "B" and vs < P * V - 1) else None)
                if k == "B" and vs == P * V - 1:
                    need = ("F", mb, vs)
                if need is not None and need not in done:
                    break
                done.add((k, mb, vs))
                pos[r] += 1
                progressed = True
    assert all(pos[r] == len(per_rank[r]) for r in range(P))
    with pytest.raises(ValueError):
        planner.pipeline_schedule_interleaved(0, 4, 6, 2)


def _pp_interleaved_worker(rank, world, port, q):
    """Two ranks, two chunks each (virtual stages 0..3), four micro-batches: loss and every gradient must equal the
    unsplit model's."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.parallel.pipeline import PipelineConfig, PipelineParallel, ScheduleType
        torch.manual_seed(0)
        mk = lambda: [torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Tanh()) for _ in range(3)] + [torch.nn.Sequential(torch.nn.Linear(8, 8))]
        full = mk()
        ref = mk()
        for a, b in zip(ref, full):
            a.load_state_dict(b.state_dict())
        x = torch.randn(8, 8, generator=torch.Generator().manual_seed(1))
        y = torch.randn(8, 8, generator=torch.Generator().manual_seed(2))
        run = lambda t: ref[3](ref[2](ref[1](ref[0](t))))
        loss_ref = sum(torch.nn.functional.mse_loss(run(a), b) for a, b in zip(x.chunk(4), y.chunk(4))) / 4
        loss_ref.backward()
        chunks = [full[rank], full[rank + world]]          # virtual stage = chunk * world + rank
        pp = PipelineParallel(chunks, config=PipelineConfig(num_micro_batches=4, schedule=ScheduleType.INTERLEAVED_ONE_F_ONE_B),
                              activation_shape=(2, 8))
        loss = pp.train_step(x if rank == 0 else None, y if rank == world - 1 else None, torch.nn.functional.mse_loss)
        ok = len(pp._links) == 4
        if rank == world - 1:
            ok &= abs(loss.item() - loss_ref.item()) < 1e-5
        for c, vs in enumerate((rank, rank + world)):
            for p, pr in zip(chunks[c].parameters(), ref[vs].parameters()):
                ok &= torch.allclose(p.grad, pr.grad, atol=1e-5)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_interleaved_pipeline_two_gloo_ranks_match_unsplit_model():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pp_interleaved_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, True), (1, True)]


def test_rpc_parameter_server_scheduler_integrations():
    import torch
    from torsh_b200.parallel import comm_scheduler as cs
    from torsh_b200.parallel import integrations as ig
    from torsh_b200.parallel import parameter_server as ps
    from torsh_b200.parallel import rpc
    from torsh_b200.parallel.store import MemoryStore
    store = MemoryStore()
    rpc.init_rpc("w0", store)
    try:
        store.set("rpc/peer", store.get("rpc/w0"))            # a second name for the same server: calls to it use TCP
        rpc.register_function("add", lambda a, b: a + b)
        rpc.register_function("mk", lambda n: torch.arange(n, dtype=torch.bfloat16))
        assert torch.equal(rpc.rpc_sync("peer", "add", (torch.ones(3), 2)), torch.full((3,), 3.0))
        assert rpc.rpc_async("peer", "add", (1, 2)).result(10) == 3
        ref = rpc.remote("peer", "mk", (4,))
        assert ref.to_here().dtype == torch.bfloat16 and ref.rpc_sync("sum").item() == 6 and rpc.delete_rref(ref)
        try:
            rpc.rpc_sync("peer", "nope")
            raise AssertionError("unregistered function must fail")
        except RuntimeError as e:
            assert "not registered" in str(e)
        srv = ps.ParameterServer(ps.ParameterServerConfig(learning_rate=0.5, max_staleness=0))
        srv.serve()
        m = torch.nn.Linear(2, 1)
        w0 = m.weight.detach().clone()
        cl = ps.ParameterServerClient("peer")
        cl.register_module(m)
        assert cl.sync(m) == 2 and cl.sync(m) == 0
        m(torch.ones(1, 2)).sum().backward()
        cl.push_gradients(m)
        stale = dict(cl.versions)
        assert cl.sync(m) == 2 and torch.allclose(m.weight, w0 - 0.5 * torch.ones(1, 2))
        cl.versions = {k: v for k, v in stale.items()}
        cl.push_gradients(m); cl.push_gradients(m)             # the second push is one version behind: rejected
        assert srv.stats["rejected"] >= 1
    finally:
        rpc.shutdown()
    sch = cs.CommunicationScheduler()
    release = sch.pause()
    futs = [sch.submit(lambda i=i: i, nbytes=10, priority=p, name=n) for i, (p, n) in
            enumerate([(cs.Priority.LOW, "prefetch"), (cs.Priority.HIGH, "bucket"), (cs.Priority.NORMAL, "other")])]
    release(); sch.drain()
    assert sch.order[1:4] == ["bucket", "other", "prefetch"] and [f.result() for f in futs] == [0, 1, 2]
    sch.shutdown()
    plan = ig.from_deepspeed({"zero_optimization": {"stage": 3, "offload_optimizer": {"device": "cpu"}}, "bf16": {"enabled": True},
                              "gradient_clipping": 1.0, "gradient_accumulation_steps": 4})
    assert (plan.strategy, plan.sharding, plan.cpu_offload, plan.param_dtype, plan.grad_accum) == ("zero_offload", "full_shard", True, "bf16", 4)
    assert ig.from_fairscale({"wrapper": "pipe", "balance": [2, 2, 2], "chunks": 8}).pipeline_stages == 3
    assert ig.from_horovod({"fusion_threshold_mb": 32, "compression": "fp16"}).bucket_mb == 32


def test_native_watchdog_and_cpu_compressors():
    import time

    import torch
    from torsh_b200.parallel import compression as cp
    from torsh_b200.parallel.fault_tolerance import NativeWatchdog
    from torsh_b200.parallel.store import MemoryStore
    store = MemoryStore()
    a = NativeWatchdog(store, 0, 3, interval_s=0.02, timeout_s=0.25)
    b = NativeWatchdog(store, 1, 3, interval_s=0.02, timeout_s=0.25)      # rank 2 never joins
    time.sleep(0.5)
    assert a.beats() > 5 and a.failed_ranks() == [2] and b.failed_ranks() == [2]
    b.stop()                                                               # rank 1 exits between steps
    time.sleep(0.5)
    assert a.failed_ranks() == [1, 2]
    a.stop()
    g = torch.randn(5000)
    q, sc = cp.Int8BlockQuantization().compress(g)
    back = cp.Int8BlockQuantization().decompress((q, sc), g.shape)
    assert q.dtype == torch.int8 and sc.numel() == 5 and (back - g).abs().max() <= sc.max() * 0.5 + 1e-6
    payload = cp.PackedSignSGD().compress(g)
    sg = cp.PackedSignSGD().decompress(payload, g.shape)
    assert payload[0].numel() == 157 and torch.equal(sg > 0, g >= 0) and torch.allclose(sg.abs(), g.abs().mean().expand_as(g))
    idx, vals = cp.threshold_sparsify(g, 2.0)
    assert torch.equal(idx.long(), (g.abs() > 2.0).nonzero().flatten()) and torch.equal(vals, g[idx.long()])


def _llama_tp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.models.llama import LlamaConfig, LlamaModel
        from torsh_b200.parallel.tensor_parallel import TensorParallelConfig, TPContext
        cfg = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_layers=2, num_heads=4, max_seq_len=32)
        torch.manual_seed(0)
        ref = LlamaModel(cfg)
        ids = torch.randint(0, cfg.vocab_size, (2, 17), generator=torch.Generator().manual_seed(5))
        inp, tgt = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
        loss_ref = ref(inp, targets=tgt)
        loss_ref.backward()
        E, F = cfg.hidden_size, cfg.intermediate_size
        sl = lambda t, n: t[rank * n // world:(rank + 1) * n // world]
        ok = True
        for vocab_parallel in (False, True):
            tpc = TPContext(dist.group.WORLD, TensorParallelConfig(tp_size=world, fused=False))
            m = LlamaModel(cfg, tp=tpc, vocab_parallel=vocab_parallel)
            with torch.no_grad():
                m.embed.copy_(ref.embed)
                m.norm.weight.copy_(ref.norm.weight)
                for a, b in zip(m.layers, ref.layers):
                    a.input_norm.weight.copy_(b.input_norm.weight)
                    a.post_attn_norm.weight.copy_(b.post_attn_norm.weight)
                    wq = b.qkv.weight
                    a.qkv.weight.copy_(torch.cat([sl(wq[:E], E), sl(wq[E:2 * E], E), sl(wq[2 * E:], E)]))
                    wg = b.gate_up.weight
                    a.gate_up.weight.copy_(torch.cat([sl(wg[:F], F), sl(wg[F:], F)]))
                    a.o.weight.copy_(b.o.weight[:, rank * E // world:(rank + 1) * E // world])
                    a.down.weight.copy_(b.down.weight[:, rank * F // world:(rank + 1) * F // world])
                if vocab_parallel:
                    vp = m.lm_head_tp.weight.shape[0]
                    full = torch.zeros(vp * world, E)
                    full[: cfg.vocab_size] = ref.lm_head[: cfg.vocab_size]
                    m.lm_head_tp.weight.copy_(full[rank * vp:(rank + 1) * vp])
                else:
                    m.lm_head.copy_(ref.lm_head)
            loss = m(inp, targets=tgt)
            loss.backward()
            for p in m.replicated_parameters():
                dist.all_reduce(p.grad)
            ok &= abs(loss.item() - loss_ref.item()) < 1e-5
            ok &= torch.allclose(m.embed.grad, ref.embed.grad, atol=1e-6)
            ok &= torch.allclose(m.norm.weight.grad, ref.norm.weight.grad, atol=1e-6)
            g = ref.layers[0].qkv.weight.grad
            ok &= torch.allclose(m.layers[0].qkv.weight.grad, torch.cat([sl(g[:E], E), sl(g[E:2 * E], E), sl(g[2 * E:], E)]), atol=1e-6)
            ok &= torch.allclose(m.layers[1].down.weight.grad, ref.layers[1].down.weight.grad[:, rank * F // world:(rank + 1) * F // world], atol=1e-6)
            if vocab_parallel:
                hg = torch.zeros(vp * world, E)
                hg[: cfg.vocab_size] = ref.lm_head.grad[: cfg.vocab_size]
                ok &= torch.allclose(m.lm_head_tp.weight.grad, hg[rank * vp:(rank + 1) * vp], atol=1e-6)
                logits = m(inp)
                ok &= torch.allclose(logits, ref(inp), atol=1e-5)
            else:
                ok &= torch.allclose(m.lm_head.grad, ref.lm_head.grad, atol=1e-6)
        # ParallelAttention: heads split over the ranks, token-sharded input and output
        from torsh_b200.parallel.tensor_parallel import ParallelAttention
        Hh, B, S = 4, 2, 8
        torch.manual_seed(1)
        wqkv, wo = torch.randn(3 * E, E) * 0.1, torch.randn(E, E) * 0.1
        x = torch.randn(B * S, E)
        qf, kf, vf = ((x @ wqkv[i * E:(i + 1) * E].t()).view(B, S, Hh, E // Hh).transpose(1, 2) for i in range(3))
        ref_out = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True).transpose(1, 2).reshape(B * S, E) @ wo.t()
        pa = ParallelAttention(E, Hh, tp=TPContext(dist.group.WORLD, TensorParallelConfig(tp_size=world, fused=False)))
        with torch.no_grad():
            pa.qkv.weight.copy_(torch.cat([sl(wqkv[:E], E), sl(wqkv[E:2 * E], E), sl(wqkv[2 * E:], E)]))
            pa.out.weight.copy_(wo[:, rank * E // world:(rank + 1) * E // world])
        rows = B * S // world
        got = pa(x[rank * rows:(rank + 1) * rows], B, S)
        ok &= torch.allclose(got, ref_out[rank * rows:(rank + 1) * rows], atol=1e-5)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_llama_tensor_parallel_heads_match_single_process_model():
    """Dense (replicated) and vocabulary-parallel LM heads under 2-way tensor + sequence parallelism give the loss and
    the gradients of the unsplit model."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_llama_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, True), (1, True)]


def _coll_variants_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.parallel import collectives as C
        ok = True
        base = torch.arange(10, dtype=torch.float32)
        total = sum(base * (r + 1) for r in range(world))
        t = base * (rank + 1)
        ok &= torch.allclose(C.hierarchical_all_reduce(t.clone(), 2), total)
        ok &= torch.allclose(C.hierarchical_all_reduce(t.clone(), 2, C.ReduceOp.MEAN), total / world)
        ok &= torch.allclose(C.ring_all_reduce(t.clone()), total)
        ok &= torch.allclose(C.pipelined_all_reduce(t.clone(), chunk_bytes=12), total)
        ts = [t.clone() * k for k in (1, 2, 3)]
        C.double_buffered_all_reduce(ts)
        ok &= all(torch.allclose(x, total * k) for x, k in zip(ts, (1, 2, 3)))
        for src in (0, 3):
            b = torch.full((5,), float(rank))
            C.tree_broadcast(b, src)
            ok &= bool((b == src).all())
        gm = C.GroupManager.for_group()
        std = gm.create_standard_groups(2)
        ok &= std["nodes"] == 2 and std["node"] == rank // 2 and gm.groups["leaders/2"].ranks == [0, 2]
        ok &= gm.groups["node1/2"].local_rank(3) == 1 and gm.groups["node1/2"].global_rank(0) == 2
        batch = C.NcclBatch()
        x, y = t.clone(), torch.full((3,), float(rank))
        got = torch.empty(4)
        batch.all_reduce(x).broadcast(y, 1).send(torch.full((4,), float(rank)), (rank + 1) % world).recv(got, (rank - 1) % world)
        ok &= len(batch) == 4 and batch.execute() == 4
        ok &= torch.allclose(x, total) and bool((y == 1).all()) and bool((got == (rank - 1) % world).all())
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_collective_variants_four_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_coll_variants_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(r, True) for r in range(4)]


def _cp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.parallel.context_parallel import ring_attention, ulysses_attention
        B, S, H, D = 2, 24, 4, 8
        g = torch.Generator().manual_seed(3)
        full = [torch.randn(B, S, H, D, generator=g, dtype=torch.float64).requires_grad_() for _ in range(3)]
        dy = torch.randn(B, S, H, D, generator=g, dtype=torch.float64)
        n = S // world
        sl = slice(rank * n, (rank + 1) * n)
        ok = True
        for causal in (False, True):
            qf, kf, vf = (t.transpose(1, 2) for t in full)
            ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=causal).transpose(1, 2)
            gref = torch.autograd.grad(ref, full, dy)
            for fn in (ulysses_attention, ring_attention):
                loc = [t.detach()[:, sl].clone().requires_grad_() for t in full]
                out = fn(*loc, causal=causal)
                ok &= torch.allclose(out, ref[:, sl].to(out.dtype), atol=1e-5)
                gl = torch.autograd.grad(out, loc, dy[:, sl].to(out.dtype))
                for a, b in zip(gl, gref):
                    ok &= torch.allclose(a, b[:, sl].to(a.dtype), atol=1e-5)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_context_parallel_attention_matches_full_attention(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_cp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(r, True) for r in range(world)]


def _zero1_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.optim.distributed import ZeroRedundancyOptimizer
        torch.manual_seed(0)
        make = lambda: torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
        model, ref = make(), make()
        ref.load_state_dict(model.state_dict())
        opt = ZeroRedundancyOptimizer(model.parameters(), torch.optim.Adam, lr=1e-2)
        ref_opt = torch.optim.Adam(ref.parameters(), lr=1e-2)
        for step in range(4):
            xs = [torch.randn(6, 8, generator=torch.Generator().manual_seed(100 * step + r)) for r in range(world)]
            opt.zero_grad()
            model(xs[rank]).pow(2).mean().backward()
            for p in model.parameters():                      # what DDP would have done
                dist.all_reduce(p.grad)
                p.grad.div_(world)
            opt.step()
            ref_opt.zero_grad()
            (sum(ref(x).pow(2).mean() for x in xs) / world).backward()
            ref_opt.step()
        ok = all(torch.allclose(a, b, atol=1e-6) for a, b in zip(model.parameters(), ref.parameters()))
        total_state = sum(2 * p.numel() * 4 for p in model.parameters())
        ok &= 0 < opt.state_bytes() < total_state                       # this rank holds only its share of the moments
        ok &= sorted(opt.consolidate_state_dict()) == list(range(len(list(model.parameters()))))
        ok &= sum(opt.partition_sizes) == sum(p.numel() for p in model.parameters())
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_zero_redundancy_optimizer_matches_plain_adam():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_zero1_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, True), (1, True)]


def _zero3_worker(rank, world, port, q):
    """ZeRO-3 + CPU offload on two gloo ranks must follow a single-process AdamW run on the global batch."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.parallel.zero_offload import (AutoMemoryStrategy, CpuCompressionMethod, Zero3CpuOffloadManager,
                                                      Zero3OffloadConfig)

        class Net(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.inp = torch.nn.Linear(6, 16)
                self.h = torch.nn.ModuleList([torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.Tanh()) for _ in range(5)])
                self.out = torch.nn.Linear(16, 3)

            def forward(self, x):
                x = self.inp(x)
                for l in self.h:
                    x = l(x)
                return self.out(x)

        xs = torch.randn(8, 6, generator=torch.Generator().manual_seed(5))
        ys = torch.randn(8, 3, generator=torch.Generator().manual_seed(6))
        torch.manual_seed(0)
        ref = Net()
        opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
        ref_losses = []
        for _ in range(4):
            loss = torch.nn.functional.mse_loss(ref(xs), ys)
            opt.zero_grad(); loss.backward(); opt.step()
            ref_losses.append(loss.item())
        ok = True
        layer_bytes = 16 * 16 * 4 + 16 * 4
        for strategy, budget_layers, prefetch in ((AutoMemoryStrategy.EXTREME, 2, 1), (AutoMemoryStrategy.CONSERVATIVE, 8, 16)):
            torch.manual_seed(0)
            net = Net()
            cfg = Zero3OffloadConfig(gpu_param_budget_gb=budget_layers * (layer_bytes + 64) / 2 ** 30, prefetch_buffer_size=prefetch,
                                     auto_memory_management=strategy)
            mgr = Zero3CpuOffloadManager(net, list(net.h), config=cfg, lr=1e-2, weight_decay=0.01)
            assert all(not pt.resident for pt in mgr.partitions)          # parameters start offloaded
            mine = slice(rank * 4, rank * 4 + 4)
            losses = []
            for _ in range(4):
                loss = torch.nn.functional.mse_loss(net(xs[mine]), ys[mine])
                loss.backward()
                mgr.step()
                l = loss.detach().clone(); dist.all_reduce(l)
                losses.append(l.item() / world)
            ok &= all(abs(a - b) < 1e-5 for a, b in zip(losses, ref_losses))
            sd = mgr.gather_state_dict()
            ok &= all(torch.allclose(sd[n], p.detach(), atol=1e-5) for n, p in ref.named_parameters())
            st = mgr.stats.as_dict()
            ok &= st["h2d_bytes"] > 0 and st["d2h_bytes"] > 0 and st["steps"] == 4
            if strategy is AutoMemoryStrategy.EXTREME:
                ok &= st["releases"] >= 5 * 2 * 4 and mgr.gpu_param_bytes() == 0     # every layer offloaded after every use
            ok &= mgr.memory_report()["host_state_bytes"] > 0
        # lossy host compression: bf16 transfer copies, fp32 masters -> still trains, parameters within bf16 rounding
        torch.manual_seed(0)
        net = Net()
        mgr = Zero3CpuOffloadManager(net, list(net.h), config=Zero3OffloadConfig(cpu_compression=CpuCompressionMethod.BF16), lr=1e-2, weight_decay=0.01)
        first = last = None
        for i in range(4):
            loss = torch.nn.functional.mse_loss(net(xs[rank * 4:rank * 4 + 4]), ys[rank * 4:rank * 4 + 4])
            loss.backward(); mgr.step()
            l = loss.detach().clone(); dist.all_reduce(l)
            first = l.item() / world if first is None else first
            last = l.item() / world
        ok &= last < first and abs(last - ref_losses[-1]) < 5e-3
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_zero3_cpu_offload_two_gloo_ranks_match_single_process():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_zero3_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, True), (1, True)]


def test_zero3_config_and_rank_mapping():
    from torsh_b200.parallel.zero_offload import AutoMemoryStrategy, CpuCompressionMethod, Zero3OffloadConfig, Zero3RankMapping
    c = Zero3OffloadConfig()
    assert (c.offload_params, c.offload_grads, c.offload_optimizer_states, c.cpu_memory_budget_gb, c.gpu_param_budget_gb,
            c.prefetch_buffer_size, c.async_prefetch, c.overlap_computation, c.pin_memory) == (True, True, True, 32.0, 2.0, 16, True, True, True)
    assert c.auto_memory_management is AutoMemoryStrategy.AGGRESSIVE and AutoMemoryStrategy.AGGRESSIVE.pressure_threshold() == 0.6
    assert CpuCompressionMethod.BF16.ratio() == 0.5 and CpuCompressionMethod.BF16.is_lossy() and not CpuCompressionMethod.LOSSLESS.is_lossy()
    assert Zero3OffloadConfig(cpu_compression=CpuCompressionMethod.FP16).effective_cpu_memory_budget() == 64 * 2 ** 30
    with pytest.raises(ValueError):
        Zero3OffloadConfig(cpu_compression=CpuCompressionMethod.INT8).validate()
    m = Zero3RankMapping(1, 4)
    assert m.owned_partitions(10) == [1, 5, 9] and m.owned_partition_count(10) == 3 and m.get_parameter_owner(6) == 2
    assert m.global_to_local_partition(5) == 1 and m.global_to_local_partition(6) is None and m.local_to_global_partition(2) == 9
    assert m.communication_group([0, 4, 5]) == [0, 1]


def test_moe_load_balancer_strategies_and_hierarchical_gate():
    from torsh_b200.parallel import expert_parallel as ep
    cfg = ep.ExpertParallelismConfig(num_experts=8, rebalancing_threshold=0.3)
    lb = ep.LoadBalancer(cfg)
    skew = [400, 300, 100, 50, 50, 40, 30, 30]               # two hot experts
    for _ in range(9):
        lb.update_expert_load(skew, sum(skew))
    assert lb.rebalancing_count == 0                          # never within the first ten updates
    for _ in range(3):
        lb.update_expert_load(skew, sum(skew))
    assert lb.rebalancing_count == 1 and lb.last_strategy is ep.RebalancingStrategy.EXPERT_MIGRATION
    assert [m.source_expert_id for m in lb.pending_migrations] == [0, 1] and [m.target_expert_id for m in lb.pending_migrations] == [3, 4]
    assert lb.pending_migrations[0].priority >= lb.pending_migrations[1].priority
    before = lb.expert_loads[0]
    m = lb.process_pending_migrations()
    assert m.migration_type is ep.MigrationType.LOAD_REDISTRIBUTION and lb.expert_loads[0] == pytest.approx(before * 0.7)
    # routing adjustment: under 0.8 of the mean load -> x1.2, above 1.2 -> x0.8, then decay towards 1
    lb.trigger_rebalancing(ep.RebalancingStrategy.ROUTING_ADJUSTMENT)
    assert lb.get_routing_adjustment(1) == 0.8 and lb.get_routing_adjustment(7) == 1.2
    lb.decay_routing_adjustments()
    assert lb.get_routing_adjustment(1) == pytest.approx(0.8 * 0.95 + 0.05) and lb.get_routing_adjustment(99) == 1.0
    lb.trigger_rebalancing(ep.RebalancingStrategy.CAPACITY_REALLOCATION)
    assert lb.expert_capacities[1] == 1.25 and lb.expert_capacities[7] == 0.75
    st = lb.get_stats()
    assert st.rebalancing_count == 3 and not st.is_well_balanced() and st.load_cv() > 0.5
    assert ep.RebalancingStrategy.EXPERT_MIGRATION.disruption_level() == 0.7 and not ep.RebalancingStrategy.EXPERT_MIGRATION.supports_rollback()
    assert ep.MigrationType.DEVICE_MIGRATION.requires_parameter_copy() and ep.MigrationType.EXPERT_CONSOLIDATION.complexity() == 4
    # hierarchical gate: ceil(sqrt(E)) groups, probabilities of a token sum to one, only real experts get mass
    torch.manual_seed(0)
    gate = ep.GateNetwork(16, 10)
    assert gate.num_groups == 4 and gate.experts_per_group == 3 and gate.get_hierarchy_stats()["total_capacity"] == 12
    x = torch.randn(5, 7, 16)
    pr = gate(x)
    assert pr.shape == (5, 7, 10) and torch.allclose(pr.sum(-1), torch.ones(5, 7), atol=1e-5) and (pr >= 0).all()
    gp = torch.softmax(x.reshape(-1, 16) @ gate.group_router, -1)
    el = x.reshape(-1, 16) @ gate.expert_routers[1]
    ref = gp[:, 1:2] * torch.softmax(el, -1)                  # group 1 holds experts 3, 4, 5
    assert torch.allclose(pr.reshape(-1, 10)[:, 3:6], ref, atol=1e-6)
    # a router with the hierarchical gate and the balancer routes and trains
    layer = ep.MoELayer(16, 32, ep.ExpertParallelismConfig(num_experts=4, top_k=2, hierarchical_gate=True, enable_load_balancing=True))
    y, aux = layer(torch.randn(12, 16))
    (y.sum() + aux).backward()
    assert layer.router.gate_network.group_router.grad is not None and layer.router.load_balancer.load_history


def _moe_migration_worker(rank, world, port, q):
    """Swapping the homes of two experts that live on different ranks must leave the layer's function unchanged."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torsh_b200.parallel import expert_parallel as ep
        torch.manual_seed(10 + rank)                           # every rank owns different experts
        layer = ep.MoELayer(16, 32, ep.ExpertParallelismConfig(num_experts=4, top_k=2, drop_tokens=False))
        for prm in layer.router.parameters():
            dist.broadcast(prm.data, 0)                        # the gate is replicated
        x = torch.randn(12, 16, generator=torch.Generator().manual_seed(rank))
        y0, _ = layer(x)
        w1_before = layer.w1.data.clone()
        m1 = torch.arange(layer.e_local, dtype=torch.float32).add(10 * rank).view(-1, 1).repeat(1, 3)   # stands for an optimizer moment
        layer.swap_experts(0, 3, extra_stacks=[m1])            # expert 0 lives on rank 0, expert 3 on rank 1
        ok = layer.expert_sharding_map()[0] == (1, 1) and layer.expert_sharding_map()[3] == (0, 0)
        ok &= not torch.equal(layer.w1.data, w1_before)
        ok &= m1[0 if rank == 0 else 1, 0].item() == (11.0 if rank == 0 else 0.0)
        y1, _ = layer(x)
        ok &= torch.allclose(y0, y1, atol=1e-6)
        layer.swap_experts(0, 1)                               # now both on rank 1 -> local swap there
        y2, _ = layer(x)
        ok &= torch.allclose(y0, y2, atol=1e-6)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_moe_expert_migration_keeps_the_function():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_moe_migration_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(30)
    assert sorted(res) == [(0, True), (1, True)]
