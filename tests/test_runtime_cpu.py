"""Caching-pool logic on the host-memory instance, and the domain libraries that need no GPU."""
import math

import pytest
import torch


def test_pool_rounding_reuse_split_merge():
    from torsh_b200.core.runtime import HostPool
    p = HostPool()
    assert p.round_size(1) == 512 and p.round_size(513) == 1024 and p.round_size((1 << 20) + 1) == 2 << 20 and p.round_size((2 << 20) + 1) == 4 << 20
    a = p.alloc(1000)
    b = p.alloc(3000)
    s = p.stats()
    assert s["raw_allocs"] == 1 and s["segments"] == 1 and s["reserved_bytes"] == 2 << 20      # both from one 2 MiB segment
    assert s["allocated_bytes"] == 1024 + 3072 and p.size_of(a) == 1024
    assert p.free(a) and not p.free(a)                                                          # double free refused
    c = p.alloc(900)                                                                            # reuses a's block
    assert c == a and p.stats()["cache_hits"] >= 1
    # another stream never reuses this stream's cached blocks
    p.free(c)
    d = p.alloc(900, stream=7)
    assert d != a and p.stats()["segments"] == 2
    p.free(b); p.free(d)
    assert p.stats()["allocated_bytes"] == 0 and p.stats()["merges"] >= 2
    assert p.release_cached() == 4 << 20 and p.stats()["reserved_bytes"] == 0 and p.stats()["segments"] == 0
    p.close()


def test_pool_large_blocks_limit_and_oom_retry():
    from torsh_b200.core.runtime import HostPool
    MB = 1 << 20
    p = HostPool(raw_budget=64 * MB)
    big = p.alloc(30 * MB)
    assert p.size_of(big) == 30 * MB
    p.free(big)
    small_large = p.alloc(4 * MB)                      # best fit takes the cached 30 MiB block and splits it
    st = p.stats()
    assert small_large == big and st["splits"] >= 1 and st["raw_allocs"] == 1
    other = p.alloc(20 * MB)                           # served by the 26 MiB remainder
    assert p.stats()["raw_allocs"] == 1
    p.free(small_large); p.free(other)
    assert p.fragmentation() == 0.0
    # the raw allocator has 34 MiB left: a 40 MiB request fails once, the cache is released, the retry succeeds
    x = p.alloc(40 * MB)
    st = p.stats()
    assert x and st["oom_retries"] == 1 and st["raw_frees"] == 1
    assert p.alloc(40 * MB) is None                    # genuinely out of budget
    assert p.pressure(64 * MB) == "low" and p.pressure(44 * MB) == "high"
    p.free(x)
    q = HostPool(limit=8 * MB)
    y = q.alloc(6 * MB)
    assert y and q.alloc(6 * MB) is None
    q.free(y)
    assert q.alloc(8 * MB)                             # cached 6 MiB segment is released to stay under the limit
    p.close(); q.close()


def test_cluster_and_sparse_and_graph():
    from torsh_b200 import cluster, graph as G, sparse as sp
    torch.manual_seed(0)
    x = torch.cat([torch.randn(40, 2) + 6, torch.randn(40, 2) - 6])
    true = torch.cat([torch.zeros(40), torch.ones(40)]).long()
    for lab in (cluster.kmeans(x, 2)[0], cluster.dbscan(x, 2.5, 3), cluster.GaussianMixture(2).fit(x).predict(x),
                cluster.spectral_clustering(x, 2, 0.05), cluster.agglomerative(x[::4], 2)):
        assert cluster.adjusted_rand_index(lab, true[:: len(true) // len(lab)]) > 0.99
    assert cluster.silhouette_score(x, true) > 0.8
    d = torch.randn(8, 12) * (torch.rand(8, 12) > 0.6)
    b = torch.randn(12, 5)
    coo = sp.CooTensor.from_dense(d)
    for t in (coo, coo.to_csr(), coo.to_csc(), sp.BsrTensor.from_dense(d, 4), sp.EllTensor.from_dense(d)):
        assert torch.allclose(t.to_dense(), d) and torch.allclose(t.matmul(b), d @ b, atol=1e-5)
    assert torch.allclose(sp.DiaTensor.from_dense(d).to_dense(), d)
    lin = torch.nn.Linear(12, 8)
    sl = sp.SparseLinear(lin, 0.5)
    assert sl(torch.randn(3, 12)).shape == (3, 8) and abs(sl.values.numel() - 48) <= 1
    data = G.stochastic_block_model()
    conv = G.GCNConv(16, 4)
    A = torch.zeros(80, 80); A[data.edge_index[1], data.edge_index[0]] = 1; A += torch.eye(80)
    dg = A.sum(1)
    assert torch.allclose(conv(data.x, data.edge_index), (dg.rsqrt()[:, None] * A * dg.rsqrt()[None]) @ conv.lin(data.x) + conv.bias, atol=1e-5)
    for layer in (G.SAGEConv(16, 8), G.GATConv(16, 8, heads=2), G.GINConv(torch.nn.Linear(16, 8))):
        out = layer(data.x, data.edge_index)
        out.sum().backward()
        assert out.shape[0] == 80 and torch.isfinite(out).all()
    batch = G.GraphData.collate([data, data])
    assert G.global_mean_pool(batch.x, batch.batch).shape == (2, 16)


def test_signal_series_linalg_quantization():
    from torsh_b200 import linalg, quantization as Q, series as S, signal
    torch.manual_seed(0)
    s = torch.sin(torch.arange(4096) * 0.05)
    assert torch.allclose(signal.istft(signal.stft(s), length=4096), s, atol=1e-4)
    a, d = signal.haar_dwt(s)
    assert torch.allclose(signal.haar_idwt(a, d), s, atol=1e-6)
    assert signal.mel_filterbank(40, 512, 16000).shape == (40, 257)
    lp = signal.lfilter_fir(torch.sin(torch.arange(2048.) * 3.0), signal.firwin(63, 0.1))
    assert lp[100:].abs().max() < 0.05                     # a tone far above the cut-off is removed
    t = torch.arange(240.)
    x = 0.05 * t + torch.sin(2 * math.pi * t / 12)
    dec = S.seasonal_decompose(x, 12)
    assert dec.residual[12:-12].abs().max() < 0.05
    assert (S.ssa(x, 24, 3) - x).abs().mean() < 0.05
    coef = S.fit_ar(x, 13)
    assert (S.forecast_ar(x, coef, 3) - (0.05 * torch.arange(240., 243) + torch.sin(2 * math.pi * torch.arange(240., 243) / 12))).abs().max() < 0.05
    kf = S.KalmanFilter(torch.tensor([[1., 1.], [0., 1.]]), torch.tensor([[1., 0.]]), 1e-4 * torch.eye(2), torch.tensor([[0.1]]))
    xs = kf.filter((0.5 * t[:60])[:, None])
    assert abs(xs[-1, 1].item() - 0.5) < 0.02 and kf.smooth().shape == (60, 2)
    A = torch.randn(20, 20); A = A @ A.T + torch.eye(20)
    assert torch.allclose(linalg.matrix_sqrt(A) @ linalg.matrix_sqrt(A), A, atol=1e-3)
    assert torch.allclose(linalg.conjugate_gradient(A, torch.ones(20), 200), torch.linalg.solve(A, torch.ones(20)), atol=1e-3)
    low = torch.randn(50, 6) @ torch.randn(6, 40)
    u, sv, vh = linalg.randomized_svd(low, 6)
    assert torch.allclose((u * sv) @ vh, low, atol=1e-3)
    w = torch.randn(64, 256)
    q, qp = Q.quantize_per_channel(w)
    assert Q.sqnr_db(w, Q.dequantize(q, qp)) > 38
    q4, sc = Q.quantize_groupwise(w, 128, 4)
    assert q4.shape == (64, 128) and Q.sqnr_db(w, Q.dequantize_groupwise(q4, sc, 128, 4)) > 15
    m = torch.nn.Sequential(torch.nn.Linear(256, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8))
    xi = torch.randn(4, 256)
    ref = m(xi)
    import copy
    assert Q.sqnr_db(ref, Q.quantize_model(copy.deepcopy(m))(xi)) > 35
    qat = Q.prepare_qat(copy.deepcopy(m))
    qat(xi).sum().backward()


def test_fx_jit_hub_package_tensorboard_cli(tmp_path):
    import torch.nn.functional as F
    from torsh_b200 import cli, fx, hub, jit
    from torsh_b200.utils import tensorboard as tbw

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w, self.b, self.g = torch.nn.Parameter(torch.randn(32, 16)), torch.nn.Parameter(torch.zeros(32)), torch.nn.Parameter(torch.ones(32))

        def forward(self, x, r):
            h = F.gelu(F.linear(x, self.w, self.b), approximate="tanh")
            a, b = torch.relu(x), torch.relu(x)
            _dead = a * 3
            return F.layer_norm(h + r, (32,), self.g, None, 1e-5) + (a + b).sum()
    m = M()
    x, r = torch.randn(4, 16), torch.randn(4, 32)
    gm = fx.symbolic_trace(m)
    stats = fx.PassManager.default().run(gm)
    assert stats["cse"] == 1 and stats["fusion"] == 2 and stats["dce"] >= 1
    assert torch.allclose(gm(x, r), m(x, r), atol=1e-5)
    assert "digraph" in fx.to_dot(gm) and len(fx.partition_by_cost(gm, 2)) == 2
    seq = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.GELU(approximate="tanh"), torch.nn.Linear(8, 2))
    c = jit.script(seq)
    assert c.stats["fusion"] == 1 and torch.allclose(c(torch.ones(3, 8)), seq(torch.ones(3, 8)), atol=1e-6)
    # hub + package
    f = tmp_path / "w.bin"; f.write_bytes(b"abc" * 100)
    reg = hub.LocalHub(tmp_path / "hub")
    reg.publish("org/model", f)
    assert reg.list() == ["org/model@v1"] and reg.fetch("org/model").read_bytes() == f.read_bytes()
    with pytest.raises(ConnectionError):
        reg.fetch("someone/remote")
    pkg = hub.Package("demo", "1.2.0", {"torsh": ">=0.1.0"})
    pkg.add_source("demo.mod", "VALUE = 41 + 1\n"); pkg.add_bytes("data.bin", b"\x00\x01")
    pkg.save(tmp_path / "demo.tpkg", key=b"k")
    back = hub.Package.load(tmp_path / "demo.tpkg", key=b"k")
    assert back.import_module("demo.mod").VALUE == 42 and back.files["data.bin"] == b"\x00\x01"
    with pytest.raises(PermissionError):
        hub.Package.load(tmp_path / "demo.tpkg", key=b"wrong")
    assert hub.resolve_dependencies({"a": "^1.2.0", "b": ">=0.3.0"}, {"a": ["1.1.0", "1.4.2", "2.0.0"], "b": ["0.2.0", "0.9.1"]}) == {"a": "1.4.2", "b": "0.9.1"}
    # tensorboard
    with tbw.SummaryWriter(str(tmp_path / "tb")) as w:
        for i in range(3):
            w.add_scalar("loss", 1.0 / (i + 1), i)
        w.add_histogram("w", torch.randn(50), 1); w.add_text("note", "hi")
    ev = tbw.read_events(w.path)
    assert [e[0] for e in ev] == [0, 1, 2] and abs(ev[1][2] - 0.5) < 1e-7 and tbw.crc32c(b"123456789") == 0xE3069283
    # CLI
    out = tmp_path / "run"
    assert cli.main(["train", "start", "--model", "gpt2-tiny", "--steps", "3", "--seq", "16", "--batch-size", "2", "--output", str(out), "--device", "cpu"]) == 0
    assert cli.main(["train", "resume", "--model", "gpt2-tiny", "--steps", "1", "--seq", "16", "--batch-size", "2", "--output", str(out), "--device", "cpu"]) == 0
    import json
    assert json.loads((out / "run.json").read_text())["step"] == 4
    assert cli.main(["model", "create", "--name", "gpt2-tiny", "-o", str(tmp_path / "m.trsm")]) == 0
    assert cli.main(["model", "convert", str(tmp_path / "m.trsm"), "-o", str(tmp_path / "m.safetensors")]) == 0
    assert cli.main(["model", "validate", str(tmp_path / "m.safetensors")]) == 0
    assert cli.main(["info"]) == 0 and cli.main(["init", str(tmp_path / "proj")]) == 0


def test_operation_coordinator_orders_streams_and_rejects_cycles():
    import time
    import pytest
    from torsh_b200.core.event_coordination import (AsyncEventWaiter, CrossStreamBarrier, DependencyCycleError, HostEvent,
                                                    OperationCoordinator)
    co = OperationCoordinator(event_factory=HostEvent)
    co.add_operation("load", "copy")
    co.add_operation("fwd", "compute", ["load"])
    co.add_operation("bwd", "compute", ["fwd"])
    co.add_operation("allreduce", "comm", ["bwd"])
    co.add_operation("step", "compute", ["allreduce", "bwd"])
    assert co.order() == ["load", "fwd", "bwd", "allreduce", "step"] and co.detect_deadlocks() == []
    trace = []
    co.run({n: (lambda n=n: trace.append(n)) for n in co.ops})
    assert trace == co.order()
    assert co.stats == {"events_recorded": 5, "cross_stream_waits": 3, "same_stream_skipped": 2}
    assert co.ops["bwd"].event.waited_by == ["comm"] and co.ops["allreduce"].event.waited_by == ["compute"]
    with pytest.raises(DependencyCycleError):
        co.add_dependency("load", "step")
    with pytest.raises(KeyError):
        co.add_operation("x", "compute", ["missing"])
    fresh = OperationCoordinator(event_factory=HostEvent)
    fresh.add_operation("a", "s0"); fresh.add_operation("b", "s1", ["a"])
    with pytest.raises(RuntimeError):
        fresh.issue("b")
    bar = CrossStreamBarrier(["s0", "s1", "s2"], event_factory=HostEvent)
    evs = bar.arrive_and_wait()
    assert [sorted(e.waited_by) for e in evs] == [["s1", "s2"], ["s0", "s2"], ["s0", "s1"]]
    w = AsyncEventWaiter()
    done, late = HostEvent(), HostEvent()
    hits = []
    w.on_complete(done, lambda: hits.append("done"))
    w.on_complete(late, lambda: hits.append("late"), timeout_s=0.02, on_timeout=lambda: hits.append("timeout"))
    done.record()
    time.sleep(0.2)
    w.shutdown()
    assert sorted(hits) == ["done", "timeout"] and (w.completed, w.timed_out, w.pending()) == (1, 1, 0)


def test_backend_capabilities_hints_and_autotuner(tmp_path):
    import json
    from torsh_b200.core import backend as B
    caps = B.capabilities()
    assert caps.sm_count == 148 and "tcgen05" in caps.features and "f16" in caps.tensor_cores
    k = B.TENSOR_CORE_KINDS["f16"]
    assert k.accumulator == "f32" and 128 in k.m and k.n_max == 256 and k.k == 16
    peaks = tmp_path / "peaks.json"
    peaks.write_text(json.dumps({"hbm_gbs": 6553.9, "bf16_tflops": 1633.7}))
    h = B.performance_hints(str(peaks))
    assert (h.hbm_gbs, h.bf16_tflops, h.grid_multiple) == (6553.9, 1633.7, 148)
    cfg = B.CudaBackendBuilder().device(0).allow_tf32(False).stream_pool_size(8).build()
    assert (cfg.allow_tf32, cfg.stream_pool_size) == (False, 8)
    cost = {"bn128": 3.0, "bn256": 1.0}
    calls = []
    tuner = B.Autotuner(str(tmp_path / "tune.json"), timer=lambda fn: fn())
    cands = {n: (lambda n=n: calls.append(n) or cost[n]) for n in cost}
    assert tuner.select("gemm/8192x1024x4096", cands) == "bn256" and sorted(calls) == ["bn128", "bn256"]
    assert tuner.select("gemm/8192x1024x4096", cands) == "bn256" and len(calls) == 2          # cached
    again = B.Autotuner(str(tmp_path / "tune.json"), timer=lambda fn: 1 / 0)
    assert again.select("gemm/8192x1024x4096", cands) == "bn256"                               # loaded from the file


def test_native_token_loader_is_deterministic_and_in_order(tmp_path):
    import numpy as np
    import torch
    from torsh_b200.data import NativeTokenLoader
    tokens = np.arange(5000, dtype=np.uint16)
    path = tmp_path / "tokens.bin"
    tokens.tofile(path)

    def take(n, **kw):
        ld = NativeTokenLoader(str(path), batch=4, seq=16, slots=3, workers=3, seed=7, pin=False, **kw)
        out = []
        for _ in range(n):
            x, y = next(ld)
            out.append((ld.batch_number, x.clone(), y.clone()))
        count = ld.num_tokens
        ld.close()
        return out, count
    a, count = take(10)
    b, _ = take(10)
    other, _ = take(3, rank=1)
    assert count == 5000 and [n for n, _, _ in a] == list(range(10))
    for (_, xa, ya), (_, xb, yb) in zip(a, b):
        assert torch.equal(xa, xb) and torch.equal(ya, yb)
    x0, y0 = a[0][1], a[0][2]
    assert x0.shape == (4, 16) and torch.equal(y0[:, :-1], x0[:, 1:]) and torch.equal(y0, x0 + 1)     # windows of arange
    assert not torch.equal(other[0][1], x0)                                                           # ranks draw different windows
    with pytest.raises(OSError):
        NativeTokenLoader(str(tmp_path / "missing.bin"), batch=1, seq=4, pin=False)


def test_multi_stream_orchestrator_plans_and_issues_with_few_events():
    """Critical-path list scheduling beats round-robin on a fork-join graph with one long branch, same-stream edges
    need no event, and issue order respects every dependency."""
    from torsh_b200.core.stream_orchestrator import MultiStreamOrchestrator

    class FakeStream:
        def __init__(self, name): self.name = name

    log = []

    def build(policy):
        o = MultiStreamOrchestrator([FakeStream("s0"), FakeStream("s1")], policy=policy)
        o.add("load", lambda: log.append("load"), cost=1)
        o.add("long1", lambda: log.append("long1"), cost=6, deps=("load",))
        o.add("long2", lambda: log.append("long2"), cost=6, deps=("long1",))
        for i in range(4):
            o.add(f"short{i}", lambda i=i: log.append(f"short{i}"), cost=2, deps=("load",))
        o.add("join", lambda: log.append("join"), cost=1, deps=("long2", "short0", "short1", "short2", "short3"))
        return o
    cp, rr, ll = build("critical_path").plan(), build("round_robin").plan(), build("least_loaded").plan()
    assert cp.makespan == 14.0                      # load + the two long tasks + join: the critical path itself
    assert rr.makespan > cp.makespan and ll.makespan >= cp.makespan
    assert cp.assignment["long1"] == cp.assignment["long2"] == cp.assignment["load"]     # the chain stays on one stream
    assert cp.order.index("long1") < cp.order.index("short0")
    o = build("critical_path")
    log.clear()
    res = o.run()
    assert set(res) == set(o.tasks) and log[0] == "load" and log[-1] == "join" and log.index("long1") < log.index("long2")
    st = o.coordinator.stats
    assert st["events_recorded"] == 8 and st["cross_stream_waits"] == cp.cross_stream_edges
    assert st["same_stream_skipped"] + st["cross_stream_waits"] == 1 + 1 + 4 + 5
    o.join()
    with pytest.raises(KeyError):
        build("round_robin").add("x", deps=("nope",))
    with pytest.raises(ValueError):
        MultiStreamOrchestrator([FakeStream("a")], policy="magic")


def test_core_storage_memory_formats_chunking_telemetry_health(tmp_path):
    import json
    from torsh_b200.core import storage as S, telemetry as T
    # memory formats agree with torch's strides
    shape = (2, 3, 4, 5)
    assert S.MemoryFormat.CONTIGUOUS.strides(shape) == torch.empty(shape).stride()
    assert S.MemoryFormat.CHANNELS_LAST.strides(shape) == torch.empty(shape).to(memory_format=torch.channels_last).stride()
    s5 = (2, 3, 4, 5, 6)
    assert S.MemoryFormat.CHANNELS_LAST_3D.strides(s5) == torch.empty(s5).to(memory_format=torch.channels_last_3d).stride()
    assert S.MemoryFormat.of(torch.empty(shape).to(memory_format=torch.channels_last)) is S.MemoryFormat.CHANNELS_LAST
    assert S.MemoryFormat.of(torch.empty(4, 6).t()) is S.MemoryFormat.STRIDED
    with pytest.raises(ValueError):
        S.MemoryFormat.CHANNELS_LAST.strides((2, 3, 4))
    # storages
    before = S.registry.total_bytes()
    st = S.Storage.aligned(1000, torch.float32, alignment=256)
    assert st.tensor.data_ptr() % 256 == 0 and len(st) == 1000 and S.registry.total_bytes() == before + 4000
    v = st.view((2, 3, 4, 5), fmt=S.MemoryFormat.CHANNELS_LAST)
    v.zero_(); v[1, 2, 3, 4] = 7.0
    assert st.tensor[1 * 60 + 3 * 15 + 4 * 3 + 2] == 7.0 and S.is_aligned(v, 256)      # NHWC position of (n=1, c=2, h=3, w=4)
    with pytest.raises(ValueError):
        st.view((40, 40))
    m = S.Storage.mapped(tmp_path / "w.bin", 16, torch.int32, create=True)
    m.tensor.copy_(torch.arange(16, dtype=torch.int32)); m.flush()
    again = S.Storage.mapped(tmp_path / "w.bin", 16, torch.int32)
    assert again.tensor.tolist() == list(range(16)) and S.registry.info["mapped"].live >= 2
    assert S.Storage.shared(8).tensor.is_shared()
    del st
    import gc; gc.collect()
    assert S.registry.info["aligned"].peak_bytes >= 4000
    # chunking
    cfg = S.TensorChunkConfig(S.ChunkingStrategy.COMPUTE_INTENSIVE)
    n = cfg.compute_chunk_size(148 * 1024 * 64, 4)
    assert n % 64 == 0 and len(cfg.chunks(148 * 1024 * 64, 4)) == 148
    mem = S.TensorChunkConfig(S.ChunkingStrategy.MEMORY_INTENSIVE).compute_chunk_size(1 << 30, 2)
    assert mem * 2 <= (126 << 20) // 4 and S.TensorChunkConfig(S.ChunkingStrategy.CACHE_FRIENDLY).compute_chunk_size(10, 4) == 10
    ch = S.TensorChunkConfig(S.ChunkingStrategy.CUSTOM, custom_bytes=4096).chunks(2500, 4)
    assert ch[0] == (0, 1024) and ch[-1] == (2048, 2500)
    # telemetry
    lines = []
    tel = T.TelemetrySystem(T.TelemetryConfig(min_level=T.LogLevel.INFO, max_events=3, sink=lines.append))
    assert tel.log(T.LogLevel.DEBUG, "hidden") is None
    root = tel.start_span("step")
    with tel.span("forward", parent_id=root) as sid:
        tel.span_add_attribute(sid, "tokens", 8192)
        tel.span_add_event(sid, "graph_replay", launches=634)
        tel.log(T.LogLevel.INFO, "running", module="engine", span_id=sid, step=3)
    with pytest.raises(ValueError):
        with tel.span("bad", parent_id=root):
            raise ValueError("boom")
    tel.end_span(root)
    names = [m.name for m in tel.finished]
    assert names == ["forward", "bad", "step"] and tel.finished[0].parent_id == root and tel.finished[0].attributes["tokens"] == 8192
    assert tel.finished[0].events[0]["name"] == "graph_replay" and tel.finished[2].duration_s >= tel.finished[0].duration_s
    rec = json.loads(lines[0])
    assert rec["level"] == "INFO" and rec["module"] == "engine" and rec["step"] == 3 and rec["span_id"] == sid
    err = tel.get_events(T.LogLevel.ERROR)[0]
    assert err.error_code is T.ErrorCode.INVALID_ARGUMENT and json.loads(err.format_structured())["error_code"] == 1001
    for i in range(5):
        tel.log(T.LogLevel.WARN, f"w{i}")
    assert len(tel.events) == 3 and tel.dropped >= 2
    assert T.ErrorCode.from_exception(FileNotFoundError()) is T.ErrorCode.IO and T.ErrorCode.from_exception(KeyError()) is T.ErrorCode.INTERNAL
    # health
    hc = T.HealthChecker()
    hc.register("store", lambda: True)
    rep = hc.check_health()
    assert {c.name for c in rep.checks} == {"host_memory", "device", "kernel_status", "store"} and rep.status.is_operational()
    hc.register("disk", lambda: (_ for _ in ()).throw(OSError("disk gone")))
    rep = hc.check_health()
    assert rep.status is T.HealthStatus.UNHEALTHY and not hc.is_ready() and hc.is_alive() and hc.count == 2
    bad = rep.failing_checks()
    assert any(c.name == "disk" and c.error_code is T.ErrorCode.IO for c in bad) and "disk" in rep.summary()
    js = json.loads(rep.to_json())
    assert js["http"] == 503 and js["status"] == "unhealthy" and len(js["checks"]) == 5
