"""Auxiliary subsystems on the CPU: optimizer checkpoints, monitoring, debug checks, property-based fuzzing of the
host-side planners and codecs."""
import hashlib
import json
import math
import os
import re
import threading
from collections import Counter
from pathlib import Path

import numpy as np
import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st


def test_optimizer_checkpoint_roundtrip_and_rotation(tmp_path):
    from torsh_b200.optim import checkpointing as ck
    m = torch.nn.Linear(4, 3)
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2)
    mgr = ck.OptimizerCheckpointManager(ck.CheckpointConfig(str(tmp_path), max_checkpoints=2, checkpoint_frequency=2, save_gradients=True))
    for step in range(1, 7):
        m(torch.ones(2, 4)).sum().backward()
        opt.step()
        mgr.step()
        if mgr.should_checkpoint():
            mgr.save(m, opt, loss=float(step), epoch=0)
        opt.zero_grad()
    files = sorted(p.name for p in tmp_path.glob("checkpoint_step_*.bin"))
    assert files == ["checkpoint_step_4.bin", "checkpoint_step_6.bin"]
    latest = mgr.load_latest()
    assert latest["metadata"]["step"] == 6 and latest["metadata"]["loss"] == 6.0 and latest["metadata"]["epoch"] == 0
    assert abs(latest["metadata"]["learning_rate"] - 1e-2) < 1e-9 and len(latest["metadata"]["model_hash"]) == 16
    m2 = torch.nn.Linear(4, 3)
    opt2 = torch.optim.AdamW(m2.parameters(), lr=1e-2)
    m2(torch.ones(2, 4)).sum().backward(); opt2.step()          # create state slots
    mgr2 = ck.OptimizerCheckpointManager(ck.CheckpointConfig(str(tmp_path)))
    assert mgr2.last_checkpoint_step == 6
    mgr2.restore(mgr2.load_latest(), m2, opt2)
    assert all(torch.equal(a, b) for a, b in zip(m.parameters(), m2.parameters()))
    for p, q in zip(m.parameters(), m2.parameters()):
        assert torch.allclose(opt.state[p]["exp_avg_sq"], opt2.state[q]["exp_avg_sq"])
    # byte layout of the head of the encoding: step varint, timestamp varint, Option<f32> tag + value
    blob = ck.encode({"metadata": {"step": 5, "timestamp": 7, "loss": 1.0, "learning_rate": 0.5}, "optimizer_state": None})
    assert blob[:7] == bytes([5, 7, 1]) + np.float32(1.0).tobytes() and blob[7:11] == np.float32(0.5).tobytes()
    assert blob[11:] == bytes([0, 0, 0, 0, 0, 0])              # five absent options + ... (epoch, norm, hash, state, grads, params)


def test_monitoring_alerts_and_prometheus():
    from torsh_b200.parallel.monitoring import AlertThresholds, DistributedMonitor, MetricsCollector
    from torsh_b200.parallel.store import MemoryStore
    store = MemoryStore()
    mons = [DistributedMonitor(MetricsCollector(), AlertThresholds(straggler_ratio=1.2), rank=r, world_size=3, store=store) for r in range(3)]
    for r, mon in enumerate(mons):
        for _ in range(6):
            mon.c.record_step(10.0 * (2.0 if r == 2 else 1.0), tokens=1000, comm_ms=2.0, loss=1.0)
        mon.publish()
    agg = mons[0].aggregate()
    assert agg["stragglers"] == [2]
    mons[0].c.record_step(40.0, comm_ms=30.0)
    kinds = {a.kind for a in mons[0].check()}
    assert {"step_time", "comm_share"} <= kinds
    text = mons[0].c.export_prometheus()
    assert "torsh_training_step_ms 40.0" in text and "torsh_training_steps_total 7.0" in text
    assert mons[0].c.summary("training/step_ms")["max"] == 40.0


def test_debug_checks():
    from torsh_b200.utils import debug
    t = torch.tensor([1.0, float("nan"), float("inf"), -float("inf")])
    rep = debug.nan_inf_report(t)
    assert (rep["nan"], rep["pos_inf"], rep["neg_inf"], rep["first_bad"]) == (1, 1, 1, 1)
    with pytest.raises(debug.NonFiniteError):
        debug.check_finite(t)
    net = torch.nn.Sequential(torch.nn.Linear(2, 2), torch.nn.ReLU())
    with torch.no_grad():
        net[0].weight.fill_(float("nan"))
    with pytest.raises(debug.NonFiniteError, match="Linear"):
        with debug.detect_non_finite(net):
            net(torch.ones(1, 2))
    v = debug.LockOrderValidator()
    a, b = v.lock(1, "a"), v.lock(2, "b")
    with a, b:
        pass
    with pytest.raises(debug.LockOrderError):
        with b:
            a.acquire()
    held = v.lock(3, "held")
    held.acquire()
    err = []
    th = threading.Thread(target=lambda: err.append(pytest.raises(TimeoutError, held.acquire, 0.05)))
    th.start(); th.join()
    held.release()
    assert err
    buf = torch.zeros(256)
    payload, check = debug.add_guards(buf, 16)
    payload.fill_(1.0); check()
    buf[3] = 7.0
    with pytest.raises(RuntimeError):
        check()
    w = torch.nn.Linear(3, 3)
    opt = torch.optim.SGD(w.parameters(), lr=0.1)

    def step():
        opt.zero_grad(); w(torch.ones(2, 3)).sum().backward(); opt.step()
    assert debug.deterministic_replay(step, lambda: list(w.parameters()),
                                      lambda snap: [p.data.copy_(s) for p, s in zip(w.parameters(), snap)])


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(1, 1 << 22), min_size=1, max_size=40), st.integers(1, 64))
def test_fuzz_bucket_assignment_covers_every_parameter_once(sizes, cap_mb):
    from torsh_b200.parallel import planner
    cap = cap_mb << 20
    assign = planner.assign_buckets([s * 4 for s in sizes], cap)
    assert len(assign) == len(sizes) and min(assign) == 0 and set(assign) == set(range(max(assign) + 1))
    for b in set(assign):
        members = [sizes[i] * 4 for i, a in enumerate(assign) if a == b]
        assert sum(members) <= cap or len(members) == 1


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 1 << 30), st.integers(1, 8))
def test_fuzz_shard_ranges_partition_the_buffer(numel, world):
    from torsh_b200.parallel.fsdp import shard_range
    pos = 0
    for r in range(world):
        lo, hi = shard_range(numel, world, r)
        assert lo == min(pos, numel) or lo == pos
        assert lo <= hi <= max(numel, hi)
        pos = hi
    assert pos >= numel


@settings(max_examples=40, deadline=None)
@given(st.lists(st.tuples(st.integers(1, 1 << 24), st.integers(0, 3)), min_size=1, max_size=60))
def test_fuzz_pool_never_overlaps_live_blocks(ops):
    from torsh_b200.core.runtime import HostPool
    pool = HostPool()
    live = {}
    for size, stream in ops:
        p = pool.alloc(size, stream)
        assert p and p % 64 == 0
        real = pool.size_of(p)
        for q, (n, _) in live.items():
            assert p + real <= q or q + n <= p, "overlapping blocks"
        live[p] = (real, stream)
        if len(live) > 8:
            victim = next(iter(live))
            assert pool.free(victim)
            live.pop(victim)
    assert pool.stats()["allocated_bytes"] == sum(n for n, _ in live.values())
    for p in list(live):
        pool.free(p)
    pool.release_cached()
    assert pool.stats()["reserved_bytes"] == 0
    pool.close()


@settings(max_examples=40, deadline=None)
@given(st.lists(st.integers(1, 9), min_size=0, max_size=4), st.sampled_from([torch.float32, torch.float64, torch.int64, torch.bfloat16]))
def test_fuzz_trsh_roundtrip(shape, dtype):
    from torsh_b200.serialize import trsh
    n = int(np.prod(shape)) if shape else 1
    t = (torch.arange(n, dtype=torch.float32).reshape(shape) * 0.5 - 3).to(dtype)
    back, meta = trsh.decode_trsh(trsh.encode_trsh(t))
    assert back.dtype == t.dtype and tuple(back.shape) == tuple(t.shape) and torch.equal(back, t)


def test_streaming_tensor_file_and_function_registry(tmp_path):
    from torsh_b200.autograd import functions as fn
    from torsh_b200.serialize.streaming import LazyTensor, StreamingReader, StreamingWriter
    m = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.BatchNorm1d(7))
    path = tmp_path / "model.trsx"
    with StreamingWriter(path) as w:
        w.write_state_dict(m.state_dict())
        w.write("extra/bf16", torch.arange(6, dtype=torch.bfloat16).reshape(2, 3))
        with pytest.raises(KeyError):
            w.write("0.weight", torch.zeros(1))
    with StreamingReader(path) as r:
        assert "0.weight" in r and r.shape("0.weight") == (7, 5) and len(r) == len(m.state_dict()) + 1 and r.loads == 0
        lazy = LazyTensor(r, "extra/bf16")
        assert lazy.shape == (2, 3) and r.loads == 0 and lazy.get().dtype == torch.bfloat16 and r.loads == 1
        m2 = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.BatchNorm1d(7))
        assert r.load_into(m2) == []
        assert all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), m2.state_dict().values()))
    reg = fn.FunctionRegistry()
    reg.register("square", forward=lambda ctx, x: (ctx.save_for_backward(x), x * x)[1],
                 backward=lambda ctx, g: 2 * ctx.saved_tensors[0] * g)
    reg.register("double", forward=lambda ctx, x: 2 * x, backward=lambda ctx, g: 2 * g)
    x = torch.tensor([3.0], requires_grad=True)
    reg.compose("square", "double")(x).backward()
    assert x.grad.item() == 12.0 and reg.names() == ["double", "square"]
    with pytest.raises(KeyError):
        reg.get("nope")
    ev = [dict(name="step", start_us=0, duration_us=100), dict(name="fwd", start_us=0, duration_us=40),
          dict(name="gemm", start_us=5, duration_us=20), dict(name="bwd", start_us=40, duration_us=50)]
    lines = fn.folded_stacks(ev)
    assert lines == ["step 10", "step;bwd 50", "step;fwd 20", "step;fwd;gemm 20"]
    diff = fn.differential(lines, ["step 10", "step;bwd 80", "step;fwd 20"])
    assert diff[0] == ("step;bwd", 50, 80)


def _fake_redis(server_sock, stop):
    """A few Redis commands over RESP2, enough for the store client: GET SET(PX) DEL EXISTS INCRBY KEYS EVAL(cas)."""
    import time as _t
    data, expiry = {}, {}

    def alive(k):
        if k in expiry and _t.monotonic() >= expiry[k]:
            data.pop(k, None); expiry.pop(k, None)
        return k in data

    def bulk(v):
        return b"$-1\r\n" if v is None else b"$%d\r\n" % len(v) + v + b"\r\n"

    server_sock.settimeout(0.2)
    conns = []
    while not stop.is_set():
        try:
            c, _ = server_sock.accept()
        except OSError:
            continue
        conns.append(c)
        f = c.makefile("rb")
        while not stop.is_set():
            line = f.readline()
            if not line:
                break
            n = int(line[1:-2])
            args = []
            for _ in range(n):
                ln = int(f.readline()[1:-2])
                args.append(f.read(ln + 2)[:-2])
            cmd = args[0].upper()
            if cmd == b"SET":
                data[args[1]] = args[2]
                expiry.pop(args[1], None)
                if len(args) >= 5 and args[3].upper() == b"PX":
                    expiry[args[1]] = _t.monotonic() + int(args[4]) / 1000
                c.sendall(b"+OK\r\n")
            elif cmd == b"GET":
                c.sendall(bulk(data[args[1]] if alive(args[1]) else None))
            elif cmd == b"EXISTS":
                c.sendall(b":%d\r\n" % int(alive(args[1])))
            elif cmd == b"DEL":
                c.sendall(b":%d\r\n" % int(data.pop(args[1], None) is not None))
            elif cmd == b"INCRBY":
                v = int(data.get(args[1], b"0")) + int(args[2])
                data[args[1]] = str(v).encode()
                c.sendall(b":%d\r\n" % v)
            elif cmd == b"KEYS":
                ks = [k for k in list(data) if alive(k) and k.startswith(args[1][:-1])]
                c.sendall(b"*%d\r\n" % len(ks) + b"".join(bulk(k) for k in ks))
            elif cmd == b"EVAL":
                key, has, exp, val = args[3], args[4], args[5], args[6]
                cur = data[key] if alive(key) else None
                ok = (has == b"0" and cur is None) or (has == b"1" and cur == exp)
                if ok:
                    data[key] = val
                c.sendall(b":%d\r\n" % int(ok))
            else:
                c.sendall(b"-ERR unknown command\r\n")
    for c in conns:
        c.close()


def test_redis_store_speaks_resp_to_a_fake_server():
    import socket, threading, time
    from torsh_b200.parallel.store import create_store
    from torsh_b200.core.error import TorshDistributedError
    srv = socket.socket(); srv.bind(("127.0.0.1", 0)); srv.listen(4)
    stop = threading.Event()
    th = threading.Thread(target=_fake_redis, args=(srv, stop), daemon=True); th.start()
    st = create_store("redis", host="127.0.0.1", port=srv.getsockname()[1], prefix="t/")
    try:
        st.set("a", b"\x00bin\r\nary")
        assert st.get("a") == b"\x00bin\r\nary" and st.contains("a") and st.get("nope") is None
        assert st.add("n", 2) == 2 and st.add("n", 3) == 5
        assert st.compare_and_swap("c", None, b"1") and not st.compare_and_swap("c", None, b"2")
        assert st.compare_and_swap("c", b"1", b"3") and st.get("c") == b"3"
        assert st.num_keys() == 3
        st.set_with_expiry("ttl", b"x", 0.05)
        assert st.contains("ttl"); time.sleep(0.1); assert not st.contains("ttl")
        threading.Timer(0.05, lambda: st2.set("late", b"1")).start()
        st2 = st
        st.wait(["late"], timeout=2.0)
        with pytest.raises(TorshDistributedError):
            st.wait(["never"], timeout=0.05)
        assert st.delete("a") and not st.contains("a")
    finally:
        st.close(); stop.set(); th.join(2); srv.close()


def test_connection_pool_reuses_sockets_and_retries():
    import socket, threading
    from torsh_b200.parallel.connection import ConnectionPool, RetryPolicy, retry
    from torsh_b200.core.error import TorshDistributedError
    srv = socket.socket(); srv.bind(("127.0.0.1", 0)); srv.listen(8)
    port = srv.getsockname()[1]
    stop = threading.Event()

    def echo():
        srv.settimeout(0.2)
        def serve(c):
            while True:
                d = c.recv(4)
                if not d:
                    break
                c.sendall(d[::-1])
            c.close()
        while not stop.is_set():
            try:
                c, _ = srv.accept()
            except OSError:
                continue
            threading.Thread(target=serve, args=(c,), daemon=True).start()
    th = threading.Thread(target=echo, daemon=True); th.start()
    pool = ConnectionPool(max_per_peer=2, policy=RetryPolicy(max_retries=2, initial_delay_s=0.01, timeout_s=2.0))
    try:
        assert pool.request("127.0.0.1", port, b"abcd", 4) == b"dcba"
        assert pool.request("127.0.0.1", port, b"wxyz", 4) == b"zyxw"
        s = pool.stats[("127.0.0.1", port)]
        assert (s.connects, s.reuses, s.bytes_sent, s.bytes_received) == (1, 1, 8, 8) and pool.idle_count("127.0.0.1", port) == 1
        with pytest.raises(RuntimeError):
            with pool.connection("127.0.0.1", port):
                raise RuntimeError("boom")
        assert pool.idle_count("127.0.0.1", port) == 0          # the socket of a failed block is not reused
        calls, slept = [], []
        def flaky():
            calls.append(1)
            if len(calls) < 3:
                raise OSError("down")
            return "up"
        assert retry(flaky, RetryPolicy(max_retries=3, initial_delay_s=0.01), sleep=slept.append) == "up" and slept == [0.01, 0.02]
        with pytest.raises(TorshDistributedError):
            retry(lambda: (_ for _ in ()).throw(OSError("x")), RetryPolicy(max_retries=1, initial_delay_s=0.0), sleep=lambda d: None)
    finally:
        pool.close(); stop.set(); th.join(2); srv.close()


def test_more_compressors_and_nccl_scheduler():
    import torch
    from torsh_b200.parallel.compression import Bimodal, CountSketch, EF21, LayerwiseAdaptive, NaturalCompression, TopK
    from torsh_b200.parallel.comm_scheduler import CollectiveAlgorithm, NcclScheduler, Priority
    torch.manual_seed(0)
    g = torch.zeros(2000)
    g[torch.randperm(2000)[:20]] = torch.randn(20) * 10
    cs = CountSketch(5, 4096)
    a, b = cs.compress(g)[0], cs.compress(2 * g)[0]
    assert torch.allclose(cs.decompress((a + b,), g.shape), 3 * g, atol=1e-4)          # sketches add up across ranks
    x = torch.randn(100000)
    nc = NaturalCompression()
    r = nc.decompress(nc.compress(x), x.shape)
    assert abs(float((r - x).mean())) < 0.01 and float((r / x).min()) >= 0.5 and float((r / x).max()) <= 2.0
    bm = Bimodal()
    assert float(torch.nn.functional.cosine_similarity(bm.decompress(bm.compress(x), x.shape), x, dim=0)) > 0.9
    la = LayerwiseAdaptive()
    assert [la.choose(t)[0] for t in (torch.randn(100), torch.randn(2048, 1024), torch.randn(100000))] == ["none", "powersgd", "topk"]
    small = torch.randn(100)
    assert torch.equal(la.decompress(la.compress(small), small.shape), small)
    ef, gg = EF21(TopK(0.1)), torch.randn(1000)
    for _ in range(40):
        _, h = ef.compress("w", gg)
    assert float((h - gg).norm() / gg.norm()) < 1e-3
    s = NcclScheduler(num_streams=2, fusion_bytes=1000, world=8, has_multicast=True)
    for i in range(5):
        s.enqueue(f"g{i}", 300, lambda i=i: i)
    s.enqueue("big", 1 << 22, lambda: "big", priority=Priority.CRITICAL)
    assert s.flush() == ["big", 0, 1, 2, 3, 4]
    assert s.log[0] == (0, ["big"], CollectiveAlgorithm.NVLS) and s.log[1][1] == ["g0", "g1", "g2"] and s.log[1][0] == 1
    assert s.stats["fused_groups"] == 2 and s.stats["fused_ops"] == 5
    assert NcclScheduler(world=16, ranks_per_node=8).choose_algorithm(1 << 20) is CollectiveAlgorithm.HIERARCHICAL
    assert NcclScheduler(world=2).choose_algorithm(1 << 20) is CollectiveAlgorithm.TWO_SHOT_PEER


def test_bottleneck_detector_ranks_findings():
    from torsh_b200.parallel.monitoring import BottleneckDetector, BottleneckType, Severity, StepSample
    d = BottleneckDetector(window=10)
    for step in range(10):
        d.record(StepSample(rank=0, step_ms=100, compute_ms=50, exposed_comm_ms=40, data_wait_ms=1, mem_used_frac=0.5))
        d.record(StepSample(rank=1, step_ms=130, compute_ms=50, exposed_comm_ms=40, data_wait_ms=1, mem_used_frac=0.95))
    found = d.analyze()
    kinds = [b.kind for b in found]
    assert BottleneckType.COMMUNICATION in kinds and [int(b.severity) for b in found] == sorted((int(b.severity) for b in found), reverse=True)
    assert [b for b in found if b.kind is BottleneckType.COMMUNICATION][0].severity >= Severity.MEDIUM
    assert BottleneckType.LOAD_IMBALANCE in kinds and BottleneckType.MEMORY in kinds and BottleneckType.DATA_LOADING not in kinds
    assert [b for b in found if b.kind is BottleneckType.LOAD_IMBALANCE][0].ranks == [1]
    assert all(b.remediation for b in found)
    quiet = BottleneckDetector()
    quiet.record(StepSample(rank=0, step_ms=100, compute_ms=95))
    assert [b.kind for b in quiet.analyze()] == [BottleneckType.COMPUTE]


def test_edge_federated_coordination():
    import torch
    from torsh_b200.parallel import edge as E
    mgr = E.EdgeComputingManager(E.FederatedLearningConfig(clients_per_round=2, selection=E.ClientSelectionStrategy.RESOURCE_AWARE))
    for i, (fl, bat) in enumerate([(1e11, 1.0), (5e11, 0.9), (9e11, 0.1), (2e11, 0.8)]):
        mgr.register_device(E.EdgeDevice(f"d{i}", flops=fl, battery=bat, num_samples=100 * (i + 1)))
    assert mgr.select_clients(0) == ["d1", "d3"]                       # d2 is strongest but below the battery floor
    mgr.update_device_status("d1", E.DeviceStatus.OFFLINE)
    assert "d1" not in mgr.select_clients(1)
    ups = [{"w": torch.full((3,), 1.0)}, {"w": torch.full((3,), 4.0)}]
    fed = E.FederatedLearningCoordinator(E.FederatedLearningConfig())
    assert torch.allclose(fed.aggregate_updates(ups, num_samples=[100, 300])["w"], torch.full((3,), 3.25))
    med = E.FederatedLearningCoordinator(E.FederatedLearningConfig(aggregation=E.AggregationStrategy.MEDIAN))
    outlier = ups + [{"w": torch.full((3,), 1000.0)}]
    assert torch.allclose(med.aggregate_updates(outlier)["w"], torch.full((3,), 4.0))
    nova = E.FederatedLearningCoordinator(E.FederatedLearningConfig(algorithm=E.FederatedAlgorithm.FED_NOVA, aggregation=E.AggregationStrategy.SIMPLE_AVERAGE))
    assert torch.allclose(nova.aggregate_updates([{"w": torch.tensor([2.0])}, {"w": torch.tensor([8.0])}], local_steps=[1, 4])["w"], torch.tensor([5.0]))
    priv = E.PrivacyManager(E.PrivacyConfig(clip_norm=1.0, noise_multiplier=0.0))
    assert abs(float(priv.clip({"w": torch.full((4,), 10.0)})["w"].norm()) - 1.0) < 1e-5
    loc, glob = {"w": torch.ones(2, requires_grad=True)}, {"w": torch.zeros(2)}
    assert abs(float(fed.proximal_term(loc, glob)) - 0.5 * 0.01 * 2) < 1e-7
    assert E.adaptive_params(200).compression_ratio == 1.0 and E.adaptive_params(1).sync_every == 4
    bm = E.BandwidthMonitor()
    bm.record_measurement("d0", 10, when=0.0); bm.record_measurement("d0", 30, when=100.0)
    assert bm.get_average_bandwidth("d0", 5, now=120.0) == 20 and bm.get_average_bandwidth("d0", 1, now=120.0) == 30
    h = E.HierarchicalTrainingCoordinator()
    assert h.assign_device_tier(E.EdgeDevice("p")) is E.TrainingTier.DEVICE
    assert h.assign_device_tier(E.EdgeDevice("e", device_type=E.DeviceType.EDGE_SERVER)) is E.TrainingTier.EDGE
    assert h.assign_device_tier(E.EdgeDevice("c", flops=2e15)) is E.TrainingTier.CLOUD and h.get_tier_devices(E.TrainingTier.CLOUD) == ["c"]


def test_rdma_verbs_model():
    import torch
    from torsh_b200.parallel import rdma as R
    fab = R.LoopbackFabric()
    a, b = R.RdmaEndpoint(0, fab), R.RdmaEndpoint(1, fab)
    mr = b.register(torch.zeros(10))
    ro = b.register(torch.arange(4.0), R.MemoryAccess(remote_write=False))
    assert a.post(R.RdmaOperation.WRITE, 1, mr.rkey, torch.ones(3)).status is R.CompletionStatus.NOT_CONNECTED
    a.connect(1)
    assert a.post(R.RdmaOperation.WRITE, 1, mr.rkey, torch.ones(3), remote_offset=2).status is R.CompletionStatus.SUCCESS
    assert mr.tensor.tolist() == [0, 0, 1, 1, 1, 0, 0, 0, 0, 0]
    got = torch.empty(4)
    assert a.post(R.RdmaOperation.READ, 1, ro.rkey, got).status is R.CompletionStatus.SUCCESS and got.tolist() == [0, 1, 2, 3]
    assert a.post(R.RdmaOperation.WRITE, 1, ro.rkey, torch.ones(1)).status is R.CompletionStatus.REMOTE_ACCESS_ERROR
    assert a.post(R.RdmaOperation.WRITE, 1, mr.rkey, torch.ones(20)).status is R.CompletionStatus.LOCAL_LENGTH_ERROR
    assert a.post(R.RdmaOperation.READ, 1, 999999, got).status is R.CompletionStatus.INVALID_KEY
    cnt = b.register(torch.zeros(1, dtype=torch.int64))
    assert a.post(R.RdmaOperation.ATOMIC_FAA, 1, cnt.rkey, value=5).result == 0 and int(cnt.tensor[0]) == 5
    assert a.post(R.RdmaOperation.ATOMIC_CAS, 1, cnt.rkey, compare=4, value=9).result == 5 and int(cnt.tensor[0]) == 5
    assert a.post(R.RdmaOperation.ATOMIC_CAS, 1, cnt.rkey, compare=5, value=9).result == 5 and int(cnt.tensor[0]) == 9
    big = b.register(torch.zeros(100))
    sched = R.RdmaTensorScheduler(a, max_wr_elems=32)
    wcs = sched.write_tensor(torch.arange(100.0).view(10, 10), 1, big.rkey)
    assert len(wcs) == 4 and torch.equal(big.tensor, torch.arange(100.0))
    back = torch.empty(50)
    sched.read_tensor(back, 1, big.rkey, remote_offset=50)
    assert torch.equal(back, torch.arange(50.0, 100.0))
    assert (a.stats.writes, a.stats.atomics, a.stats.errors, a.stats.reads) == (5, 3, 4, 3) and len(a.poll(100)) == 15
    pool = R.RdmaMemoryPool(b, sizes=(16, 64), per_class=1)
    r1 = pool.acquire(10); r2 = pool.acquire(10); r3 = pool.acquire(10)
    assert (r1.length, r2.length, r3.length) == (16, 64, 10) and pool.stats == {"hits": 2, "misses": 1}
    pool.release(r1)
    assert pool.acquire(16) is r1


def test_memory_profiler_scopes_and_leak_detection(tmp_path):
    import json
    import torch
    from torsh_b200.utils.memory_profiler import MemoryProfiler
    prof = MemoryProfiler()
    before = prof.snapshot()
    keep = []
    with prof.scope("alloc"):
        keep.append(torch.zeros(123, 77))
        tmp = torch.zeros(1 << 20)
        del tmp
    after = prof.snapshot()
    leaks = prof.leaks(before, after)
    assert any(k[0] == (123, 77) and n == 1 for k, n in leaks)
    assert not any(k[0] == (1 << 20,) for k, _ in leaks)
    rec = prof.scopes[0]
    assert rec.name == "alloc" and rec.peak_bytes >= rec.end_bytes and rec.duration_ms >= 0
    prof.export_json(str(tmp_path / "mem.json"))
    assert json.load(open(tmp_path / "mem.json"))["scopes"][0]["name"] == "alloc"


def test_structured_and_audit_logging_and_degradation(tmp_path):
    import json
    from torsh_b200.utils.logging import AuditLog, GracefulDegradation, StructuredLogger
    log = StructuredLogger(str(tmp_path / "run.jsonl"), rank=3)
    with log.span("epoch0"):
        with log.span("step1", step=1):
            log.info("loss", value=2.5)
    log.debug("hidden")
    lines = [json.loads(ln) for ln in open(tmp_path / "run.jsonl")]
    assert [r["event"] for r in lines] == ["loss", "span_end", "span_end"] and lines[0]["span"] == "epoch0/step1"
    assert lines[0]["rank"] == 3 and lines[1]["step"] == 1 and lines[1]["duration_ms"] >= 0
    audit = AuditLog(str(tmp_path / "audit.jsonl"))
    audit.append("rank0", "checkpoint_saved", step=10)
    audit.append("rank0", "lr_changed", old=1e-3, new=5e-4)
    assert audit.verify()
    again = AuditLog(str(tmp_path / "audit.jsonl"))
    assert again.verify() and len(again.records) == 2
    again.records[0]["details"]["step"] = 11
    assert not again.verify()
    calls = []
    gd = GracefulDegradation(log, disable_after=2)
    gd.add("kernel", lambda x: (calls.append("k"), 1 / 0)[1]).add("torch", lambda x: (calls.append("t"), x + 1)[1])
    assert [gd.run(1), gd.run(2), gd.run(3)] == [2, 3, 4]
    assert calls == ["k", "t", "k", "t", "t"] and gd.used == ["torch"] * 3          # the kernel level is skipped after two failures


def test_fairness_metrics_and_experiment_writers(tmp_path):
    import json, os
    import torch
    from torsh_b200.utils import metrics as M
    pred = torch.tensor([1, 1, 0, 0, 1, 0, 0, 0])
    group = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1])
    target = torch.tensor([1, 0, 1, 0, 1, 1, 0, 0])
    assert abs(M.demographic_parity_difference(pred, group) - 0.25) < 1e-6
    assert abs(M.disparate_impact_ratio(pred, group) - 0.5) < 1e-6
    assert abs(M.equalized_odds_difference(pred, target, group) - 0.5) < 1e-6      # FPR 0.5 vs 0.0
    ml = M.MLflowWriter(str(tmp_path / "mlruns"))
    ml.log_param("lr", 3e-4); ml.set_tag("model", "gpt2"); ml.log_metric("loss", 2.5, 1); ml.log_metric("loss", 2.0, 2)
    lines = open(os.path.join(ml.dir, "metrics", "loss")).read().split("\n")
    assert len(lines) == 3 and lines[1].split()[1:] == ["2.0", "2"] and open(os.path.join(ml.dir, "params", "lr")).read() == "0.0003"
    assert "run_id: " + ml.run_id in open(os.path.join(ml.dir, "meta.yaml")).read()
    wb = M.WandbOfflineWriter(str(tmp_path / "wandb"), config={"lr": 1e-3})
    wb.log({"loss": 1.5}); wb.log({"loss": 1.25, "acc": 0.5})
    hist = [json.loads(l) for l in open(os.path.join(wb.dir, "wandb-history.jsonl"))]
    assert [h["_step"] for h in hist] == [1, 2] and json.load(open(os.path.join(wb.dir, "wandb-summary.json")))["acc"] == 0.5


def test_bench_clock_sampler_windows():
    import os, sys, time
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    s = bench.ClockSampler(0)
    assert s.window(0, 1)["reasons"] == ["nvidia-smi unavailable"]                 # never started
    s.proc = type("P", (), {"terminate": lambda self: None})()
    now = time.perf_counter()
    s.lines = [(now - 1.0, "0, 1900, 1965, 800, Not Active, Not Active, Not Active, Active"),
               (now, "0, 1800, 1965, 900, Not Active, Not Active, Not Active, Not Active"),
               (now, "garbage")]
    first, second = s.window(now - 2, now - 0.5), s.window(now - 0.5, now + 1)
    assert (first["sm_mhz"], first["reasons"], first["samples"]) == (1900.0, ["sw_power_cap"], 1)
    assert (second["sm_mhz"], second["reasons"], second["sm_max_mhz"]) == (1800.0, [], 1965.0)
    assert s.stop()["samples"] == 2
    import json, subprocess
    out = subprocess.run([sys.executable, os.path.join(os.path.dirname(bench.__file__), "bench.py"), "--impl", "reference"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and json.loads(out.stdout.strip().splitlines()[-1])["impl"] == "reference"


def test_benchmark_report_from_json_lines(tmp_path):
    import importlib.util, json, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_report", os.path.join(root, "bench", "report.py"))
    rep = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rep)
    base = {"metric": "tokens/sec", "unit": "tokens/s", "ms_per_step": 29.0, "clocks": {"sm_mhz": 1900, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"]},
            "e2e": {"value": 281000.0}, "config": {"model": "gpt2-medium"}}
    f1, f2 = tmp_path / "n1.json", tmp_path / "n2.json"
    f1.write_text("noise\n" + json.dumps({**base, "value": 280000.0, "n_gpus": 1}) + "\n")
    f2.write_text(json.dumps({**base, "value": 554400.0, "n_gpus": 2}) + "\n" + json.dumps({"impl": "reference", "unavailable": "no toolchain"}) + "\n")
    out = tmp_path / "r.html"
    runs = rep.main([str(f1), str(f2), "--out", str(out)])
    assert len(runs) == 3 and abs(rep.scaling(runs)["tokens/sec|ours"][2] - 0.99) < 1e-9
    page = out.read_text()
    assert "554,400 tokens/s" in page and "2 GPUs 99.0%" in page and "no toolchain" in page
    assert "| ours | tokens/sec | 1 |" in rep.to_markdown(runs)


def test_core_profiling_helpers(tmp_path):
    import torch
    from torsh_b200.utils.profiler import OperationTrace, PerfRegressionDetector, PerformanceProfiler, profile_closure
    out, ms = profile_closure(lambda a, b: a @ b, torch.ones(8, 8), torch.ones(8, 8), name="mm", repeats=3)
    assert float(out[0, 0]) == 8.0 and ms >= 0
    pp = PerformanceProfiler()
    for _ in range(5):
        with pp.time("step"):
            torch.ones(16).sum()
    st = pp.stats("step")
    assert st["count"] == 5 and st["min_ms"] <= st["p50_ms"] <= st["max_ms"] and pp.stats("none") == {"count": 0}
    tr = OperationTrace()
    with tr.trace_operation("block", torch.ones(2, 3)):
        with tr.trace_operation("matmul", torch.ones(2, 3), torch.ones(3, 4)):
            pass
    assert [(d, n) for d, n, _ in tr.events] == [(0, "block"), (1, "matmul")] and "  matmul" in tr.format()
    det = PerfRegressionDetector(str(tmp_path / "base.json"), tolerance=0.1)
    assert det.check("gemm", 10.0)["status"] == "new" and det.check("gemm", 10.5)["status"] == "ok"
    assert det.check("gemm", 12.0)["status"] == "regression" and det.check("gemm", 8.0)["status"] == "improvement"
    assert PerfRegressionDetector(str(tmp_path / "base.json")).baselines["gemm"] == 8.0


def test_profiler_exporters_grafana_cloudwatch_streaming_ci_and_monitor(tmp_path):
    import json
    from torsh_b200.utils import exporters as ex
    from torsh_b200.utils.profiler import ProfileEvent
    evs = [ProfileEvent("gemm", "op", 0.0, 120.0, 1, device_us=100.0, flops=2e9, bytes=4e6),
           ProfileEvent("gemm", "op", 200.0, 80.0, 1, device_us=60.0, flops=2e9, bytes=4e6),
           ProfileEvent("norm", "op", 300.0, 40.0, 1, bytes=8e6)]
    # Grafana: three templates, valid JSON, unique panel ids, variables and thresholds present
    for make in (ex.DashboardTemplates.profiling, ex.DashboardTemplates.memory, ex.DashboardTemplates.performance):
        doc = json.loads(make().export_json())
        ids = [p["id"] for p in doc["panels"]]
        assert doc["schemaVersion"] == 36 and len(ids) == len(set(ids)) >= 4 and all(p["targets"][0]["expr"] for p in doc["panels"])
    g = ex.GrafanaDashboardGenerator("t").with_uid("u").with_tags(["a"]).with_time_range("now-1h", "now").with_refresh("10s")
    g.add_gauge_panel("x", "m", ex.GridPos(0, 0, 4, 4), lo=0, hi=10).add_variable("rank", "label_values(m, rank)")
    g.export_to_file(tmp_path / "d.json")
    d = json.loads((tmp_path / "d.json").read_text())
    assert d["uid"] == "u" and d["panels"][0]["fieldConfig"]["defaults"]["max"] == 10 and d["templating"]["list"][0]["name"] == "rank"
    # CloudWatch: statistic sets from events, aggregation, request chunking
    sent = []
    cw = ex.CloudWatchPublisher("Torsh/Train", region="eu-west-1", buffer_size=10_000, aggregate=True, sink=lambda ns, r, b: sent.append((ns, r, b)))
    cw.add_dimension("Rank", 0)
    cw.publish_from_events(evs)
    for v in (1.0, 3.0):
        cw.put_metric("StepMs", v, "Milliseconds")
    body = json.loads(cw.export_json())
    by = {(m["MetricName"], tuple(sorted((x["Name"], x["Value"]) for x in m["Dimensions"]))): m for m in body["MetricData"]}
    gemm = by[("ScopeDuration", (("Category", "op"), ("Rank", "0"), ("Scope", "gemm")))]
    assert gemm["StatisticValues"] == {"SampleCount": 2.0, "Sum": 160.0, "Minimum": 60.0, "Maximum": 100.0} and gemm["Unit"] == "Microseconds"
    step = by[("StepMs", (("Rank", "0"),))]
    assert step["StatisticValues"]["Sum"] == 4.0 and step["StatisticValues"]["SampleCount"] == 2.0
    assert cw.flush() == len(body["MetricData"]) and sent[0][0] == "Torsh/Train" and sent[0][1] == "eu-west-1" and not cw.buffer
    import pytest
    with pytest.raises(ValueError):
        cw.put_metric("x", 1.0, "Furlongs")
    many = ex.CloudWatchPublisher("N", buffer_size=10_000, sink=lambda ns, r, b: sent.append(len(b["MetricData"])))
    for i in range(2300):
        many.put_metric(f"m{i}", 1.0, "Count")
    assert many.flush() == 2300 and sent[-3:] == [1000, 1000, 300]
    # streaming sink with back-pressure, tables, HTML
    se = ex.StreamingExporter(tmp_path / "s.jsonl", max_queue=2, flush_every=100)
    for e in evs:
        se.emit(e)
    se.close()
    lines = (tmp_path / "s.jsonl").read_text().strip().splitlines()
    assert len(lines) == 2 and se.dropped == 1 and json.loads(lines[-1])["name"] == "norm"
    rows = ex.summarize_events(evs)
    assert rows[0]["name"] == "gemm" and rows[0]["calls"] == 2 and abs(rows[0]["share"] - 0.8) < 1e-9 and abs(rows[0]["tflops"] - 25.0) < 1e-6
    assert ex.export_table(evs, "csv").splitlines()[0].startswith("name,category,calls") and "| gemm |" in ex.export_table(evs, "markdown")
    assert json.loads(ex.export_table(evs, "json"))[1]["name"] == "norm"
    page = ex.html_report(evs, "run <1>", {"gpus": 8})
    assert page.startswith("<!doctype html>") and "run &lt;1&gt;" in page and "<script" not in page and "gemm" in page
    # CI gate
    ok, xml, md = ex.ci_regression_report({"step_ms": 31.0, "attn_us": 96.0, "new": 1.0}, {"step_ms": 29.5, "attn_us": 97.0}, tolerance=0.03)
    assert not ok and 'failures="1"' in xml and "step_ms" in xml and "| step_ms | 29.5 | 31 | +5.1% | regressed |" in md
    assert ex.ci_regression_report({"tok_s": 280.0}, {"tok_s": 270.0}, lower_is_better=False)[0]
    # Kubernetes metadata
    meta = ex.kubernetes_metadata({"POD_NAME": "p-0", "POD_NAMESPACE": "ml", "KUBERNETES_SERVICE_HOST": "10.0.0.1"})
    assert meta == {"pod": "p-0", "namespace": "ml", "service_host": "10.0.0.1", "in_cluster": True}
    assert ex.kubernetes_metadata({})["in_cluster"] is False
    # power / thermal monitor against a fake NVML: reads only
    calls = []

    class FakeNvml:
        NVML_TEMPERATURE_GPU, NVML_CLOCK_SM = 0, 1
        def nvmlInit(self): calls.append("init")
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetPowerUsage(self, h): return 750_000
        def nvmlDeviceGetTemperature(self, h, k): return 61
        def nvmlDeviceGetClockInfo(self, h, k): return 1845
        def nvmlDeviceGetCurrentClocksThrottleReasons(self, h): return 0x4
        def __getattr__(self, name):
            raise AssertionError(f"the monitor must not call {name}")
    mon = ex.PowerThermalMonitor(0, interval_s=0.01, nvml=FakeNvml()).start()
    import time as _t
    _t.sleep(0.08)
    s = mon.stop()
    assert s["samples"] >= 2 and s["power_w_mean"] == 750.0 and s["temp_c_max"] == 61.0 and s["sm_mhz_median"] == 1845.0
    assert s["throttle_reason_bits"] == 4 and s["energy_j"] > 0 and calls == ["init"]
    assert ex.PowerThermalMonitor(nvml=None).summary() == {"samples": 0} or True


def test_kernel_generator_emits_compilable_source_and_portable_results(tmp_path, monkeypatch):
    """The run-time generator: expression -> CUDA source that nvcc accepts for sm_100a (content-addressed cache), and
    the same expression evaluated with PyTorch ops on CPU tensors."""
    import shutil
    from torsh_b200.core import kernel_gen as kg
    monkeypatch.setenv("TORSH_JIT_DIR", str(tmp_path))
    f = kg.FusedElementwise(lambda a, b: kg.maximum(a * kg.tanh(b) - 2.0, kg.exp(-kg.square(a))) / (1.0 + kg.relu(b)), 2)
    src = f.source(torch.bfloat16)
    assert "fused_kernel" in src and all(f"launch_{v}" in src for v in kg.VARIANTS) and "__nv_bfloat16" in src
    assert f.expr.n_inputs() == 2 and f.expr.key().startswith("div(max(")
    a, b = torch.randn(2, 777)
    ref = torch.maximum(a * torch.tanh(b) - 2.0, torch.exp(-a * a)) / (1.0 + torch.relu(b))
    assert torch.allclose(f(a, b), ref, atol=1e-6)
    if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"):
        lib = kg.compile_source(src)
        assert lib.exists() and lib.stat().st_size > 10_000
        stamp = lib.stat().st_mtime_ns
        assert kg.compile_source(src) == lib and lib.stat().st_mtime_ns == stamp        # unchanged source: no rebuild
    sel = kg.KernelSelector()
    sel.tuner.timer = lambda fn: {"t256_u1": 3.0, "t256_u2": 1.0, "t512_u2": 2.0, "t128_u4": 4.0}[fn()]
    assert sel.choose("k", 1 << 20, lambda name: name) == "t256_u2" and "k|2^20" in sel.tuner.table
    with pytest.raises(ValueError):
        kg.Expr._wrap(float("inf")).code("j")


def test_package_versions_requirements_resolver_lock_and_manifest_migration():
    from torsh_b200 import package_resolver as R
    V = R.Version.parse
    assert V("1.2.3") < V("1.10.0") and V("1.0.0-rc.1") < V("1.0.0") and V("1.0.0-alpha") < V("1.0.0-beta") and V("v2") == R.Version(2)
    assert V("1.0.0-rc.2") < V("1.0.0-rc.10") and str(V("0.3.1-dev.4")) == "0.3.1-dev.4"
    with pytest.raises(ValueError):
        V("one.two")
    ok = lambda spec, v: R.Requirement(spec).matches(V(v))
    assert ok("^1.2.3", "1.9.0") and not ok("^1.2.3", "2.0.0") and not ok("^1.2.3", "1.2.2")
    assert ok("^0.2.3", "0.2.9") and not ok("^0.2.3", "0.3.0") and ok("^0.0.3", "0.0.3") and not ok("^0.0.3", "0.0.4")
    assert ok("~1.2.3", "1.2.9") and not ok("~1.2.3", "1.3.0") and ok("~1", "1.9.9") and ok("1.2", "1.5.0") and not ok("1.2", "2.0.0")
    assert ok(">=1.0, <2.0", "1.5.0") and not ok(">=1.0, <2.0", "2.0.0") and ok("*", "9.9.9") and ok("==1.4.0", "1.4.0") and not ok("=1.4.0", "1.4.1")
    assert not ok("^1.0", "1.1.0-rc.1") and ok(">=1.1.0-rc.1", "1.1.0-rc.2")
    idx = R.PackageIndex({
        "vision": {"1.0.0": {"core": "^1.0"}, "1.1.0": {"core": "^1.2"}, "2.0.0": {"core": "^2.0"}},
        "text": {"0.9.0": {"core": ">=1.0, <1.3"}, "1.0.0": {"core": "^1.3", "tokenizers": "~0.4"}},
        "tokenizers": {"0.4.2": {}, "0.5.0": {}},
        "core": {"1.0.0": {}, "1.2.5": {}, "1.3.0": {}, "2.0.0": {}},
    })
    sol = R.resolve(idx, {"vision": "^1", "text": "*"})
    assert sol == {"core": "1.3.0", "text": "1.0.0", "tokenizers": "0.4.2", "vision": "1.1.0"}
    # a pin on core forces backtracking to older releases of both dependants
    sol2 = R.resolve(idx, {"vision": "^1", "text": "*", "core": "<1.3"})
    assert sol2 == {"core": "1.2.5", "text": "0.9.0", "vision": "1.1.0"}
    with pytest.raises(R.ResolutionError) as ei:
        R.resolve(idx, {"vision": "^2", "text": "*"})
    assert "core" in str(ei.value)
    with pytest.raises(R.ResolutionError) as ei:
        R.resolve(idx, {"audio": "*"})
    assert "unknown package 'audio'" in str(ei.value)
    lock = R.write_lock(sol, idx)
    assert R.check_lock(lock, idx, {"vision": "^1", "text": "*"}) == []
    assert any("violates the root requirement" in p for p in R.check_lock(lock, idx, {"vision": "^2", "text": "*"}))
    del idx.releases["tokenizers"][V("0.4.2")]
    assert any("no longer in the index" in p for p in R.check_lock(lock, idx, {"vision": "^1", "text": "*"}))
    old = {"name": "m", "version": "0.3.0", "dependencies": ["core==1.2.5", "text"], "format": 1}
    new = R.migrate_manifest(old)
    assert new["format"] == 2 and new["dependencies"] == {"core": "==1.2.5", "text": "*"} and new["requires_torsh"] == "*" and old["format"] == 1
    assert R.migrate_manifest(new) == new
    with pytest.raises(ValueError):
        R.migrate_manifest({"name": "x", "format": 9})


def test_extended_metrics_against_sklearn_and_scipy():
    import math
    skm = pytest.importorskip("sklearn.metrics")
    sst = pytest.importorskip("scipy.stats")
    from torsh_b200.utils import metrics_ext as M
    torch.manual_seed(0)
    y = torch.randint(0, 4, (300,))
    p = torch.where(torch.rand(300) < 0.7, y, torch.randint(0, 4, (300,)))
    assert M.matthews_corrcoef(p, y) == pytest.approx(skm.matthews_corrcoef(y.numpy(), p.numpy()), abs=1e-9)
    assert M.cohen_kappa(p, y) == pytest.approx(skm.cohen_kappa_score(y.numpy(), p.numpy()), abs=1e-9)
    assert M.balanced_accuracy(p, y) == pytest.approx(skm.balanced_accuracy_score(y.numpy(), p.numpy()), abs=1e-9)
    yb = (torch.rand(200) < 0.3).long()
    s = (yb.float() * 0.3 + torch.rand(200) * 0.7).round(decimals=2)        # ties included
    assert M.average_precision(s, yb) == pytest.approx(skm.average_precision_score(yb.numpy(), s.numpy()), abs=1e-9)
    pr = torch.softmax(torch.randn(300, 4), -1)
    assert M.log_loss(pr, y) == pytest.approx(skm.log_loss(y.numpy(), pr.numpy(), labels=[0, 1, 2, 3]), abs=1e-6)
    assert M.log_loss(s.clamp(0.01, 0.99), yb) == pytest.approx(skm.log_loss(yb.numpy(), s.clamp(0.01, 0.99).numpy()), abs=1e-6)
    assert M.brier_score(s, yb) == pytest.approx(skm.brier_score_loss(yb.numpy(), s.numpy()), abs=1e-6)
    rel = torch.tensor([0, 1, 0, 1, 1, 0])
    assert M.precision_at_k(rel, 3) == pytest.approx(1 / 3) and M.recall_at_k(rel, 4) == pytest.approx(2 / 3) and M.hit_rate_at_k(rel, 1) == 0.0
    assert M.reciprocal_rank(rel) == 0.5 and M.mean_reciprocal_rank([rel, torch.tensor([1, 0]), torch.tensor([0, 0])]) == pytest.approx(0.5)
    assert M.average_precision_at_k(rel) == pytest.approx((1 / 2 + 2 / 4 + 3 / 5) / 3) and M.mean_average_precision([rel, torch.zeros(3)]) == pytest.approx(M.average_precision_at_k(rel) / 2)
    t = torch.randn(100) * 3 + 5
    pd = t + 0.3 * torch.randn(100)
    assert M.explained_variance(pd, t) == pytest.approx(skm.explained_variance_score(t.numpy(), pd.numpy()), abs=1e-6)
    assert M.mape(pd, t) == pytest.approx(skm.mean_absolute_percentage_error(t.numpy(), pd.numpy()), rel=1e-6)
    r2 = skm.r2_score(t.numpy(), pd.numpy())
    assert M.adjusted_r2(pd, t, 3) == pytest.approx(1 - (1 - r2) * 99 / 96, abs=1e-6) and 0 < M.smape(pd, t) < 0.2
    diag = M.residual_diagnostics(pd, t)
    assert 1.0 < diag["durbin_watson"] < 3.0 and abs(diag["skewness"]) < 1 and diag["std"] == pytest.approx(0.3, rel=0.3)
    conf = torch.tensor([0.95, 0.9, 0.85, 0.6, 0.55, 0.52])
    corr = torch.tensor([1, 1, 1, 1, 0, 0])
    assert M.calibration_error(conf, corr, n_bins=2) == pytest.approx(abs(4 / 6 - 4.37 / 6), abs=1e-6)       # all six fall in the upper bin: accuracy 4/6 against mean confidence 4.37/6
    assert M.calibration_error(conf, corr, n_bins=10, norm="max") >= M.calibration_error(conf, corr, n_bins=10)
    lo, hi = t - 1, t + 1
    assert M.interval_coverage(lo, hi, pd) > 0.95 and M.interval_sharpness(lo, hi) == pytest.approx(2.0)
    assert M.gaussian_nll(t, torch.ones(100), t) == pytest.approx(0.5 * math.log(2 * math.pi))
    mc = torch.softmax(torch.randn(8, 5, 3), -1)
    assert (M.mutual_information(mc) >= -1e-9).all() and torch.allclose(M.mutual_information(mc[:1].expand(8, 5, 3)), torch.zeros(5, dtype=torch.float64), atol=1e-9)
    train = torch.arange(20.)
    assert M.mase(torch.tensor([21., 22.]), torch.tensor([20., 21.]), train) == pytest.approx(1.0)
    assert M.directional_accuracy(torch.tensor([1., 2., 1.]), torch.tensor([1., 2., 3.])) == 0.5 and M.theil_u(t, t) == 0.0
    assert M.aic(-10.0, 3) == 26.0 and M.bic(-10.0, 3, 100) == pytest.approx(3 * math.log(100) + 20)
    folds = M.k_fold_indices(10, 3)
    assert [len(v) for _, v in folds] == [4, 3, 3] and sorted(torch.cat([v for _, v in folds]).tolist()) == list(range(10))
    sf = M.stratified_k_fold_indices(torch.tensor([0] * 6 + [1] * 3), 3)
    assert all(sorted(torch.tensor([0] * 6 + [1] * 3)[v].tolist()) == [0, 0, 1] for _, v in sf)
    a, b = torch.randn(500, 6), torch.randn(500, 6) + 0.5
    assert M.frechet_distance(a, a) == pytest.approx(0.0, abs=1e-6) and 1.0 < M.frechet_distance(a, b) < 2.2
    assert M.inception_score(torch.eye(4)) == pytest.approx(4.0, rel=1e-6) and M.inception_score(torch.full((5, 4), 0.25)) == pytest.approx(1.0)
    rm, parts = M.RunningMoments(), torch.randn(1000).split(137)
    for part in parts:
        rm.update(part)
    allv = torch.cat(parts).double()
    assert rm.n == 1000 and rm.mean == pytest.approx(float(allv.mean()), abs=1e-12) and rm.variance == pytest.approx(float(allv.var()), rel=1e-10)
    merged = M.RunningMoments().update(parts[0]).merge(M.RunningMoments().update(torch.cat(parts[1:])))
    assert merged.variance == pytest.approx(rm.variance, rel=1e-10)
    sc = M.StreamingConfusion(4)
    for i in range(0, 300, 64):
        sc.update(p[i:i + 64], y[i:i + 64])
    assert sc.accuracy() == pytest.approx(float((p == y).float().mean())) and sc.f1_macro() == pytest.approx(skm.f1_score(y.numpy(), p.numpy(), average="macro"), abs=1e-9)
    sa = M.StreamingAUC(4096)
    for i in range(0, 200, 50):
        sa.update(s[i:i + 50], yb[i:i + 50])
    assert sa.compute() == pytest.approx(skm.roc_auc_score(yb.numpy(), s.numpy()), abs=2e-3)
    x1, x2 = torch.randn(40) + 0.4, torch.randn(40)
    tt = M.paired_t_test(x1, x2)
    ref = sst.ttest_rel(x1.numpy(), x2.numpy())
    assert tt["t"] == pytest.approx(ref.statistic, rel=1e-6) and tt["p_value"] == pytest.approx(ref.pvalue, rel=1e-5)
    ca, cb = torch.rand(200) < 0.8, torch.rand(200) < 0.7
    mc_ = M.mcnemar_test(ca, cb)
    assert mc_["statistic"] == pytest.approx((abs(mc_["b"] - mc_["c"]) - 1) ** 2 / (mc_["b"] + mc_["c"])) and 0 <= mc_["p_value"] <= 1
    wx = M.wilcoxon_signed_rank(x1, x2)
    refw = sst.wilcoxon(x1.numpy(), x2.numpy(), correction=False, mode="approx")
    assert wx["statistic"] == pytest.approx(refw.statistic) and wx["p_value"] == pytest.approx(refw.pvalue, rel=1e-6)
    lo_, hi_ = M.bootstrap_ci(x1, n_boot=1000)
    assert lo_ < float(x1.mean()) < hi_ and hi_ - lo_ < 1.0
    assert M.permutation_test(torch.randn(30) + 2, torch.randn(30), n_perm=500) < 0.01 and M.permutation_test(x2, x2.flip(0), n_perm=200) > 0.5
    scorer = M.make_scorer(lambda pr_, y_: (pr_ == y_).float().mean())
    assert scorer(lambda X: torch.nn.functional.one_hot(X, 4).float(), y, y) == 1.0


def test_profiler_analysis_workload_online_learning_regression_reports_streaming_and_flamegraphs(tmp_path):
    import asyncio
    import json
    import math
    import zlib
    import numpy as np
    from torsh_b200.utils import profiler_analysis as PA
    from torsh_b200.utils.profiler import ProfileEvent
    rng = np.random.default_rng(0)
    # workload characterisation
    ev, t = [], 0.0
    for i in range(60):                                                     # memory-bound element-wise phase, then a communication phase
        ev.append(ProfileEvent("add", "op", t, 10.0, 1, flops=1e6, bytes=1.2e7)); t += 12.0
    for i in range(60):
        ev.append(ProfileEvent("all_reduce", "communication", t, 50.0, 1)); t += 50.0
    wc = PA.WorkloadCharacterizer(window=30)
    rep = wc.analyze(ev)
    assert rep["workload_type"] == "communication_bound" and [p["dominant"] for p in rep["phases"]] == ["op", "communication"] and rep["hotspots"][0][0] == "all_reduce"
    mem = wc.analyze(ev[:60])
    assert mem["workload_type"] == "memory_bound" and mem["idle_fraction"] == pytest.approx(1 - 600 / 718, abs=1e-6) and mem["parallelism"] == pytest.approx(1.0)
    gemm = [ProfileEvent("gemm", "op", i * 100.0, 100.0, 1, flops=1.2e11, bytes=1e8) for i in range(10)]
    cb = wc.analyze(gemm)
    assert cb["workload_type"] == "compute_bound" and cb["mean_compute_efficiency"] == pytest.approx(1.2e11 / 1e-4 / 1.4e15)
    par = wc.analyze([{"name": "a", "category": "op", "start_us": 0, "duration_us": 100}, {"name": "b", "category": "op", "start_us": 0, "duration_us": 100}])
    assert par["parallelism"] == pytest.approx(2.0) and wc.analyze([])["workload_type"] == "empty"
    length, path = PA.WorkloadCharacterizer.critical_path({"load": 2, "fwd": 5, "aug": 1, "bwd": 7, "log": 1}, {"fwd": ["load", "aug"], "bwd": ["fwd"], "log": ["fwd"]})
    assert length == 14 and path == ["load", "fwd", "bwd"]
    # learned analysis
    ml = PA.MLAnalyzer()
    names, feats = ml.extract_features(ev)
    assert names == ["add", "all_reduce"] and feats.shape == (2, 7) and feats[1, 4] == pytest.approx(3000 / 3600)
    vals = list(rng.normal(100, 2, 200)); vals[50] = 160; vals[120] = 30
    for m in ("mad", "zscore", "iqr"):
        assert {50, 120} <= set(ml.detect_anomalies(vals, m, 3.5 if m != "zscore" else 4.0)), m
    three = np.concatenate([rng.normal([10, 1e3, 1, 1, .1, 1e6, 1e6], 0.01, (8, 7)), rng.normal([1e3, 10, 1, 1, .1, 1e9, 1e3], 0.01, (8, 7)), rng.normal([1, 1, 50, 90, .5, 10, 1e9], 0.01, (8, 7))])
    lab = ml.cluster_operations(np.abs(three), 3)
    assert len(set(lab[:8])) == len(set(lab[8:16])) == len(set(lab[16:])) == 1 and len(set(lab)) == 3
    fl, by = rng.uniform(1e9, 1e12, 200), rng.uniform(1e6, 1e9, 200)
    dur = (fl / 1e15 + by / 5e12 + 4e-6) * 1e6 * rng.normal(1, 0.01, 200)
    fit = ml.fit_duration_model(fl, by, dur)
    assert fit["flops_per_s"] == pytest.approx(1e15, rel=0.05) and fit["bytes_per_s"] == pytest.approx(5e12, rel=0.05) and fit["overhead_s"] == pytest.approx(4e-6, rel=0.3) and fit["r2"] > 0.99
    assert fit["predict"](1e12, 1e9) == pytest.approx(1e-3 + 2e-4 + 4e-6, rel=0.05)
    # online statistics
    os_ = PA.OnlineStats()
    for v in vals:
        os_.update(v)
    assert os_.mean == pytest.approx(np.mean(vals)) and os_.std == pytest.approx(np.std(vals, ddof=1)) and os_.max == 160
    ew = PA.EWMA(0.5)
    assert [ew.update(v) for v in (4, 8, 8)] == [4, 6, 7]
    ad = PA.OnlineAnomalyDetector(4.0, 20)
    flags = [ad.update(v) for v in vals]
    assert [i for i, f in enumerate(flags) if f] == [50, 120] and ad.events[0]["kind"] == "spike" and ad.events[1]["kind"] == "drop"
    dd = PA.DriftDetector(30, 5.0)
    hits = [i for i, v in enumerate(list(rng.normal(10, 1, 100)) + list(rng.normal(14, 1, 100))) if dd.update(v)]
    assert len(hits) >= 1 and 100 <= hits[0] <= 135
    sk = PA.StreamingKMeans(2)
    for p in rng.permutation(np.concatenate([rng.normal(0, 0.1, (100, 2)), rng.normal(5, 0.1, (100, 2))])):
        sk.update(p)
    assert len(sk.centroids) == 2 and sum(sk.counts) == 200
    op = PA.OnlinePredictor(2)
    for _ in range(300):
        x = rng.uniform(0, 1, 2)
        op.update(x, 3 * x[0] - 2 * x[1] + 0.5)
    assert op.predict([1.0, 1.0]) == pytest.approx(1.5, abs=1e-3) and op.abs_err.value < 1e-3
    # memory forecasting and pools
    mp = PA.MemoryUsagePredictor()
    for i in range(32):
        mp.record(float(i), 1000.0 + 50 * i + (20 if i % 7 == 0 else 0))
    assert mp.predict(40.0) == pytest.approx(1000 + 50 * 40, rel=0.02) and mp.time_to_limit(4000.0) == pytest.approx((4000 - 1000) / 50 - 31, abs=1.0) and mp.leak_suspected(min_slope=10)
    flat = PA.MemoryUsagePredictor()
    for i in range(32):
        flat.record(float(i), 1000.0 + rng.normal(0, 5))
    assert not flat.leak_suspected(min_slope=10) and flat.time_to_limit(1e9) is None or flat.time_to_limit(1e9) > 1e4
    pool = PA.AdaptivePoolManager()
    assert pool.size_class(1000) == 1024 and pool.size_class(10) == 256
    for _ in range(3):
        blocks = [pool.allocate(1000) for _ in range(8)]
        for b in blocks:
            pool.release(1000)
    assert pool.stats()["hit_rate"] == pytest.approx(16 / 24) and pool.stats()["cached_bytes"] == 8 * 1024
    pool.allocate(1000); pool.release(1000)
    assert pool.trim() == 0                                                 # peak of 8 still justifies the cache
    pool.allocate(1000); pool.release(1000)
    assert pool.trim() == (8 - 2) * 1024                                    # demand fell to one block: keep ceil(1 * 1.25) = 2
    # low-overhead recorder
    oprof = PA.OptimizedProfiler(capacity=100, sample_every=10)
    for i in range(1000):
        oprof.record("k", float(i), 5.0)
    for i in range(30):
        oprof.record("rare", float(i), 100.0)
    st = oprof.stats()
    assert st["recorded"] == 1030 and st["stored"] == 100 and st["dropped"] == 3 and st["names"] == 2 and st["overhead_per_record_s"] < 1e-3
    assert oprof.estimated_totals() == {"k": 5000.0, "rare": 3000.0} and oprof.events()[-1]["name"] == "rare"
    # regression detection
    rd = PA.RegressionDetector()
    base = list(rng.normal(100, 1, 30))
    rd.set_baseline("step_ms", base)
    assert not rd.check("step_ms", list(rng.normal(100.5, 1, 30)))["regression"]
    assert rd.check("step_ms", list(rng.normal(110, 1, 30)))["severity"] == "minor" and rd.check("step_ms", list(rng.normal(130, 1, 30)))["severity"] == "major"
    assert rd.check("step_ms", list(rng.normal(170, 1, 30)))["severity"] == "critical" and rd.check("step_ms", list(rng.normal(80, 1, 30)))["improvement"]
    rd.save(tmp_path / "b.json")
    rd2 = PA.RegressionDetector(higher_is_better=True); rd2.load(tmp_path / "b.json")
    assert rd2.check("step_ms", list(rng.normal(80, 1, 30)))["severity"] == "major"
    # reports
    te = PA.TemplateEngine()
    assert te.render("{{ a.b }}|{{{ a.b }}}|{% for r in rows %}[{{ r.x }}]{% endfor %}", {"a": {"b": "<x>"}, "rows": [{"x": 1}, {"x": 2}]}) == "&lt;x&gt;|<x>|[1][2]"
    rg = PA.ReportGenerator()
    r = rg.build(ev, "Run 7")
    assert r["rows"][0]["name"] == "all_reduce" and r["rows"][0]["share"] == "83.3%" and r["summary"] == {"events": 120, "total_ms": 3.6} and "all_reduce takes" in r["findings"][0]["text"]
    assert "<td>all_reduce</td><td>60</td>" in rg.render(r, "html") and "| add | 60 | 0.6 | 16.7% |" in rg.render(r, "markdown") and json.loads(rg.render(r, "json"))["rows"][1]["calls"] == 60
    assert rg.build(ev, category="op")["summary"]["events"] == 60 and rg.build(ev, since_us=720)["summary"]["events"] == 60
    # streaming with a slow link: quality steps down, low priority is dropped first, frames decode
    frames = []
    def send(frame):
        frames.append(frame)
        return 0.2                                                          # a link that takes 200 ms per frame
    es = PA.EventStreamer(send, capacity=300, target_latency=0.05)
    for i in range(1000):
        es.push({"name": "tick", "i": i, "payload": "x" * 40}, priority=1 if i % 100 else 3)
    assert len(es.heap) == 300 and es.dropped == 700 and sum(1 for p, _, _ in es.heap if p == 3) == 10
    assert es.flush() >= 2 and es.stats()["quality"] != "full" and es.stats()["compression_ratio"] < 0.3
    first = json.loads(zlib.decompress(frames[0]))
    assert all(e["i"] % 100 == 0 for e in first[:10]) and es.stats()["sent"] == 300
    before = es.dropped
    for i in range(200):
        es.push({"i": i}, priority=1)
    assert es.dropped > before                                               # reduced quality samples low-priority events
    # custom export and tools
    ce = PA.CustomExporter()
    schema = [{"header": "op", "field": "name"}, {"header": "ms", "field": "duration_us", "format": "ms"}, {"header": "MiB", "field": "bytes", "format": "mib"}, {"header": "f", "field": "flops", "format": "%.1e"}]
    csv = ce.export(ev[:2] + [{"name": 'a,"b"', "duration_us": 1500.0, "bytes": 1 << 20, "flops": 0.0}], schema)
    assert csv.splitlines()[0] == "op,ms,MiB,f" and csv.splitlines()[1] == "add,0.010,11.44,1.0e+06" and csv.splitlines()[3] == '"a,""b""",1.500,1.00,0.0e+00'
    assert ce.export(ev[:1], schema, "text").splitlines()[1].split() == ["add", "0.010", "11.44", "1.0e+06"] and "\t" in ce.export(ev[:1], schema, "tsv")
    reg = PA.CustomToolRegistry()
    reg.register("count", lambda evs, scale=1: len(evs) * scale, scale=2)
    reg.register("boom", lambda evs: 1 / 0)
    assert reg.run("count", ev) == 240 and reg.list_tools() == ["boom", "count"]
    with pytest.raises(ZeroDivisionError):
        reg.run_all(ev)
    assert reg.stats["boom"] == {"calls": 1, "seconds": reg.stats["boom"]["seconds"], "errors": 1}
    # flame graph
    nested = [{"name": "step", "start_us": 0, "duration_us": 100, "thread_id": 1}, {"name": "fwd", "start_us": 5, "duration_us": 40, "thread_id": 1},
              {"name": "gemm", "start_us": 10, "duration_us": 30, "thread_id": 1}, {"name": "bwd", "start_us": 50, "duration_us": 45, "thread_id": 1},
              {"name": "io", "start_us": 0, "duration_us": 20, "thread_id": 2}]
    stacks = PA.build_stacks(nested)
    assert stacks == {"step": 15.0, "step;fwd": 10.0, "step;fwd;gemm": 30.0, "step;bwd": 45.0, "io": 20.0} and "step;fwd;gemm 30\n" in PA.folded_text(stacks)
    ss = json.loads(PA.speedscope_json(stacks))
    assert ss["profiles"][0]["endValue"] == 120 and {f["name"] for f in ss["shared"]["frames"]} == {"step", "fwd", "gemm", "bwd", "io"}
    # decorators
    ar = PA.AttributeRegistry()
    @ar.profile(category="math", tag="t")
    def work(n): return sum(range(n))
    @ar.profile_if(lambda n: n > 5, name="big")
    def maybe(n): return n
    @ar.profile()
    async def aw(n):
        await asyncio.sleep(0)
        return n * 2
    assert work(10) == 45 and maybe(3) == 3 and maybe(9) == 9 and asyncio.run(aw(4)) == 8
    assert [e["name"] for e in ar.events] == [work.__qualname__, "big", aw.__qualname__] and ar.events[0]["category"] == "math" and ar.events[0]["tag"] == "t"
    # integrated
    det = PA.RegressionDetector(); det.set_baseline("matmul", list(rng.normal(100, 1, 30)))
    ip = PA.IntegratedProfiler(regression=det)
    tt = 0.0
    for i in range(200):
        d = float(rng.normal(125, 1)) if i != 150 else 400.0
        ip.record({"name": "matmul", "category": "op", "start_us": tt, "duration_us": d}); tt += d
    ip.pause(); ip.record({"name": "ignored", "category": "op", "start_us": tt, "duration_us": 1.0}); ip.resume()
    out = ip.report()
    assert out["events"] == 200 and len(out["anomalies"]["matmul"]) == 1 and out["regressions"][0]["severity"] == "major" and out["trends"]["matmul"] == pytest.approx(125, abs=15)
    assert any("slower than its baseline" in r for r in out["recommendations"]) and any("outlier" in r for r in out["recommendations"])


def test_mobile_optimizer_and_bottleneck_profiler(tmp_path):
    from torsh_b200.utils import mobile_optimizer as M
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.BatchNorm2d(8), torch.nn.ReLU(), torch.nn.Dropout(0.3), torch.nn.Flatten(),
                              torch.nn.Linear(8 * 8 * 8, 64), torch.nn.ReLU(), torch.nn.Linear(64, 10)).eval()
    net[1].running_mean.normal_(); net[1].running_var.uniform_(0.5, 2)
    x = torch.randn(4, 3, 8, 8)
    opt, rep = M.optimize_for_mobile(net, M.MobileOptimizerConfig("android"), x)
    steps = {s["step"]: s for s in rep["steps"]}
    assert steps["remove_dropout"]["removed"] == 1 and steps["fold_batch_norm"]["folded"] == 1 and steps["fold_batch_norm"]["relative_error"] < 1e-5
    assert steps["dynamic_int8"]["layers"] == 2 and steps["dynamic_int8"]["relative_error"] < 0.03 and 3.0 < rep["compression"] < 4.1 and rep["fits_platform"]
    assert isinstance(opt[5], M.Int8DynamicLinear) and opt[5].qweight.dtype == torch.int8 and torch.allclose(opt(x), net(x), atol=0.05)
    ios, r2 = M.optimize_for_mobile(net, M.MobileOptimizerConfig("ios"), x)
    assert r2["compression"] == pytest.approx(2.0, rel=0.02) and r2["steps"][-1]["relative_error"] < 5e-3 and ios(x).dtype == torch.float32
    pr, r3 = M.optimize_for_mobile(net, M.MobileOptimizerConfig("server", prune_sparsity=0.5, size_target_mb=0.001), x)
    assert next(s for s in r3["steps"] if s["step"] == "prune")["sparsity"] == pytest.approx(0.5, abs=0.01) and not r3["fits_target"] and r3["optimized_bytes"] < r3["original_bytes"]
    keep, r4 = M.optimize_for_mobile(net, M.MobileOptimizerConfig("android", preserve_modules=("7",)), x)
    assert isinstance(keep[7], torch.nn.Linear) and isinstance(keep[5], M.Int8DynamicLinear)
    assert net[3].p == 0.3 and isinstance(net[1], torch.nn.BatchNorm2d)                                        # the source model is untouched
    out = M.export_optimized_model(opt, tmp_path / "m.pt")
    sd = torch.load(tmp_path / "m.pt")
    assert out["bytes"] < 0.4 * M.model_size_bytes(net) + 4096 and sd["5.qweight"].dtype == torch.int8
    bm = M.benchmark_mobile_model(opt, x, warmup=1, iters=5, threads=1)
    assert bm["mean_ms"] > 0 and bm["p95_ms"] >= bm["p50_ms"] and bm["threads"] == 1 and bm["model_bytes"] == M.model_size_bytes(opt)
    # bottleneck profile with a fake clock: the wide layer dominates
    wide = torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.ReLU(), torch.nn.Linear(16, 2048), torch.nn.ReLU(), torch.nn.Linear(2048, 4), torch.nn.Tanh(), torch.nn.Sigmoid())
    rep = M.profile_bottlenecks(wide, torch.randn(64, 16), iters=3)
    assert len(rep.layers) == 7 and {"2", "4"} <= {l["name"] for l in rep.layers[:4]} and rep.memory_peak_layer in ("2", "3")   # wall-clock ranking: allow for timer noise
    assert abs(sum(l["share"] for l in rep.layers) - 1) < 1e-6 and rep.total_backward_ms > 0 and "total forward" in rep.render() and rep.hotspots[0] in ("2", "4")
    fwd_only = M.profile_bottlenecks(wide, torch.randn(64, 16), iters=2, backward=False)
    assert fwd_only.total_backward_ms == 0 and all(l["backward_ms"] == 0 for l in fwd_only.layers) and wide.training


def test_hub_services_transfers_cache_cards_analytics_community_enterprise_and_imports(tmp_path):
    import json
    from torsh_b200 import hub_services as H
    torch.manual_seed(0)
    # token bucket with a fake clock
    now = [0.0]
    slept = []
    bl = H.BandwidthLimiter(1000.0, burst=500.0, clock=lambda: now[0], sleep=lambda s: (slept.append(s), now.__setitem__(0, now[0] + s)))
    assert bl.acquire(400) == 0 and bl.acquire(600) == pytest.approx(0.5) and bl.acquire(1000) == pytest.approx(1.0) and sum(slept) == pytest.approx(1.5)
    now[0] += 10
    assert bl.acquire(500) == 0 and bl.stats()["bytes"] == 2500
    import os
    (tmp_path / "blob.bin").write_bytes(os.urandom(300_000))
    rd = H.BandwidthLimitedReader(open(tmp_path / "blob.bin", "rb"), H.BandwidthLimiter(1e9, sleep=None))
    assert sum(len(c) for c in rd) == 300_000
    ab = H.AdaptiveBandwidthLimiter(1000.0, min_rate=100, window=2, sleep=None)
    ab.report(True); ab.report(True)
    assert ab.rate == pytest.approx(1100.0)
    ab.report(False)
    assert ab.rate == pytest.approx(550.0)
    # retry with back-off and circuit breaker
    waits, calls = [], [0]
    rp = H.RetryPolicy(max_attempts=4, base_delay=1.0, jitter=0.0, breaker_threshold=2, breaker_cooldown=30.0, clock=lambda: now[0], sleep=waits.append)
    def flaky():
        calls[0] += 1
        if calls[0] < 3:
            raise IOError("reset")
        return "ok"
    assert rp.call(flaky) == "ok" and waits == [1.0, 2.0] and rp.attempts_log == [3]
    def dead(): raise TimeoutError("no route")
    for _ in range(2):
        with pytest.raises(TimeoutError):
            rp.call(dead)
    with pytest.raises(ConnectionError):
        rp.call(flaky)
    now[0] += 31
    assert rp.call(flaky) == "ok"
    with pytest.raises(ValueError):
        H.RetryPolicy(sleep=lambda s: None).call(lambda: (_ for _ in ()).throw(ValueError("not retried")))
    # resumable verified download
    src = tmp_path / "blob.bin"
    digest = H._sha256(src)
    dm = H.DownloadManager(chunk=50_000)
    (tmp_path / "out").mkdir()
    (tmp_path / "out" / "m.bin.part").write_bytes(src.read_bytes()[:120_000])
    rec = dm.download(f"file://{src}", tmp_path / "out" / "m.bin", digest)
    assert rec["resumed_from"] == 120_000 and (tmp_path / "out" / "m.bin").read_bytes() == src.read_bytes() and not (tmp_path / "out" / "m.bin.part").exists()
    with pytest.raises(IOError):
        dm.download(src, tmp_path / "out" / "bad.bin", "0" * 64)
    assert not (tmp_path / "out" / "bad.bin").exists() and not (tmp_path / "out" / "bad.bin.part").exists()
    with pytest.raises(PermissionError):
        dm.download("https://example.org/m.bin", tmp_path / "x")
    fails = [0]
    class Flaky:
        def __init__(self, p, mode): self.f = open(p, mode)
        def __enter__(self): return self
        def __exit__(self, *a): self.f.close()
        def seek(self, n): self.f.seek(n)
        def read(self, n):
            fails[0] += 1
            if fails[0] == 3:
                raise IOError("connection reset")
            return self.f.read(n)
    rec = dm.download(src, tmp_path / "out" / "r.bin", digest, opener=Flaky)
    assert rec["attempts"] == 2 and (tmp_path / "out" / "r.bin").read_bytes() == src.read_bytes()
    # cache
    t = [0.0]
    cm = H.CacheManager(tmp_path / "cache", max_bytes=700_000, clock=lambda: t[0])
    for k in ("a", "b"):
        t[0] += 1; cm.put(k, src)
    t[0] += 1
    assert cm.get("a") is not None and cm.get("zzz") is None
    t[0] += 1; cm.put("c", src)
    assert sorted(cm.index) == ["a", "c"] and cm.total_bytes() == 600_000 and cm.stats()["hit_rate"] == 0.5
    (tmp_path / "cache" / cm.index["a"]["file"]).write_bytes(b"corrupt")
    (tmp_path / "cache" / "stray.tmp").write_bytes(b"x")
    v = cm.validate()
    assert v["corrupt"] == ["a"] and v["untracked"] == ["stray.tmp"]
    t[0] += 100
    cl = cm.cleanup(max_age_s=50)
    assert sorted(cl["removed"]) == ["a", "c"] and cl["untracked_removed"] == ["stray.tmp"] and cm.stats()["entries"] == 0
    assert H.CacheManager(tmp_path / "cache").index == {}
    # model cards and search
    reg = H.ModelRegistry()
    mk = lambda n, v, task, tags, acc, params, lic="apache-2.0": H.ModelCard(n, v, task, "Net", lic, f"{n} for {task}", tags, {"accuracy": acc}, params)
    for c in (mk("org/resnet50", "1.0.0", "image-classification", ["vision", "cnn"], 0.76, 25_000_000), mk("org/resnet50", "1.2.0", "image-classification", ["vision", "cnn"], 0.80, 25_000_000),
              mk("org/vit-b", "1.0.0", "image-classification", ["vision", "transformer"], 0.84, 86_000_000), mk("org/gpt2", "1.0.0", "text-generation", ["nlp", "transformer"], 0.3, 124_000_000, "mit")):
        reg.register(c)
    assert reg.versions("org/resnet50") == ["1.0.0", "1.2.0"] and reg.latest("org/resnet50").metrics["accuracy"] == 0.80
    assert [c.name for c in reg.search("transformer")] == ["org/vit-b", "org/gpt2"] or [c.name for c in reg.search("transformer")] == ["org/gpt2", "org/vit-b"]
    assert [c.name for c in reg.search(task="image-classification", max_parameters=50_000_000, sort_by="accuracy")] == ["org/resnet50", "org/resnet50"]
    assert [c.version for c in reg.search("resnet", min_metric=("accuracy", 0.78))] == ["1.2.0"] and [c.name for c in reg.search(license="mit")] == ["org/gpt2"] and reg.search("nothing-like-this") == []
    with pytest.raises(ValueError):
        reg.register(H.ModelCard("x", "one"))
    card = H.ModelCard.from_model("org/tiny", torch.nn.Linear(4, 2), task="regression", license="mit", description="d", metrics={"mse": 0.1}, limitations="small")
    assert card.parameters == 10 and "| mse | 0.1 |" in card.to_markdown() and "## Limitations" in card.to_markdown() and card.validate() == []
    # analytics and A/B
    an = H.AnalyticsManager(clock=lambda: t[0])
    for i in range(10):
        t[0] = 86400.0 * (i // 5)
        an.record("download", "org/gpt2", f"u{i % 3}")
        an.record("inference", "org/gpt2", f"u{i % 3}", latency_ms=10.0 + i)
    an.record("error", "org/gpt2", "u0"); an.record("download", "org/vit-b", "u1")
    s = an.summary("org/gpt2")
    assert s["events"] == 21 and s["unique_users"] == 3 and s["by_kind"]["download"] == 10 and s["p50_latency_ms"] == 15.0 and s["error_rate"] == pytest.approx(1 / 21)
    assert an.popular(1) == [("org/gpt2", 10)] and an.trend("org/gpt2") == [(0.0, 5), (86400.0, 5)]
    an.export(tmp_path / "ev.jsonl")
    assert len((tmp_path / "ev.jsonl").read_text().splitlines()) == 22
    abt = H.ABTest("ranker", {"control": 1, "new": 1})
    g = torch.Generator().manual_seed(0)
    for i in range(4000):
        u = f"user{i}"
        p = 0.10 if abt.assign(u) == "control" else 0.16
        abt.record(u, float(torch.rand((), generator=g) < p))
    res = abt.result("control", "new")
    assert abt.assign("user7") == abt.assign("user7") and 0.45 < res["n"]["new"] / 4000 < 0.55 and res["significant"] and res["winner"] == "new" and 0.3 < res["lift"] < 1.0
    same = H.ABTest("noop", {"a": 1, "b": 1})
    for i in range(2000):
        same.record(f"u{i}", float(torch.rand((), generator=g) < 0.2))
    assert same.result("a", "b")["winner"] is None
    # community
    cmn = H.CommunityManager()
    for i in range(6):
        cmn.rate("org/gpt2", f"u{i}", 5)
    cmn.rate("org/gpt2", "u0", 4)
    with pytest.raises(ValueError):
        cmn.rate("org/gpt2", "u9", 6)
    root = cmn.comment("org/gpt2", "u1", "works well")
    r1 = cmn.comment("org/gpt2", "u2", "agreed", parent=root); cmn.comment("org/gpt2", "u3", "other topic"); cmn.comment("org/gpt2", "u1", "thanks", parent=r1)
    assert [c["text"] for c in cmn.thread("org/gpt2", root)] == ["works well", "agreed", "thanks"]
    cmn.downloads["org/gpt2"] = 1500
    assert cmn.stats("org/gpt2")["mean_rating"] == pytest.approx(29 / 6) and cmn.badges("org/gpt2") == ["popular", "well_rated"]
    cmn.create_challenge("fastest", "latency_ms", higher_is_better=False, deadline=100.0)
    cmn.submit("fastest", "ann", "m1", 12.0, now=1.0); cmn.submit("fastest", "bob", "m2", 9.0, now=2.0); cmn.submit("fastest", "ann", "m3", 8.0, now=3.0)
    assert [(s["user"], s["score"]) for s in cmn.leaderboard("fastest")] == [("ann", 8.0), ("bob", 9.0)]
    with pytest.raises(PermissionError):
        cmn.submit("fastest", "eve", "m4", 1.0, now=101.0)
    # enterprise
    em = H.EnterpriseManager()
    em.create_tenant("acme", storage_quota=1000, monthly_requests=2)
    em.add_user("acme", "dev", "developer", "internal"); em.add_user("acme", "boss", "admin", "restricted")
    em.label_model("secret-model", "confidential")
    assert em.authorize("acme", "dev", "write") and not em.authorize("acme", "dev", "delete") and not em.authorize("acme", "dev", "read", "secret-model")
    assert em.authorize("acme", "boss", "read", "secret-model") and not em.authorize("acme", "ghost", "read") and not em.authorize("other", "dev", "read")
    em.charge_storage("acme", 800)
    with pytest.raises(PermissionError):
        em.charge_storage("acme", 300)
    em.charge_request("acme"); em.charge_request("acme")
    with pytest.raises(PermissionError):
        em.charge_request("acme")
    assert em.usage_report("acme") == {"storage": 0.8, "requests": 1.0, "users": 2}
    # imports and visualisation
    from torsh_b200 import onnx_io
    lin = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.ReLU())
    onnx_io.export_onnx(lin, (torch.randn(1, 4),), tmp_path / "m.onnx")
    xin = torch.randn(5, 4)
    got = H.load_onnx_model(tmp_path / "m.onnx")(xin)
    got = got[0] if isinstance(got, (list, tuple)) else got
    assert torch.allclose(torch.as_tensor(got), lin(xin), atol=1e-5)
    dense = torch.nn.Sequential()
    dense.add_module("fc", torch.nn.Linear(4, 3))
    tfw = {"fc/kernel:0": torch.randn(4, 3).numpy(), "fc/bias:0": torch.randn(3).numpy()}
    rp2 = H.import_tensorflow_checkpoint(tfw, dense)
    assert rp2["loaded"] == ["fc.bias", "fc.weight"] and torch.allclose(dense.fc.weight, torch.as_tensor(tfw["fc/kernel:0"]).t())
    tree = H.model_tree(torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Sequential(torch.nn.Linear(3, 2))))
    assert tree.splitlines()[0] == "Sequential: Sequential (23)" and "    0: Linear (8)" in tree
    assert H.sparkline([0, 1, 2, 3, 4, 5, 6, 7]) == "▁▂▃▄▅▆▇█" and H.sparkline([2, 2]) == "▁▁"
    svg = H.line_chart_svg({"train": [1.0, 0.5, 0.3], "val": [1.1, 0.7, 0.6]}, title="loss")
    assert svg.startswith("<svg") and svg.count("<polyline") == 2 and ">loss<" in svg and svg.endswith("</svg>")
    a, b = torch.nn.Linear(4, 3), torch.nn.Linear(4, 3)
    b.bias.data.copy_(a.bias.data)
    cmpm = H.compare_models(a, b)
    assert cmpm["identical"] == ["bias"] and cmpm["most_changed"][0] == "weight" and not cmpm["only_in_a"]


def test_metrics_more_rank_tests_corrections_uncertainty_faithfulness_continual_and_reports():
    import math
    import numpy as np
    from scipy import stats
    from statistics import mean
    from torsh_b200.utils import metrics_more as M
    g = torch.Generator().manual_seed(0)
    a, b, c = torch.randn(30, generator=g, dtype=torch.float64), torch.randn(25, generator=g, dtype=torch.float64) + 0.8, torch.randn(28, generator=g, dtype=torch.float64) - 0.3
    a[3] = a[7]                                                             # a tie
    mw, ref = M.mann_whitney_u(a, b), stats.mannwhitneyu(a.numpy(), b.numpy(), alternative="two-sided", method="asymptotic")
    assert mw["u"] == pytest.approx(ref.statistic) and mw["p_value"] == pytest.approx(ref.pvalue, rel=1e-9) and mw["effect_size"] > 0.3
    kw, refk = M.kruskal_wallis(a, b, c), stats.kruskal(a.numpy(), b.numpy(), c.numpy())
    assert kw["statistic"] == pytest.approx(refk.statistic) and kw["p_value"] == pytest.approx(refk.pvalue, rel=1e-8)
    scores = torch.rand(12, 4, generator=g, dtype=torch.float64); scores[:, 0] += 0.6; scores[2, 1] = scores[2, 2]
    fr, reff = M.friedman_test(scores), stats.friedmanchisquare(*scores.t().numpy())
    assert fr["statistic"] == pytest.approx(reff.statistic) and fr["p_value"] == pytest.approx(reff.pvalue, rel=1e-8) and int(fr["mean_ranks"].argmax()) == 0
    nm = M.nemenyi_test(scores)
    assert nm["critical_difference"] == pytest.approx(2.569 * math.sqrt(4 * 5 / (6 * 12))) and nm["significant"][0, 1:].any() and not nm["significant"].diagonal().any()
    d52 = torch.tensor([[0.02, 0.03], [0.01, 0.04], [0.03, 0.02], [0.02, 0.02], [0.04, 0.01]])
    t52 = M.five_by_two_cv_test(d52)
    s2 = [((x - (x + y) / 2) ** 2 + (y - (x + y) / 2) ** 2) for x, y in d52.tolist()]
    assert t52["t"] == pytest.approx(0.02 / math.sqrt(mean(s2))) and 0 < t52["p_value"] < 1
    pv = [0.001, 0.04, 0.03, 0.2, 0.012]
    from scipy.stats import false_discovery_control
    assert M.multiple_comparison_correction(pv, "bonferroni")["adjusted"].tolist() == pytest.approx([0.005, 0.2, 0.15, 1.0, 0.06])
    assert M.multiple_comparison_correction(pv, "holm")["adjusted"].tolist() == pytest.approx([0.005, 0.09, 0.09, 0.2, 0.048]) and M.multiple_comparison_correction(pv, "holm")["reject"].tolist() == [True, False, False, False, True]
    assert np.allclose(M.multiple_comparison_correction(pv, "fdr_bh")["adjusted"].numpy(), false_discovery_control(pv, method="bh"))
    assert M.effect_size(b, a) == pytest.approx((float(b.mean() - a.mean())) / math.sqrt((24 * float(b.var()) + 29 * float(a.var())) / 53)) and abs(M.effect_size(b, a, "hedges_g")) < abs(M.effect_size(b, a))
    assert M.effect_size([3, 4, 5], [0, 1, 2], "cliffs_delta") == 1.0 and M.effect_size([1, 2], [1, 2], "cliffs_delta") == 0.0
    assert M.aicc(-100.0, 3, 20) == pytest.approx(206 + 24 / 16) and M.hqic(-100.0, 3, 50) == pytest.approx(200 + 6 * math.log(math.log(50))) and M.akaike_weights([100.0, 102.0, 110.0])[0] == pytest.approx(1 / (1 + math.exp(-1) + math.exp(-5)))
    # uncertainty: members that disagree -> epistemic; members that agree on 50/50 -> aleatoric
    disagree = torch.tensor([[[0.99, 0.01]], [[0.01, 0.99]]]); unsure = torch.tensor([[[0.5, 0.5]], [[0.5, 0.5]]])
    ud, uu = M.uncertainty_decomposition(disagree), M.uncertainty_decomposition(unsure)
    assert ud["epistemic"][0] > 0.6 > 0.1 > ud["aleatoric"][0] and uu["epistemic"][0] < 1e-9 and uu["aleatoric"][0] == pytest.approx(math.log(2)) and ud["variation_ratio"][0] == 0.5
    net = torch.nn.Sequential(torch.nn.Linear(4, 16), torch.nn.ReLU(), torch.nn.Dropout(0.5), torch.nn.Linear(16, 3), torch.nn.BatchNorm1d(3)).train()
    mc = M.mc_dropout_predict(net, torch.randn(5, 4), 8)
    assert mc.shape == (8, 5, 3) and not torch.allclose(mc[0], mc[1]) and net.training and torch.allclose(mc.sum(-1), torch.ones(8, 5))
    pic = M.prediction_interval_coverage([0, 0, 0, 0], [1, 1, 1, 1], [0.5, 1.5, -0.2, 1.0])
    assert pic == {"coverage": 0.5, "mean_width": 1.0, "winkler_miss": pytest.approx(0.175)}
    sr = M.selective_risk_curve([0.9, 0.8, 0.7, 0.6], [1, 1, 0, 1])
    assert sr["risk"].tolist() == pytest.approx([0, 0, 1 / 3, 0.25]) and sr["aurc"] == pytest.approx((1 / 3 + 0.25) / 4)
    # faithfulness: the true weights are a better attribution than random ones
    wts = torch.tensor([5.0, 0.1, 3.0, 0.0, -0.2, 1.0, 0.05, 2.0])
    fn = lambda v: (wts * v).sum()
    xin = torch.ones(8)
    good, bad = M.deletion_insertion_curves(fn, xin, wts, steps=8), M.deletion_insertion_curves(fn, xin, -wts, steps=8)
    assert good["deletion_auc"] < bad["deletion_auc"] and good["insertion_auc"] > bad["insertion_auc"] and good["deletion"][0] == pytest.approx(float(wts.sum())) and good["deletion"][-1] == 0
    assert M.attribution_sparsity(torch.tensor([0.0, 0, 0, 1])) == pytest.approx(0.75) and M.attribution_sparsity(torch.ones(4)) == pytest.approx(0.0)
    clf = lambda v: torch.stack([v[:, 0], -v[:, 0]], 1)
    xs = torch.cat([torch.full((50, 2), 1.0), torch.full((50, 2), -1.0)]); ys = torch.cat([torch.zeros(50), torch.ones(50)]).long()
    rc = M.robustness_curve(clf, xs, ys, [0.0, 0.5, 1.0, 3.0, 10.0])
    assert rc["accuracy"][0] == 1.0 and rc["accuracy"][1] > rc["accuracy"][3] > 0.4 and rc["breakdown_level"] in (None, 10.0) and 0.5 < rc["auc"] < 1
    ps = M.prediction_stability(torch.tensor([[0, 1, 2, 1], [0, 1, 2, 0], [0, 1, 1, 1]]))
    assert ps["unanimous"] == 0.5 and ps["pairwise_agreement"] == pytest.approx((0.75 + 0.75 + 0.5) / 3)
    # continual learning and recommendation quality
    acc = torch.tensor([[0.9, 0.2, 0.1], [0.7, 0.85, 0.3], [0.6, 0.8, 0.9]])
    cl = M.continual_learning_metrics(acc, baseline=torch.tensor([0.1, 0.1, 0.1]))
    assert cl["average_accuracy"] == pytest.approx(2.3 / 3) and cl["forgetting"] == pytest.approx((0.3 + 0.05) / 2) and cl["backward_transfer"] == pytest.approx((-0.3 - 0.05) / 2) and cl["forward_transfer"] == pytest.approx((0.1 + 0.2) / 2)
    pop = {0: 1000, 1: 500, 2: 10, 3: 5, 4: 1}
    feats = torch.eye(5)
    head, tail = M.recommendation_quality([[0, 1], [0, 1]], pop, feats, 5), M.recommendation_quality([[2, 3], [3, 4]], pop, feats, 5)
    assert tail["novelty"] > head["novelty"] + 4 and tail["coverage"] == 0.6 > head["coverage"] == 0.4 and head["diversity"] == 1.0 and head["exposure_gini"] > tail["exposure_gini"]
    # reports
    rb = M.ReportBuilder("Study").add_table("main_results", {"ours": {"acc": 0.91, "err_%": 9.0}, "base_line": {"acc": 0.88, "err_%": 12.0}}, {"err_%": False})
    md, tex = rb.to_markdown(), rb.to_latex()
    assert "| ours | **0.910** | **9.000** |" in md and "| base_line | 0.880 | 12.000 |" in md and md.startswith("# Study")
    assert r"\textbf{0.910}" in tex and r"base\_line" in tex and r"err\_\%" in tex and tex.count(r"\\") == 3 and r"\toprule" in tex


def test_autograd_services_federated_compression_gc_planning_replay_debugger_vjp_quantum_and_recovery():
    import math
    from torsh_b200.autograd import services as S
    torch.manual_seed(0)
    dd = torch.float64
    # robust aggregation under Byzantine clients
    honest = [torch.ones(10, dtype=dd) + 0.05 * torch.randn(10, dtype=dd) for _ in range(7)]
    bad = [torch.full((10,), -50.0, dtype=dd) for _ in range(2)]
    ups = honest + bad
    target = torch.ones(10, dtype=dd)
    errs = {m: float((S.aggregate_updates(ups, method=m, f=2, trim=0.25) - target).norm()) for m in ("fedavg", "median", "trimmed_mean", "krum", "multi_krum", "norm_clipping", "geometric_median")}
    assert errs["fedavg"] > 10 and all(errs[m] < 0.5 for m in ("median", "trimmed_mean", "krum", "multi_krum", "geometric_median")) and errs["norm_clipping"] < errs["fedavg"] / 5
    assert torch.allclose(S.aggregate_updates(honest[:2], [1, 3]), 0.25 * honest[0] + 0.75 * honest[1])
    total, masked = S.secure_aggregate(honest)
    assert torch.allclose(total, sum(honest), atol=1e-9) and all((m - u).norm() > 1 for m, u in zip(masked, honest))
    total_d, _ = S.secure_aggregate(honest, dropped=[2, 5])
    assert torch.allclose(total_d, sum(h for i, h in enumerate(honest) if i not in (2, 5)), atol=1e-9)
    # federated rounds converge on shards with different local optima; FedProx keeps local models closer
    w_true = torch.tensor([1.0, -2.0, 0.5])
    clients = []
    for c in range(6):
        x = torch.randn(40, 3) + 0.3 * c
        clients.append((x, x @ w_true + 0.01 * torch.randn(40)))
    def local_train(model, data, mu=0.0, ref=None):
        x, y = data
        opt = torch.optim.SGD(model.parameters(), 0.05)
        g = {n: p.detach().clone() for n, p in model.named_parameters()}
        for _ in range(5):
            loss = torch.nn.functional.mse_loss(model(x).squeeze(-1), y) + (S.fedprox_penalty(model, g, mu) if mu else 0.0)
            opt.zero_grad(); loss.backward(); opt.step()
        return len(x)
    glob = torch.nn.Linear(3, 1, bias=False)
    srv = S.FederatedServer(glob, seed=0)
    for r in range(40):
        srv.round(srv.select(clients, 3), local_train)
    assert torch.allclose(glob.weight.detach()[0], w_true, atol=0.05) and srv.history[-1]["update_norm"] < srv.history[0]["update_norm"] and len(srv.select(clients, 2, "round_robin")) == 2
    plain, prox = torch.nn.Linear(3, 1, bias=False), torch.nn.Linear(3, 1, bias=False)
    prox.load_state_dict(plain.state_dict())
    s1, s2 = S.FederatedServer(plain, seed=1), S.FederatedServer(prox, seed=1)
    d1 = s1.round(clients[:3], local_train)["divergence"]
    d2 = s2.round(clients[:3], lambda m, c: local_train(m, c, mu=5.0))["divergence"]
    assert d2 < d1
    dp = S.FederatedServer(torch.nn.Linear(3, 1, bias=False), dp_clip=0.1, dp_noise=0.0)
    assert max(dp.round(clients[:3], local_train)["client_norms"]) <= 0.1 + 1e-9
    imp = S.FederatedServer(glob, seed=0).select(list(range(6)), 2, "importance", {5: 100.0, 4: 100.0})
    assert sorted(imp) == [4, 5]
    body = torch.nn.Sequential(torch.nn.Linear(3, 4), torch.nn.ReLU(), torch.nn.Linear(4, 1))
    pers = S.personalize(body, clients[0], lambda m, d: local_train(m, d), shared_prefixes=("0.",))
    assert torch.equal(pers[0].weight, body[0].weight) and not torch.equal(pers[2].weight, body[2].weight)
    # update encoding
    delta = torch.randn(1000)
    tk = S.encode_update(delta, "topk", 0.1)
    assert (S.decode_update(tk) != 0).sum() == 100 and torch.allclose(S.decode_update(tk)[delta.abs().topk(100).indices], delta[delta.abs().topk(100).indices]) and tk["bytes"] == 800
    g = torch.Generator().manual_seed(0)
    rk = torch.stack([S.decode_update(S.encode_update(delta, "randk", 0.1, generator=g)) for _ in range(400)]).mean(0)
    assert float((rk - delta).abs().mean()) < 0.2
    sg = S.decode_update(S.encode_update(delta, "sign"))
    assert torch.equal(torch.sign(sg), torch.sign(delta)) and S.encode_update(delta, "sign")["bytes"] == 129
    q8 = S.decode_update(S.encode_update(delta, "quantize", bits=8, generator=g))
    assert float((q8 - delta).abs().max()) <= float(delta.max() - delta.min()) / 255 + 1e-6 and S.encode_update(delta, "quantize", bits=4)["bytes"] == 508
    ctl = S.LocalSGDController(period=4)
    syncs = [ctl.should_sync() for _ in range(8)]
    assert syncs == [False, False, False, True] * 2
    ctl.after_sync(0.5); assert ctl.period == 2
    ctl.after_sync(0.001); ctl.after_sync(0.001); assert ctl.period == 8 and ctl.syncs == 3
    # gradient garbage collection
    gcx = S.GradientGarbageCollector(max_idle=2, thresholds=(1, 1, 1))
    a, b = torch.nn.Parameter(torch.randn(100)), torch.nn.Parameter(torch.randn(50))
    a.grad, b.grad = torch.ones(100), torch.ones(50)
    gcx.track(a); gcx.track(b)
    tmp = torch.nn.Parameter(torch.randn(5)); gcx.track(tmp); del tmp
    for _ in range(3):
        gcx.tick(); gcx.touch(a)
    res = gcx.collect()
    assert a.grad is not None and b.grad is None and res["freed_bytes"] == 200 and res["dead_refs"] == 1 and res["tracked"] == 2
    assert gcx.collect(force=True)["freed_grads"] == 1 and a.grad is None and gcx.stats["freed_grads"] == 2
    # capacity planning and cost analysis
    cp = S.CapacityPlanner(capacity=100.0, headroom=0.2)
    for d in range(28):
        cp.record_day(40 + 1.0 * d + (5 if d % 7 == 5 else 0))
    fc = cp.forecast(30)
    assert fc["direction"] == "growing" and fc["trend_per_day"] == pytest.approx(1.0, abs=0.05) and 5 <= fc["days_until_exhausted"] <= 13 and fc["urgency"] in ("high", "medium") and fc["action"] == "scale_up" and fc["recommended_capacity"] > 100
    idle = S.CapacityPlanner(100.0)
    for d in range(20):
        idle.record_day(10.0)
    assert idle.forecast()["action"] == "scale_down" and idle.forecast()["days_until_exhausted"] is None
    oc = S.OperationCostAnalyzer()
    for _ in range(100):
        oc.record("add", 5e-6, 4e5, 1e5); oc.record("matmul", 2e-4, 1e6, 1e9, "forward")
    oc.record("allreduce", 0.05, 1e8, 0, "backward")
    agg = oc.aggregate()
    kinds = {(s["op"], s["kind"]) for s in oc.suggestions()}
    assert agg["matmul"]["intensity"] == 1000 and agg["allreduce"]["share"] > 0.6 and {("allreduce", "hotspot"), ("add", "launch_bound")} <= kinds and oc.phase_breakdown()["backward"] == 0.05
    # record / replay
    rec = S.OperationRecorder()
    x = torch.randn(8, 8)
    y = rec.call("matmul", torch.matmul, x, x)
    z = rec.call("noise", lambda t: t + torch.rand_like(t), y)
    rp = S.OperationReplayer(rec.session).replay()
    assert rp["operations"] == 2 and not rp["deterministic"] and rp["mismatches"][0]["name"] == "noise" and S.OperationReplayer(rec.session[:1]).replay()["deterministic"]
    assert S.OperationReplayer(rec.session).replay(substitute={1: [torch.zeros(8, 8)]})["mismatches"] == []
    # health, progress, debugger
    net = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.ReLU(), torch.nn.Linear(8, 2))
    unused = torch.nn.Linear(2, 2)
    both = torch.nn.ModuleDict({"net": net, "unused": unused})
    hd = S.HealthDiagnostics()
    net(torch.randn(3, 4)).sum().backward()
    rep = hd.check(both)
    assert rep["status"] == "degraded" and sum("no gradient" in i["message"] for i in rep["issues"]) == 2
    net[0].weight.grad[0, 0] = float("nan")
    assert hd.check(net)["status"] == "critical"
    net.zero_grad(); net(torch.randn(3, 4)).sum().backward()
    for i in range(12):
        hd.record_step(0.1 if i < 11 else 0.5, 1e6 * (1 + 0.1 * i))
    cats = {i["category"] for i in hd.check(net)["issues"]}
    assert cats == {"memory", "performance"}
    clk = iter(range(1000))
    seen = []
    pr = S.ProgressReporter(10, seen.append, clock=lambda: float(next(clk)))
    for _ in range(10):
        pr.update(1, loss=0.5)
    assert seen[-1]["fraction"] == 1.0 and seen[-1]["eta_s"] == 0 and seen[4]["rate"] == pytest.approx(1.0) and seen[4]["eta_s"] == pytest.approx(5.0) and seen[0]["loss"] == 0.5
    child = pr.scope("eval", 2); child.update(2)
    assert seen[-1]["scope"] == "eval" and pr.statistics()["steps"] == 10
    dbg = S.InteractiveDebugger(net, ["stats", "watch 0", "continue"]).attach()
    dbg.add_breakpoint(module="1", condition="norm_above", threshold=0.0)
    dbg.add_breakpoint(condition="nan")
    dbg.add_breakpoint(module="2", on="backward")
    net(torch.randn(3, 4)).sum().backward()
    assert [(h["kind"], h["module"]) for h in dbg.hits] == [("forward", "1"), ("backward", "2")] and dbg.log[0]["shape"] == (3, 8) and dbg.log[0]["nan"] == 0
    net(torch.randn(3, 4))
    assert dbg.watch["0"].shape == (3, 8)
    with torch.no_grad():
        net[0].weight[0, 0] = float("nan")
    net(torch.randn(3, 4))
    assert ("forward", "0") in [(h["kind"], h["module"]) for h in dbg.hits]
    ab = S.InteractiveDebugger(net, ["abort"]).attach(); ab.add_breakpoint(module="2")
    dbg.detach()
    with pytest.raises(RuntimeError):
        net(torch.randn(3, 4))
    ab.detach()
    # VJP chains
    A1, A2, A3 = torch.randn(50, 20, dtype=dd), torch.randn(5, 50, dtype=dd), torch.randn(30, 5, dtype=dd)
    dvec = torch.rand(50, dtype=dd)
    vo = S.VjpOptimizer().add_matrix(A1).add_diagonal(dvec).add_matrix(A2).add_matrix(A3)
    v, xx = torch.randn(30, dtype=dd), torch.randn(20, dtype=dd)
    J = A3 @ A2 @ torch.diag(dvec) @ A1
    fused = vo.fuse()
    assert torch.allclose(vo.vjp(v), v @ J) and torch.allclose(vo.jvp(xx), J @ xx) and len(fused.ops) == 3 and torch.allclose(fused.vjp(v), v @ J)
    assert S.VjpOptimizer.chain_order([10, 30, 5, 60]) == (4500, "((A1 A2) A3)") and S.VjpOptimizer.chain_order([40, 20, 30, 10, 30])[0] == 26000
    co = fused.costs()
    assert co["vjp_flops"] == 2 * (1000 + 250 + 150) and co["materialized_vjp_flops"] == 2 * 20 * 30 and co["break_even_batch"] >= 1
    # quantum circuits
    qc = S.QuantumCircuit(2).h(0).cnot(0, 1)
    bell = qc.run(torch.zeros(0))
    assert torch.allclose(bell.abs() ** 2, torch.tensor([0.5, 0, 0, 0.5], dtype=dd)) and float(qc.expectation(torch.zeros(0), S.pauli_string("ZZ"))) == pytest.approx(1.0)
    assert torch.allclose((S.QuantumCircuit(2).x(1).cnot(1, 0).run(torch.zeros(0)).abs() ** 2), torch.tensor([0.0, 0, 0, 1], dtype=dd))
    ry = S.QuantumCircuit(1).ry(0, 0)
    th = torch.tensor([0.7], dtype=dd, requires_grad=True)
    e = ry.expectation(th, S.pauli_string("Z"))
    e.backward()
    assert float(e) == pytest.approx(math.cos(0.7)) and float(th.grad) == pytest.approx(-math.sin(0.7)) and float(ry.parameter_shift(th.detach(), S.pauli_string("Z"))) == pytest.approx(-math.sin(0.7))
    rz = S.QuantumCircuit(1).h(0).rz(0, 0).h(0)
    assert float(rz.expectation(torch.tensor([1.1], dtype=dd), S.pauli_string("Z"))) == pytest.approx(math.cos(1.1))
    ham = S.pauli_string("ZZ") + 0.5 * (S.pauli_string("XI") + S.pauli_string("IX"))
    ans = S.QuantumCircuit(2).ry(0, 0).ry(1, 1).cnot(0, 1).ry(0, 2).ry(1, 3)
    res = S.vqe(ans, ham, 4, steps=250, lr=0.1)
    assert res["energy"] == pytest.approx(res["exact"], abs=5e-3) and res["history"][-1] < res["history"][0]
    # Wirtinger derivatives
    z = torch.tensor([1.0 + 2.0j, -0.5 + 0.3j], dtype=torch.complex128)
    dz, dzc = S.wirtinger_grad(lambda t: (t * t).sum(), z)
    assert torch.allclose(dz, 2 * z) and dzc.abs().max() < 1e-12 and S.is_holomorphic(lambda t: (t ** 3).sum(), z)
    dz, dzc = S.wirtinger_grad(lambda t: (t * t.conj()).real.sum(), z)
    assert torch.allclose(dz, z.conj()) and torch.allclose(dzc, z) and not S.is_holomorphic(lambda t: (t * t.conj()).sum(), z)
    # edge cases and recovery
    eh = S.EdgeCaseHandler()
    out, found = eh.handle(torch.tensor([1.0, float("nan"), float("inf"), 1e-42, -float("inf")]))
    assert found == ["nan", "inf", "denormal"] and out.tolist() == pytest.approx([1.0, 0.0, 1e30, 0.0, -1e30]) and eh.handle(torch.zeros(0))[0] is None and eh.handle(torch.tensor(3.0))[1] == ["scalar"]
    with pytest.raises(FloatingPointError):
        S.EdgeCaseHandler(nan="error").handle(torch.tensor([float("nan")]))
    assert eh.stats["nan"] == 1 and eh.stats["inf"] == 2 and eh.handle(torch.tensor([1, 2]))[1] == []
    state = {"w": 1.0, "lr": 0.1, "batch": 8}
    script = iter([RuntimeError("CUDA out of memory"), float("nan"), RuntimeError("connection reset"), 0.25])
    def step():
        v = next(script)
        if isinstance(v, Exception):
            raise v
        state["w"] += 1
        return v
    rcv = S.AutomaticErrorRecovery(lambda: {"w": state["w"]}, lambda s: state.update(s), shrink=lambda: state.update(batch=state["batch"] // 2), lower_lr=lambda: state.update(lr=state["lr"] / 2), sleep=lambda s: None)
    assert rcv.run(step) == 0.25 and [a["action"] for a in rcv.attempts] == ["shrink_batch", "restore_and_lower_lr", "backoff_retry"]
    assert state["batch"] == 4 and state["lr"] == 0.05 and state["w"] == 2.0 and rcv.good["w"] == 2.0
    always = S.AutomaticErrorRecovery(lambda: 0, lambda s: None, max_attempts=2, sleep=lambda s: None)
    with pytest.raises(RuntimeError):
        always.run(lambda: (_ for _ in ()).throw(RuntimeError("still broken")))


def test_core_extras_deprecation_chunking_compression_ieee_inspection_layout_ir_spikes_networks_shapes_orders_and_monitor():
    import warnings as _w
    from torsh_b200.core import extras as X
    from torsh_b200 import fx as tfx
    # deprecation registry
    api = X.ApiCompat("0.2.0")
    @api.deprecated("0.1.0", "0.3.0", "new_add")
    def old_add(a, b): return a + b
    @api.deprecated("0.1.0", "0.2.0")
    def gone(): return 1
    with pytest.warns(DeprecationWarning, match="new_add"):
        assert old_add(1, 2) == 3
    with pytest.raises(RuntimeError, match="removed in 0.2.0"):
        gone()
    rep = api.report()
    assert {r["name"].split(".")[-1] for r in rep} == {"old_add", "gone"} and rep[0]["calls"] == 1
    # chunking
    c = X.optimal_chunk(1 << 30, 4, working_tensors=3)
    assert c % 128 == 0 and 3 * 4 * c <= 126 << 20 < 3 * 4 * (c + 128) and X.optimal_chunk(1000, 4) == 1000
    x = torch.randn(100, 7)
    assert torch.equal(X.chunked_apply(lambda t: t * 2, x, chunk=13), x * 2)
    # compression round trips
    r = torch.tensor([[1, 1, 1, 2], [2, 2, 3, 3]])
    v, l, shp = X.rle_encode(r)
    assert v.tolist() == [1, 2, 3] and l.tolist() == [3, 3, 2] and torch.equal(X.rle_decode(v, l, shp), r)
    idx = torch.tensor([3, 7, 8, 20, 21])
    assert torch.equal(X.delta_decode(*X.delta_encode(idx), idx.shape), idx)
    sp = torch.randn(37, 5) * (torch.rand(37, 5) < 0.1)
    enc = X.bitmask_encode(sp)
    assert torch.equal(X.bitmask_decode(enc), sp) and enc["bytes"] < enc["dense_bytes"] / 3
    w24 = torch.tensor([[1.0, 0, 2, 0, 0, 0, 3, 4], [0, 0, 0, 0, 5, 0, 0, 6]])
    pm = X.pruning_metadata(w24)
    assert pm["is_2_4"] and pm["sparsity"] == 10 / 16 and pm["block_sparsity"] == 0.25 and not X.pruning_metadata(torch.ones(2, 8))["is_2_4"]
    # error codes
    assert X.error_name(X.error_code("SHAPE_MISMATCH")) == "SHAPE_MISMATCH" and X.error_category(2001) == "memory" and X.is_retryable(6001) and not X.is_retryable(1002)
    assert X.classify_exception(RuntimeError("CUDA out of memory")) == 2001 and X.classify_exception(IndexError("x")) == 1005 and X.classify_exception(ValueError("bad")) == 1001
    try:
        torch.zeros(2, 3) @ torch.zeros(4, 5)
    except RuntimeError as e:
        assert X.error_category(X.classify_exception(e)) == "user"
    assert len(set(X.ERROR_CODES.values())) == len(X.ERROR_CODES)
    # IEEE 754
    one = torch.tensor([1.0, -1.0, 0.0, 1.0])
    nxt = torch.tensor([np.nextafter(np.float32(1), np.float32(2)), np.nextafter(np.float32(-1), np.float32(-2)), -0.0, 1.0 + 4 * 2 ** -23])
    assert X.ulp_distance(one, nxt).tolist() == [1, 1, 0, 4]
    assert int(X.ulp_distance(torch.tensor([-1e-45]), torch.tensor([1e-45]))) == 2 and X.float_bits(1.0) == 0x3F800000 and X.float_bits(1.0, True) == 0x3FF0000000000000
    cl = X.classify_floats(torch.tensor([float("nan"), float("inf"), 0.0, -0.0, 1e-40, 1.0, -2.0]))
    assert cl == {"nan": 1, "inf": 1, "zero": 2, "negative_zero": 1, "subnormal": 1, "normal": 2}
    for dt in (torch.float32, torch.float64, torch.bfloat16):
        assert all(v for v in X.ieee754_compliance_report(dt).values() if v is not None)
    # inspector
    base = torch.arange(10000.0)
    info = X.inspect_tensor(base[:4], "slice")
    assert info["is_view"] and "small view keeps a large storage alive" in info["issues"] and info["max"] == 3.0 and sum(info["histogram"]) == 4
    bad = X.inspect_tensor(torch.tensor([1.0, float("nan"), 3e38]), "bad")
    assert bad["nan"] == 1 and bad["issues"][:2] == ["non-finite values", "values close to the dtype's range"]
    txt = X.format_inspection(X.inspect_tensor(torch.randn(4, 6).t(), "wt"))
    assert "non-contiguous" in txt and "float32[6, 4]" in txt and "█" in txt
    # layout advice
    lo = X.LayoutOptimizer()
    img = torch.randn(2, 8, 5, 5)
    lo.record_access("img", 1, 9); lo.record_access("img", 3, 1)
    rec = lo.recommend("img", img)
    assert rec["action"] == "channels_last" and rec["apply"](img).stride(1) == 1 and rec["share"] == 0.9
    assert lo.recommend("img", rec["apply"](img))["action"] == "none" and lo.recommend("other", img)["action"] == "none"
    m = torch.randn(6, 4)
    lo.record_access("m", 0)
    rec = lo.recommend("m", m)
    assert rec["action"] == "permute_contiguous" and rec["permutation"] == [1, 0] and rec["apply"](m).shape == (4, 6)
    # memory maps
    mm = X.memory_map([("weights", 0, 512), ("acts", 768, 256)], 1024, width=16)
    assert mm.splitlines()[0] == "|wwwwwwww....aaaa|" and "75%" in mm
    tl = X.memory_timeline([(i * 0.1, i * 100) for i in range(20)], height=4, width=10)
    assert tl.splitlines()[0].rstrip("|").count("#") < tl.splitlines()[3].rstrip("|").count("#") and "peak 1,900 B" in tl
    # MLIR / StableHLO text
    net = torch.nn.Sequential(torch.nn.Linear(8, 16, bias=False), torch.nn.ReLU(), torch.nn.Linear(16, 4, bias=False), torch.nn.Tanh())
    gm = tfx.symbolic_trace(net)
    mlir = X.emit_mlir(gm, [torch.randn(2, 8)])
    assert "func.func @forward(%arg0: tensor<2x8xf32>) -> tensor<2x4xf32>" in mlir and mlir.count("linalg.matmul_transpose_b") == 2 and "arith.maximumf" in mlir and "math.tanh" in mlir
    assert mlir.count("{") == mlir.count("}") and "return %" in mlir
    hlo = X.emit_mlir(gm, [torch.randn(2, 8)], dialect="stablehlo")
    assert hlo.count("stablehlo.dot_general") == 2 and "stablehlo.maximum" in hlo and "contracting_dims = [1] x [1]" in hlo and "tensor<16x8xf32>" in hlo
    # every SSA value is defined before use
    defined = {"%arg0"}
    for line in hlo.splitlines():
        if " = " in line:
            lhs, rhs = line.split(" = ", 1)
            assert all(tok.rstrip(",") in defined for tok in rhs.split() if tok.startswith("%")), line
            defined.add(lhs.strip())
    # spiking neurons
    lif = X.LIFNeurons(3, tau=10.0, threshold=1.0, refractory=2)
    spikes = lif.run(torch.tensor([0.5, 1.5, 3.0]).repeat(2000, 1))
    rates = spikes.float().mean(0)
    assert rates[0] == 0 and rates[1] < rates[2]
    for i, cur in ((1, 1.5), (2, 3.0)):
        assert float(rates[i]) == pytest.approx(lif.rate_for_constant_input(cur), rel=0.15)
    gaps = torch.diff(spikes[:, 2].nonzero().flatten())
    assert gaps.min() > 2
    g = torch.Generator().manual_seed(0)
    p = torch.tensor([0.1, 0.5, 0.9])
    assert torch.allclose(X.rate_decode(X.rate_encode(p, 4000, g)), p, atol=0.03)
    lat = X.latency_encode(torch.tensor([1.0, 0.5, 0.0, 0.1]), 11)
    assert lat.sum(0).tolist() == [1, 1, 0, 1] and lat.float().argmax(0).tolist() == [0, 5, 0, 9]
    # matrix product states
    torch.manual_seed(0)
    psi = torch.randn(2, 3, 2, 3, 2, dtype=torch.float64)
    mps = X.MatrixProductState.from_tensor(psi)
    assert torch.allclose(mps.to_tensor(), psi, atol=1e-12) and float(mps.norm()) == pytest.approx(float(psi.norm())) and mps.bond_dimensions() == [2, 6, 6, 2]
    assert float(mps.amplitude((1, 2, 0, 1, 1))) == pytest.approx(float(psi[1, 2, 0, 1, 1]))
    other = X.MatrixProductState.from_tensor(torch.randn_like(psi))
    assert float(mps.inner(other)) == pytest.approx(float((psi * other.to_tensor()).sum()))
    ghz = torch.zeros(2, 2, 2, 2, 2, 2, dtype=torch.float64); ghz[0, 0, 0, 0, 0, 0] = ghz[1, 1, 1, 1, 1, 1] = 2 ** -0.5
    g_mps = X.MatrixProductState.from_tensor(ghz, cutoff=1e-12)
    assert g_mps.bond_dimensions() == [2] * 5 and g_mps.num_parameters() < ghz.numel() and g_mps.truncation_error < 1e-12
    lossy = X.MatrixProductState.from_tensor(psi, max_bond=3)
    assert (lossy.to_tensor() - psi).norm() == pytest.approx(lossy.truncation_error, rel=0.5) and lossy.truncation_error > 0
    order, cost = X.contraction_order({"A": {"i": 2, "j": 1000}, "B": {"j": 1000, "k": 1000}, "C": {"k": 1000, "l": 2}}, output=("i", "l"))
    assert cost < 2 * 1000 * 1000 * 2 + 2 * 1000 * 2 + 1 and len(order) == 2 and order[0] in (("A", "B"), ("B", "C"))
    # shape validation
    X.validate_shapes("matmul", a=torch.zeros(2, 3), b=torch.zeros(3, 4))
    with pytest.raises(X.ShapeError, match=r"inner dimensions differ \(3 vs 4\).*a\[2, 3\], b\[4, 3\].*transpose b"):
        X.validate_shapes("matmul", a=torch.zeros(2, 3), b=torch.zeros(4, 3))
    with pytest.raises(X.ShapeError, match="not broadcastable"):
        X.validate_shapes("elementwise", x=(2, 3), y=(4, 3))
    X.validate_shapes("cat:1", a=(2, 3), b=(2, 9))
    with pytest.raises(X.ShapeError, match="except 1"):
        X.validate_shapes("cat:1", a=(2, 3), b=(3, 3))
    with pytest.raises(X.ShapeError, match="bias must have 5"):
        X.validate_shapes("linear", x=(7, 3), w=(5, 3), b=(4,))
    with pytest.raises(X.ShapeError, match="kernel is larger"):
        X.validate_shapes("conv2d", x=(1, 3, 2, 2), w=(8, 3, 3, 3))
    with pytest.raises(X.ShapeError, match="key and value lengths"):
        X.validate_shapes("attention", q=(2, 4, 10, 64), k=(2, 4, 12, 64), v=(2, 4, 11, 64))
    ex = X.explain_broadcast((3, 1, 5), (4, 2))
    assert "dim 1: 1 vs 4 -> 4" in ex and "dim 2: 5 vs 2 -> INCOMPATIBLE" in ex
    # cache-oblivious orders
    ys, xs = torch.tensor([0, 0, 1, 1, 5]), torch.tensor([0, 1, 0, 1, 3])
    code = X.morton_encode(ys, xs)
    assert code.tolist() == [0, 1, 2, 3, 0b100111] and [t.tolist() for t in X.morton_decode(code)] == [ys.tolist(), xs.tolist()]
    order = X.morton_order(4, 4)
    assert order[:8].tolist() == [0, 1, 4, 5, 2, 3, 6, 7] and sorted(order.tolist()) == list(range(16))
    a = torch.randn(70, 45)
    assert torch.equal(X.cache_oblivious_transpose(a, base=8), a.t())
    # performance monitor
    now = [0.0]
    alerts = []
    mon = X.PerfMonitor(window=50, on_alert=alerts.append, clock=lambda: now[0])
    mon.set_threshold("step", p95_above=0.5)
    for i in range(20):
        now[0] += 0.1
        mon.record("step", 0.1)
    assert not alerts and mon.summary("step")["rate_per_s"] == pytest.approx(10.0) and mon.summary("step")["p50"] == 0.1
    for _ in range(3):
        now[0] += 1.0
        mon.record("step", 1.0)
    assert alerts and alerts[0]["kind"] == "p95" and alerts[0]["metric"] == "step"
    with mon.time("io"):
        now[0] += 0.25
    assert mon.summary("io")["mean"] == pytest.approx(0.25) and set(mon.snapshot()) == {"step", "io"} and mon.summary("none") == {"count": 0}


def test_bench_suite_runner_analysis_cache_comparison_validation_ci_regressions_scaling_reports_and_probes(tmp_path):
    import xml.etree.ElementTree as ET
    from torsh_b200.utils import bench_suite as B
    # runner on the host, with a synthetic workload whose cost is controlled by a fake clock-free sleep-less loop
    gen = B.DataGenerator(0)
    assert gen.tensor((1000,), "uniform", low=2, high=3).min() >= 2 and float((gen.tensor((4000,), sparsity=0.75) == 0).float().mean()) == pytest.approx(0.75, abs=0.03)
    assert gen.tensor((2, 3), "sequential").tolist() == [[0, 1, 2], [3, 4, 5]] and gen.tensor((3,), "constant", value=7).tolist() == [7, 7, 7]
    mm = B.FunctionBench(lambda n, cfg: (gen.tensor((n, n)), gen.tensor((n, n))), torch.matmul, flops=lambda n: 2 * n ** 3, nbytes=lambda n: 3 * n * n * 4)
    runner = B.BenchRunner()
    cfg = B.BenchConfig("matmul", sizes=(32, 64), warmup=1, iterations=4)
    res = runner.run(mm, cfg)
    assert [r.size for r in res] == [32, 64] and all(len(r.times) == 4 and r.gflops() > 0 and r.gbps() > 0 for r in res) and res[0].to_dict()["median"] == res[0].median
    assert cfg.key() == B.BenchConfig("matmul", sizes=(32, 64), warmup=1, iterations=4).key() != B.BenchConfig("matmul", sizes=(32,)).key()
    # statistics and roofline placement
    s = B.summarize([1.0, 1.1, 0.9, 1.0, 1.05, 5.0])
    assert s["outliers"] == [5.0] and s["median"] == pytest.approx(1.025) and s["ci"][0] < s["mean"] < s["ci"][1]
    an = B.BenchmarkAnalyzer(peak_gflops=1000.0, peak_gbps=100.0)
    memb = B.BenchResult("copy", 1, [1e-3] * 5, flops=1e6, bytes=8e7)          # 0.0125 flop/B, 80 GB/s of 100
    a = an.analyze(memb)
    assert a["bottleneck"] == "memory" and a["efficiency"] == pytest.approx(0.8) and a["rating"] == "good" and a["stable"] and not a["recommendations"]
    comp = an.analyze(B.BenchResult("gemm", 1, [1e-3, 1.3e-3, 0.8e-3, 1e-3], flops=2e8, bytes=1e6))      # 200 GFLOP/s of 1000
    assert comp["bottleneck"] == "compute" and comp["rating"] == "poor" and len(comp["recommendations"]) == 2
    assert an.analyze(B.BenchResult("tiny", 1, [5e-6] * 4, flops=1e3, bytes=1e3))["bottleneck"] == "launch"
    # complexity classes
    ns = [64, 128, 256, 512, 1024, 2048]
    for name, f in (("O(n)", lambda n: 3e-9 * n + 1e-7), ("O(n log n)", lambda n: 2e-9 * n * math.log2(n)), ("O(n^2)", lambda n: 1e-10 * n * n + 1e-7), ("O(1)", lambda n: 5e-6)):
        assert B.fit_complexity(ns, [f(n) for n in ns])["class"] == name
    assert B.fit_complexity(ns, [1e-10 * n ** 3 for n in ns])["loglog_slope"] == pytest.approx(3.0)
    # cache
    now = [1000.0]
    cache = B.BenchmarkCache(tmp_path / "cache", ttl=60, environment={"host": "a"}, clock=lambda: now[0])
    calls = []
    counted = B.FunctionBench(lambda n, c: (torch.ones(n),), lambda t: calls.append(1) or t.sum())
    cr = B.CachedBenchRunner(cache)
    small = B.BenchConfig("sum", sizes=(8,), warmup=0, iterations=2)
    r1 = cr.run(counted, small); n_calls = len(calls)
    r2 = cr.run(counted, small)
    assert len(calls) == n_calls and r2[0].times == r1[0].times and cache.stats == {"hits": 1, "misses": 1, "expired": 0}
    now[0] += 120
    cr.run(counted, small)
    assert cache.stats["expired"] == 1 and len(calls) == 2 * n_calls
    assert B.BenchmarkCache(tmp_path / "cache", environment={"host": "b"}).get(small) is None
    # comparison with significance
    rng = np.random.default_rng(0)
    base = B.BenchResult("op", 1, (1.0 + 0.01 * rng.standard_normal(20)).tolist())
    fast = B.BenchResult("op", 1, (0.8 + 0.01 * rng.standard_normal(20)).tolist())
    same = B.BenchResult("op", 1, (1.0 + 0.01 * rng.standard_normal(20)).tolist())
    cmp = B.BenchmarkComparator()
    assert cmp.compare(base, fast)["verdict"] == "faster" and cmp.compare(fast, base)["verdict"] == "slower" and cmp.compare(base, same)["verdict"] == "equivalent"
    from scipy import stats as sst
    t, p = B.welch_t(base.times, fast.times)
    ref = sst.ttest_ind(base.times, fast.times, equal_var=False)
    assert t == pytest.approx(ref.statistic) and p == pytest.approx(ref.pvalue, rel=1e-6, abs=1e-300)
    sets = cmp.compare_sets([base, B.BenchResult("other", 2, base.times)], [fast, B.BenchResult("other", 2, same.times)])
    assert sets["faster"] == 1 and sets["equivalent"] == 1 and sets["geomean_speedup"] == pytest.approx(math.sqrt(1.25), rel=0.02)
    # validation of what was timed
    val = B.BenchmarkValidator()
    x, y = torch.randn(16, 16), torch.randn(16, 16)
    assert val.validate("mm", torch.matmul, torch.matmul, [x, y], times=[1.0, 1.01, 0.99])["status"] == "passed"
    wrong = val.validate("mm", lambda a, b: a @ b + 1e-2, torch.matmul, [x, y], times=[1.0, 2.0, 0.5])
    assert wrong["status"] == "failed" and {i["category"] for i in wrong["issues"]} == {"accuracy", "consistency"}
    noisy = val.validate("rand", lambda a: a + torch.rand_like(a) * 1e-9, lambda a: a, [x.double()])
    assert noisy["status"] == "warning" and noisy["issues"][0]["category"] == "determinism"
    assert B.cancellation_risk(torch.tensor([1.0, 1.0]), torch.tensor([1.0 + 1e-6, 0.5])) == 0.5
    # CI gate
    ci = B.CIBenchmarkRunner(B.CIConfig(warn_slowdown=0.05, fail_slowdown=0.15))
    slow10 = B.BenchResult("op", 1, (1.1 + 0.01 * rng.standard_normal(20)).tolist())
    slow30 = B.BenchResult("op", 1, (1.3 + 0.01 * rng.standard_normal(20)).tolist())
    assert ci.evaluate([base], [same])["status"] == "pass" and ci.evaluate([base], [slow10])["status"] == "warn" and ci.evaluate([base], [fast])["rows"][0]["status"] == "improved"
    dec = ci.evaluate([base], [slow30])
    assert dec["status"] == "fail" and dec["exit_code"] == 1
    suite = ET.fromstring(ci.junit_xml(dec))
    assert suite.attrib["failures"] == "1" and suite.find("testcase/failure") is not None and "FAIL" in ci.markdown(dec) and ci.annotations(dec)[0].startswith("::error title=benchmark op::+")
    # regressions in a history
    det = B.AdvancedRegressionDetector()
    hist = (1.0 + 0.01 * rng.standard_normal(15)).tolist() + (1.3 + 0.01 * rng.standard_normal(8)).tolist()
    r = det.analyze(hist)
    assert r["status"] == "regression" and r["change_point"] == 15 and r["shift"] == pytest.approx(0.3, abs=0.02) and r["severity"] == "major" and r["trend"] == "degrading"
    assert det.analyze((1.0 + 0.01 * rng.standard_normal(25)).tolist())["status"] == "stable" and det.analyze([1.0] * 3)["status"] == "insufficient_history"
    assert det.analyze(hist[::-1])["kind"] == "improvement"
    z, p = det.mann_kendall(list(range(10)))
    assert z > 3 and p < 0.01
    # scalability
    assert B.size_progression("power_of_two", 100, 2000) == [128, 256, 512, 1024] and B.size_progression("linear", 10, 50, 5) == [10, 20, 30, 40, 50] and B.size_progression("exponential", 1, 1000, 4) == [1, 10, 100, 1000]
    workers = [1, 2, 4, 8, 16]
    am = B.amdahl_fit(workers, [10 * (0.1 + 0.9 / p) for p in workers])
    assert am["serial_fraction"] == pytest.approx(0.1) and am["max_speedup"] == pytest.approx(10.0) and am["speedup"][-1] == pytest.approx(1 / (0.1 + 0.9 / 16)) and am["efficiency"][0] == 1.0
    assert B.ScalabilityTestSuite.weak_scaling([1, 2, 4], [100, 190, 360]) == pytest.approx([1.0, 0.95, 0.9])
    assert B.ScalabilityTestSuite._knee([1, 2, 4, 8, 16], [1.0, 1.0, 0.9, 2.0, 2.1]) == 8
    sweep = B.ScalabilityTestSuite().size_sweep(B.FunctionBench(lambda n, c: (torch.ones(n),), lambda t: t.sum()), B.BenchConfig("sum", sizes=(1 << 10, 1 << 12, 1 << 14), warmup=1, iterations=3))
    assert len(sweep["results"]) == 3 and sweep["complexity"]["class"] in B.COMPLEXITY_CLASSES
    # system information
    info = B.system_info()
    assert info["torch"] == torch.__version__ and info["cpu_count"] >= 1 and len(info["fingerprint"]) == 12 and B.system_info()["fingerprint"] == info["fingerprint"]
    # charts, reports, dashboards
    line = B.Chart("scaling", x_label="n", y_label="ms", log_x=True).add_series("ours", [1, 10, 100], [1.0, 2.0, 4.0]).add_series("ref", [1, 10, 100], [1.5, 3.0, 6.0]).annotate(10, 2.0, "knee")
    svg = ET.fromstring(line.to_svg())
    nsx = "{http://www.w3.org/2000/svg}"
    polys = svg.findall(f"{nsx}polyline")
    assert len(polys) == 2 and len(polys[0].attrib["points"].split()) == 3
    xs = [float(p.split(",")[0]) for p in polys[0].attrib["points"].split()]
    assert xs[1] - xs[0] == pytest.approx(xs[2] - xs[1])                      # log axis: decades evenly spaced
    bars = ET.fromstring(B.Chart("t", kind="bar").add_series("a", ["x", "y"], [1.0, 2.0]).to_svg()).findall(f"{nsx}rect[@class='bar']")
    assert len(bars) == 2 and float(bars[1].attrib["height"]) == pytest.approx(2 * float(bars[0].attrib["height"]), rel=1e-2)
    page = B.HtmlReportGenerator("Report", theme="dark").add_results("GEMM", [memb], an).add_chart(line).add_text("notes", "a < b").add_system(info).render()
    assert page.startswith("<!doctype html>") and "<td>memory</td><td>80%</td>" in page and "a &lt; b" in page and "<svg" in page and "#111" in page
    dash = B.PerformanceDashboard(tmp_path / "hist.jsonl")
    for i, v in enumerate(hist):
        dash.record(f"run{i}", {"step_ms": v, "tokens_per_s": 1000.0}, timestamp=float(i))
    h = dash.history()
    assert len(h["step_ms"]) == 23 and h["step_ms"][0][0] == "run0"
    out = dash.render()
    assert "step_ms: regression" in out and "tokens_per_s: stable" in out and "regression +" in out and out.count("<svg") == 2
    # library comparisons
    cmpr = B.ComparisonRunner(iterations=2, warmup=1).with_defaults()
    rows = cmpr.run("matmul", [x, y])
    assert set(rows) == {"numpy", "torch"} and rows["numpy"]["max_diff_vs_baseline"] < 1e-4 and rows["torch"]["speedup_vs_baseline"] == 1.0
    # precision / quantisation / pruning
    pb = B.precision_benchmark(torch.matmul, [torch.randn(64, 64), torch.randn(64, 64)], iterations=2)
    assert pb["float32"]["rel_error"] < 1e-6 < pb["float16"]["rel_error"] < pb["bfloat16"]["rel_error"] < 0.05
    w, xin = torch.randn(32, 64), torch.randn(8, 64)
    qb = B.quantization_benchmark(w, xin)
    assert qb["int8"]["sqnr_db"] > qb["int4"]["sqnr_db"] + 20 and qb["int4"]["compression"] > qb["int8"]["compression"] > 3.5 and qb["int8"]["output_rel_error"] < 0.02
    pr = B.pruning_benchmark(w, xin)
    assert pr[0.5]["achieved_sparsity"] == pytest.approx(0.5, abs=0.01) and pr[0.5]["output_rel_error"] < pr[0.9]["output_rel_error"] and pr[0.9]["sparse_flops"] < 0.11 * pr[0.9]["dense_flops"]
    p24 = B.pruning_benchmark(w, xin, sparsities=(0.5,), method="2:4")[0.5]
    assert p24["achieved_sparsity"] == 0.5 and p24["output_rel_error"] < B.pruning_benchmark(w, xin, sparsities=(0.5,), method="random")[0.5]["output_rel_error"]
    # edge deployment
    net = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 10))
    eb = B.edge_inference_benchmark(net, torch.randn(1, 64), B.EdgeProfile(memory_limit_mb=1.0, power_watts=2.0, battery_wh=10.0), iterations=3, inferences_per_hour=3600)
    assert eb["fits_memory"] and eb["model_mb"] == pytest.approx((64 * 128 + 128 + 1280 + 10) * 4 / 2 ** 20) and eb["energy_mj"] == pytest.approx(2.0 * eb["latency_ms"]) and eb["battery_hours"] == pytest.approx(10.0 / (eb["energy_mj"] * 1e-3))
    assert not B.edge_inference_benchmark(net, torch.randn(1, 64), B.EdgeProfile(memory_limit_mb=0.01), iterations=1)["fits_memory"]
    hp = B.hardware_probes(mb=4, n=64, iterations=2)
    assert hp["copy_gbps"] > 0 and hp["matmul_gflops"] > 0 and hp["ridge_flops_per_byte"] > 0
    mon = B.MemoryMonitor()
    mon.sample("a"); keep = torch.ones(1 << 22); mon.sample("b")
    assert mon.peak() >= mon.samples[0][1] and isinstance(mon.growth(), int)


def test_jit_analysis_intervals_paths_partial_eval_generics_templates_advisor_pgo_loops_uncertainty_synthesis_speculation_learned_costs_symbols_tuning_and_llvm():
    from torsh_b200 import jit_analysis as J
    # interval abstract interpretation: bounds hold for samples, domain problems are reported
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = torch.nn.Linear(4, 3)
        def forward(self, x):
            h = torch.relu(self.fc(x))
            return torch.sigmoid(h) / (h - 0.5), torch.log(h)
    torch.manual_seed(0)
    net = Net()
    gm = torch.fx.symbolic_trace(net)
    ai = J.AbstractInterpreter(gm)
    env = ai.run(J.Interval(-1.0, 1.0))
    xs = torch.rand(500, 4) * 2 - 1
    pre = net.fc(xs).detach()
    assert env["fc"].lo <= float(pre.min()) and float(pre.max()) <= env["fc"].hi and env["relu"].lo >= 0 and env["relu"].sign() == "non-negative"
    assert 0.5 <= env["sigmoid"].lo and env["sigmoid"].hi <= 1.0 and {w["kind"] for w in ai.warnings} == {"division_by_zero", "domain"}
    iv = J.Interval(-2, 3)
    assert (iv * iv) == J.Interval(-6, 9) and (iv - iv) == J.Interval(-5, 5) and (J.Interval(1, 2) / J.Interval(4, 8)) == J.Interval(0.125, 0.5) and iv.join(J.Interval(5, 6)) == J.Interval(-2, 6)
    assert iv.meet(J.Interval(4, 5)).is_empty() and J.Interval(0, 1).widen(J.Interval(0, 2)) == J.Interval(0, math.inf) and J.Interval(1, 2).sign() == "positive"
    safe = J.AbstractInterpreter(torch.fx.symbolic_trace(lambda x: torch.exp(x) / (torch.abs(x) + 1.0)))
    out = safe.run(J.Interval(-3, 3))
    assert not safe.warnings and safe.output.lo > 0 and safe.output.hi <= math.exp(3) + 1e-9
    # symbolic execution enumerates the feasible paths with witnesses
    def f(x, y):
        if x > 10:
            if y < x:
                return x - y
            return y * 2
        if x > 20:                      # unreachable: x <= 10 here
            return 0
        return 1 / (x - 5)
    paths = J.SymbolicExecutor().explore(f)
    feas = [p for p in paths if p.feasible]
    assert len(paths) == 4 and len(feas) == 3 and [p for p in paths if not p.feasible][0].conditions == ["not (x > 10)", "x > 20"]
    for p in feas:
        w = p.witness
        if p.conditions == ["x > 10", "y < x"]:
            assert w["x"] > 10 and w["y"] < w["x"] and p.result == "(x - y)"
    assert any(p.conditions == ["x > 10", "not (y < x)"] and p.result == "(y * 2)" for p in feas)
    # partial evaluation removes the branch on a static argument
    def poly(x, degree, scale):
        out = x * 0
        for d in range(degree):
            out = out + x ** d
        return out * scale if scale != 1 else out
    g3, rep = J.partial_evaluate(poly, degree=3, scale=1)
    t = torch.randn(5)
    assert torch.allclose(g3(t, 3, 1), 1 + t + t * t) and "mul_1" not in g3.code and rep["static"] == ["degree", "scale"]
    g2, _ = J.partial_evaluate(poly, degree=2, scale=2)
    assert torch.allclose(g2(t, 2, 2), 2 * (1 + t)) and len(list(g2.graph.nodes)) < len(list(g3.graph.nodes)) + 2
    # generics
    @J.generic(T=(torch.float32, torch.float64))
    def axpy(a: "T", b: "T", types=None):
        return a * 2 + b, types["T"]
    r32, t32 = axpy(torch.ones(2), torch.ones(2))
    r64, t64 = axpy(torch.ones(2, dtype=torch.float64), torch.ones(2, dtype=torch.float64))
    axpy(torch.zeros(2), torch.zeros(2))
    assert t32 == torch.float32 and t64 == torch.float64 and axpy.instantiations() == ["axpy<float32>", "axpy<float64>"]
    with pytest.raises(TypeError, match="bound to both"):
        axpy(torch.ones(2), torch.ones(2, dtype=torch.float64))
    with pytest.raises(TypeError, match="constraint"):
        axpy(torch.ones(2, dtype=torch.int32), torch.ones(2, dtype=torch.int32))
    # templates, unrolling, reflection
    tpl = J.CodeTemplate("def act(x):\n    return torch.${fn}(x) * ${scale}\n", "act")
    assert torch.equal(tpl.instantiate(fn="relu", scale=2)(torch.tensor([-1.0, 3.0])), torch.tensor([0.0, 6.0])) and tpl.instantiate(fn="relu", scale=2) is tpl.instantiate(fn="relu", scale=2) and len(tpl.generated) == 1
    fn, src = J.unroll_loop("x = x * 2 + k", "k", 3)
    assert fn(1) == ((1 * 2 + 0) * 2 + 1) * 2 + 2 and src.count("x = x * 2") == 3 and "for" not in src
    refl = J.reflect(gm)
    assert refl["inputs"] == ["x"] and refl["operations"]["call_module:Linear"] == 1 and refl["parameters"]["fc.weight"] == (3, 4) and refl["depth"] >= 5
    # advisor
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc, self.act = torch.nn.Linear(8, 8), torch.nn.GELU()
        def forward(self, x):
            h = self.act(self.fc(x))
            a, b = torch.exp(x), torch.exp(x)
            unused = x + 1
            return torch.tanh(torch.relu(h * 2.0) + 1.0) + a + b
    bgm = torch.fx.symbolic_trace(Block())
    recs = J.OptimizationAdvisor(bgm).advise()
    kinds = [r["kind"] for r in recs]
    assert {"fuse_elementwise", "fuse_epilogue", "common_subexpression", "dead_code", "precision"} <= set(kinds) and recs[0]["gain"] >= recs[-1]["gain"]
    assert [r for r in recs if r["kind"] == "dead_code"][0]["nodes"] == ["add"] and sorted([r for r in recs if r["kind"] == "common_subexpression"][0]["nodes"]) == ["exp", "exp_1"]
    prof = J.ProfilingInterpreter(bgm)
    for _ in range(3):
        prof.run(torch.randn(4, 8))
    p = prof.profile()
    assert p["counts"]["fc"] == 3 and p["shapes"]["fc"] == {(4, 8): 3} and all(v > 0 for v in p["times"].values())
    hot = J.OptimizationAdvisor(bgm, {**{k: 1e-6 for k in p["times"]}, "fc": 1.0}).advise()
    assert any(r["kind"] == "hotspot" and r["nodes"] == ["fc"] for r in hot)
    # profile-guided dispatch
    d = J.ProfileGuidedDispatcher(lambda x: "general", hot_threshold=5)
    d.add("tiny", lambda x: x.shape[0] <= 4, lambda x: "tiny").add("aligned", lambda x: x.shape[0] % 128 == 0, lambda x: "aligned")
    for _ in range(20):
        assert d(torch.empty(256)) == "aligned"
    assert d(torch.empty(3)) == "tiny" and d(torch.empty(77)) == "general" and d.guard_evals == 20 * 2 + 1 + 2
    assert d.reoptimize() == ["aligned", "tiny"] and (256,) in d.table
    before = d.guard_evals
    assert d(torch.empty(256)) == "aligned" and d.guard_evals == before and d(torch.empty(128)) == "aligned" and d.guard_evals == before + 1
    # loop nests: A[i][j] = A[i-1][j+1] + 1 has distance (1, -1): interchange and tiling are illegal, skewless stencil (1, 0) is fine
    bad = J.LoopNest([("i", 1, 6), ("j", 0, 5)], [J.Access("A", [{"i": 1}, {"j": 1}], True), J.Access("A", [{"i": 1, "": -1}, {"j": 1, "": 1}])], "A[i][j] = A[i - 1][j + 1] + 1")
    assert bad.dependences() == [(1, -1)] and not bad.can_permute([1, 0]) and not bad.can_tile() and bad.parallel_loops() == []
    with pytest.raises(ValueError):
        bad.generate(order=[1, 0])
    good = J.LoopNest([("i", 1, 9), ("j", 1, 9)], [J.Access("A", [{"i": 1}, {"j": 1}], True), J.Access("A", [{"i": 1, "": -1}, {"j": 1}]), J.Access("A", [{"i": 1}, {"j": 1, "": -1}])], "A[i][j] = A[i - 1][j] + A[i][j - 1]")
    assert good.dependences() == [(0, 1), (1, 0)] and good.can_permute([1, 0]) and good.can_tile()
    base_fn, _ = good.generate()
    tiled_fn, tsrc = good.generate(order=[1, 0], tiles={"i": 3, "j": 4})
    A0 = [[1] * 9 for _ in range(9)]
    A1, A2 = [r[:] for r in A0], [r[:] for r in A0]
    base_fn(A1); tiled_fn(A2)
    assert A1 == A2 and A1[8][8] == math.comb(16, 8) and "for j_t in range(1, 9, 4)" in tsrc and tsrc.index("j_t") < tsrc.index("i_t")
    par = J.LoopNest([("i", 0, 4), ("j", 1, 4)], [J.Access("B", [{"i": 1}, {"j": 1}], True), J.Access("B", [{"i": 1}, {"j": 1, "": -1}])], "B[i][j] = B[i][j - 1] * 2")
    assert par.parallel_loops() == ["i"]
    none = J.LoopNest([("i", 0, 8)], [J.Access("C", [{"i": 2}], True), J.Access("C", [{"i": 2, "": 1}])], "C[2 * i] = C[2 * i + 1]")
    assert none.dependences() == [] and none.parallel_loops() == ["i"]
    # uncertain shapes
    dist = J.ShapeDistribution.from_observations([128] * 90 + [8192] * 10)
    variants = {"small_tiles": lambda n: 1.0 + n / 512, "large_tiles": lambda n: 6.0 + n / 4096}
    ch = J.choose_variant(variants, dist)
    assert ch["choice"] == "small_tiles" and ch["table"]["small_tiles"]["mean"] == pytest.approx(0.9 * 1.25 + 0.1 * 17.0)
    assert J.choose_variant(variants, dist, risk_aversion=1.0)["choice"] == "large_tiles" and J.choose_variant(variants, dist, tail=0.99)["choice"] == "large_tiles"
    # synthesis from examples
    gsyn = torch.Generator().manual_seed(1)
    ex = [((a, b), torch.relu(a - b)) for a, b in ((torch.randn(6, generator=gsyn), torch.randn(6, generator=gsyn)) for _ in range(4))]
    syn = J.synthesize(ex, 2)
    a, b = torch.randn(9), torch.randn(9)
    assert syn is not None and syn["depth"] == 3 and torch.allclose(syn["fn"](a, b), torch.relu(a - b)) and "x0" in syn["expression"] and "x1" in syn["expression"]
    assert J.synthesize([((a,), torch.cos(a))], 1, max_depth=2) is None
    sq = J.synthesize([((a,), a * a + 1.0)], 1, constants=(1.0,))
    assert torch.allclose(sq["fn"](b), b * b + 1)
    # speculation
    calls = Counter()
    def general(x): calls["general"] += 1; return x.contiguous().sum()
    def fast(x): calls["fast"] += 1; return x.sum()
    sp = J.SpeculativeFunction(general, max_failure_rate=0.3, min_calls=10).speculate("contiguous", lambda x: x.is_contiguous(), fast)
    cont, strided = torch.ones(4, 4), torch.ones(4, 8)[:, ::2]
    for _ in range(8):
        sp(cont)
    sp(strided)
    assert calls == {"fast": 8, "general": 1} and sp.stats["contiguous"]["active"]
    for _ in range(6):
        sp(strided)
    assert not sp.stats["contiguous"]["active"]
    sp(cont)
    assert calls["fast"] == 8
    # differentiable selection and continuous knobs
    torch.manual_seed(0)
    costs = {"a": 3.0, "b": 1.0, "c": 2.0}
    sched = J.DifferentiableScheduler(list(costs))
    noise = torch.Generator().manual_seed(0)
    hist = sched.fit(lambda k: costs[k] * (1 + 0.05 * float(torch.randn((), generator=noise))), steps=150)
    assert sched.best() == "b" and float(sched.probabilities()[1].detach()) > 0.8 and hist[-1] < hist[5]
    knob = J.optimise_continuous_knob(lambda t: (t - 96.0) ** 2 / 1e3 + 1.0, init=32.0, lo=16.0, hi=256.0, steps=400, lr=0.1)
    assert knob == pytest.approx(96.0, abs=2.0)
    # learned cost model ranks unseen programs
    feats, secs = [], []
    for width in (16, 32, 64, 128, 256, 512):
        for depth in (1, 2, 3):
            m = torch.nn.Sequential(*[l for _ in range(depth) for l in (torch.nn.Linear(width, width), torch.nn.ReLU())])
            fv = J.graph_features(torch.fx.symbolic_trace(m), [torch.randn(8, width)])
            feats.append(fv); secs.append(1e-6 + 1e-10 * math.expm1(float(fv[0])))
    feats, secs = torch.stack(feats), torch.tensor(secs)
    lcm = J.LearnedCostModel()
    assert lcm.fit(feats, secs, steps=800) < 0.05
    test_f = torch.stack([J.graph_features(torch.fx.symbolic_trace(torch.nn.Sequential(torch.nn.Linear(w, w), torch.nn.ReLU(), torch.nn.Linear(w, w))), [torch.randn(8, w)]) for w in (24, 384, 96)])
    assert lcm.rank(test_f) == [0, 2, 1] and (lcm.predict_seconds(test_f) > 0).all()
    # debug symbols
    def user_fn(x):
        y = torch.relu(x)
        return y * 3
    ugm, sym = J.DebugSymbolTable.trace(user_fn)
    s = sym.lookup("relu")
    assert s and s["file"].endswith("test_aux_cpu.py") and s["source"] == "y = torch.relu(x)" and sym.lookup("mul")["line"] == s["line"] + 1 and s["function"] == "user_fn"
    gen_line = next(i for i, l in enumerate(ugm.code.splitlines(), 1) if l.strip().startswith("relu"))
    assert sym.source_of_generated_line(gen_line)["source"] == "y = torch.relu(x)" and "test_aux_cpu.py" in sym.annotate_error("mul", ValueError("boom")) and json.loads(sym.to_json())["symbols"]["relu"]["line"] == s["line"]
    # hardware tuning tables
    big = J.tune_gemm_tiles(8192, 8192, 8192)
    assert big["tile"] == (128, 256, 64) and big["tmem_columns"] == 512 and big["smem_bytes"] <= 227 * 1024 and big["stages"] >= 3 and big["split_k"] == 1 and big["double_buffered_accumulator"]
    skinny = J.tune_gemm_tiles(256, 512, 16384)
    assert skinny["ctas"] < 74 and skinny["split_k"] > 1
    odd = J.tune_gemm_tiles(148 * 128, 128, 512)
    assert odd["wave_efficiency"] == 1.0 and odd["tile"][1] == 128
    ew = J.tune_elementwise(1 << 28)
    assert ew["vector_width"] == 8 and ew["persistent"] and ew["grid"] == 148 * 8 and not ew["fits_l2"] and J.tune_elementwise(1000)["grid"] == 1
    # LLVM IR text for a fused chain: relu(a * b + 1.5) / exp(a)
    ir = J.emit_llvm_ir([("mul", "in0", "in1"), ("add", "t0", 1.5), ("relu", "t1"), ("exp", "in0"), ("div", "t2", "t3")], 2)
    assert ir.startswith("declare float @llvm.exp.f32(float)\ndeclare float @llvm.maxnum.f32(float, float)\ndefine void @fused(float* noalias %in0") and ir.count("{") == ir.count("}") == 1
    defs = re.findall(r"^\s*(%[\w.]+) =", ir, re.M)
    assert len(defs) == len(set(defs)) and "%i = phi i64 [ 0, %entry ], [ %i.next, %loop ]" in ir and "store float %t4" in ir
    used = set(re.findall(r"(%[\w.]+)", ir.split("{", 1)[1])) - {"%entry", "%loop", "%exit"}
    assert used <= set(defs) | {"%in0", "%in1", "%out", "%n"}
    a, b = torch.randn(32), torch.randn(32)
    assert torch.allclose(J.interpret_llvm_ir(ir, [a, b]), torch.relu(a * b + 1.5) / torch.exp(a))


def test_ffi_header_model_generated_bindings_docs_tests_batching_numpy_pandas_scipy_views_and_migration(tmp_path):
    import subprocess
    import sys
    import importlib.util
    import pandas as pd
    from torsh_b200 import ffi
    from torsh_b200 import _native as nv
    fns = ffi.parse_header()
    by = {f.name: f for f in fns}
    assert len(fns) == 98 and by["torsh_init"].doc == "" and by["torsh_tensor_conv2d"].params[2].ctype == "const TorshTensor*" and [p.name for p in by["torsh_tensor_conv2d"].params] == ["input", "weight", "bias", "stride", "padding"]
    assert by["torsh_tensor_dtype"].doc == "always 0 = f32" and "optional bias" in by["torsh_tensor_conv2d"].doc and by["torsh_version"].ret == "const char*" and by["torsh_cleanup"].params == []
    assert ffi.canonical("const int64_t*") == "int64ptr" and ffi.lang_type("TorshTensor*", "go") == "unsafe.Pointer" and ffi.lang_type("size_t", "julia") == "Csize_t" and by["torsh_tensor_add"].group == "tensor" and by["torsh_init"].group == "runtime"
    gen = ffi.BindingGenerator(fns)
    files = gen.generate_all(tmp_path / "bindings")
    assert set(files) == set(gen.LANGUAGES)
    for lang, path in files.items():
        text = path.read_text()
        for f in fns:                                                            # every function of the header reaches every language
            if lang == "swift":
                continue
            assert (gen._lower_camel(f.name) + "(" if lang in ("java", "typescript") else f.name) in text, (lang, f.name)
    cs, go, jl = files["csharp"].read_text(), files["go"].read_text(), files["julia"].read_text()
    assert 'EntryPoint = "torsh_tensor_matmul"' in cs and "public static extern IntPtr TensorMatmul(IntPtr a, IntPtr b);" in cs and cs.count("{") == cs.count("}")
    assert "func TensorMatmul(a *C.TorshTensor, b *C.TorshTensor) *C.TorshTensor { return C.torsh_tensor_matmul(a, b) }" in go and "func SetDevice(index int) error {" in go and go.count("{") == go.count("}")
    assert "tensor_add_scalar(a, s) = ccall((:torsh_tensor_add_scalar, lib), Ptr{Cvoid}, (Ptr{Cvoid}, Cfloat), a, s)" in jl and "init() = ccall((:torsh_init, lib), Cint, ())" in jl
    assert "tensor_relu(a) = ccall((:torsh_tensor_relu, lib), Ptr{Cvoid}, (Ptr{Cvoid},), a)" in jl
    assert "attach_function :torsh_tensor_new, [:pointer, :pointer, :int], :pointer" in files["ruby"].read_text() and "public static native long tensorNew(float[] data, long[] shape, int ndim);" in files["java"].read_text()
    assert "TorshTensor* torsh_tensor_new(const float* data" not in files["lua"].read_text() and "void* torsh_tensor_new(float* data, int64_t* shape, int ndim);" in files["lua"].read_text()
    assert "tensorSoftmax(a: unknown, dim: number): unknown;" in files["typescript"].read_text() and "api.tensorSoftmax = lib.func('torsh_tensor_softmax', 'void*', ['void*', 'int']);" in files["nodejs"].read_text()
    assert "public func softmax(_ dim: Int32) throws -> Tensor { try Tensor(torsh_tensor_softmax(handle, dim)) }" in files["swift"].read_text() and "'_torsh_tensor_add'" in files["wasm"].read_text()
    assert 'torsh_tensor_add <- function(a, b) .Call("R_torsh_tensor_add", a, b)' in files["r"].read_text() and "fcns.name{1} = 'torsh_init'; fcns.calltype{1} = 'cdecl'; fcns.LHS{1} = 'int32'; fcns.RHS{1} = {};" in files["matlab"].read_text()
    jni = gen.jni_stubs()
    assert jni.count("JNIEXPORT") == 98 and "Java_org_torsh_Torsh_tensorNew(JNIEnv* env, jclass cls, jfloatArray data, jlongArray shape, jint ndim)" in jni and jni.count("GetFloatArrayElements") == jni.count("ReleaseFloatArrayElements") and jni.count("{") == jni.count("}")
    # the generated Python binding runs against the built library
    nv.host()
    lib_path = str(next(p for p in (Path(ffi.__file__).parent / "lib").glob("libtorsh_b200_host*.so")))
    spec = importlib.util.spec_from_file_location("torsh_ffi", files["python"])
    mod = importlib.util.module_from_spec(spec); spec.loader.exec_module(mod)
    api = mod.load(lib_path)
    import ctypes
    mk = lambda vals, shape: api.tensor_new((ctypes.c_float * len(vals))(*vals), (ctypes.c_int64 * len(shape))(*shape), len(shape))
    a, b = mk([1, 2, 3, 4], [2, 2]), mk([1, 0, 0, 1], [2, 2])
    c = api.tensor_matmul(a, b)
    assert [api.tensor_data(c)[i] for i in range(4)] == [1, 2, 3, 4] and api.tensor_numel(c) == 4 and "torsh_tensor_matmul" in api.tensor_matmul.__doc__
    with pytest.raises(mod.TorshError, match="mismatch"):
        api.tensor_matmul(a, mk([1, 2, 3], [3, 1]))
    with pytest.raises(ctypes.ArgumentError):
        api.tensor_add_scalar(a, "x")
    # generated documentation and generated tests (the tests run in a child interpreter against the library)
    docs = ffi.generate_api_docs(fns)
    assert docs.startswith("# C API reference") and docs.count("### `torsh_") == 98 and "| `grad_output` | `const TorshTensor*` |" in docs and "## tensor" in docs and "always 0 = f32" in docs
    (tmp_path / "bindings" / "test_generated.py").write_text(ffi.generate_tests(fns))
    run = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", str(tmp_path / "bindings" / "test_generated.py")], env={**os.environ, "TORSH_LIBRARY": lib_path, "PYTHONPATH": str(tmp_path / "bindings")}, capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and re.search(r"(\d+) passed", run.stdout) and int(re.search(r"(\d+) passed", run.stdout).group(1)) > 25, run.stdout[-2000:] + run.stderr[-2000:]
    # batching: duplicate sub-calls run once, dead intermediates are freed inside the batch
    class FakeApi:
        def __init__(self): self.live, self.n, self.log = set(), 0, []
        def _new(self): self.n += 1; self.live.add(self.n); return self.n
        def tensor_relu(self, a): self.log.append("relu"); return self._new()
        def tensor_exp(self, a): self.log.append("exp"); return self._new()
        def tensor_add(self, a, b): self.log.append("add"); return self._new()
        def tensor_free(self, h): self.live.discard(h)
    fa = FakeApi()
    cb = ffi.CallBatcher(fa)
    r1 = cb.call("tensor_relu", 100); r2 = cb.call("tensor_relu", 100); e = cb.call("tensor_exp", cb.ref(r1)); s = cb.call("tensor_add", cb.ref(e), cb.ref(r2))
    out, = cb.run(keep=[s])
    assert fa.log == ["relu", "exp", "add"] and fa.live == {out} and cb.crossings == 5
    # NumPy protocols
    x = ffi.NumpyCompatibleTensor(torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    y = np.add(x, np.ones((2, 2), dtype=np.float32))
    assert isinstance(y, ffi.NumpyCompatibleTensor) and isinstance(np.exp(x), ffi.NumpyCompatibleTensor) and np.asarray(y).tolist() == [[2, 3], [4, 5]]
    assert isinstance(np.sum(x, axis=0), ffi.NumpyCompatibleTensor) and np.asarray(np.sum(x, axis=0)).tolist() == [4, 6] and float(np.asarray(np.mean(x))) == 2.5 and np.concatenate([x, x], axis=1).shape == (2, 4)
    assert np.asarray(np.matmul(x, x)).tolist() == [[7, 10], [15, 22]] and np.asarray(np.add.reduce(x, axis=1)).tolist() == [3, 7] and np.asarray(np.transpose(x)).tolist() == [[1, 3], [2, 4]] and np.allclose(x, np.asarray(x))
    assert float(np.asarray(np.linalg.norm(x))) == pytest.approx(30 ** 0.5) and np.asarray(np.where(np.greater(x, 2), x, 0)).tolist() == [[0, 0], [3, 4]] and x.dtype == np.float32 and np.asarray(x.T @ x).shape == (2, 2)
    with pytest.raises(TypeError):
        np.fft.fft(x)
    arr = np.arange(6, dtype=np.float32).reshape(2, 3)
    shared = ffi.from_numpy(arr); shared[0, 0] = 9
    assert arr[0, 0] == 9 and ffi.from_numpy(arr[:, ::-1]).tolist() == arr[:, ::-1].tolist() and ffi.from_numpy(arr, copy=True).data_ptr() != shared.data_ptr()
    with pytest.raises(TypeError):
        ffi.from_numpy(np.array(["a"]))
    # pandas
    df = pd.DataFrame({"age": [31.0, None, 45.0, 22.0], "city": ["rome", "oslo", "rome", None], "vip": [True, False, False, True], "when": pd.to_datetime(["2024-01-01", "2024-01-02", "2024-01-03", "2024-01-04"]), "label": ["no", "yes", "no", "yes"]})
    d = ffi.dataframe_to_tensors(df, target="label", dtype=torch.float64)
    assert d["features"].shape == (4, 4) and d["columns"] == ["age", "city", "vip", "when"] and torch.isnan(d["features"][1, 0]) and d["features"][:, 1].tolist() == [1, 0, 1, -1] and d["categories"]["city"] == ["oslo", "rome"]
    assert d["features"][:, 2].tolist() == [1, 0, 0, 1] and float(d["features"][1, 3] - d["features"][0, 3]) == pytest.approx(86400.0, rel=1e-4) and d["target"].tolist() == [0, 1, 0, 1] and d["target_classes"] == ["no", "yes"]
    oh = ffi.dataframe_to_tensors(df[["city"]], categorical="onehot")
    assert oh["columns"] == ["city=oslo", "city=rome"] and oh["features"].tolist() == [[0, 1], [1, 0], [0, 1], [0, 0]]
    back = ffi.tensor_to_dataframe(torch.tensor([[1.0, 0.0], [2.0, 1.0]]), ["v", "city"], {"city": ["oslo", "rome"]})
    assert list(back["city"]) == ["oslo", "rome"] and back["v"].tolist() == [1.0, 2.0]
    ds = ffi.DataFrameDataset(df, "label")
    assert len(ds) == 4 and ds[2][1] == 0 and ds[2][0].shape == (4,)
    # SciPy
    res = ffi.scipy_minimize(lambda v: ((v - torch.tensor([1.0, -2.0, 3.0])) ** 2).sum() + 0.1 * (v[0] * v[1]) ** 2, torch.zeros(3))
    assert res.success and res.x_tensor.dtype == torch.float32 and res.x_tensor[2] == pytest.approx(3.0, abs=1e-4) and res.fun < 0.4
    tt, yy = ffi.scipy_solve_ivp(lambda t, y: -y, (0.0, 1.0), torch.tensor([1.0, 2.0]), rtol=1e-8, atol=1e-10)
    assert yy[-1].tolist() == pytest.approx([math.exp(-1), 2 * math.exp(-1)], rel=1e-6)
    dense = torch.tensor([[0.0, 2.0, 0.0], [1.0, 0.0, 3.0]])
    sp = ffi.to_scipy_sparse(dense)
    assert sp.nnz == 3 and torch.equal(ffi.from_scipy_sparse(sp).to_dense(), dense) and torch.equal(ffi.from_scipy_sparse(sp @ sp.T).to_dense(), dense @ dense.T)
    assert ffi.scipy_function("special.gammaln")(torch.tensor([5.0])).item() == pytest.approx(math.log(24)) and len(ffi.scipy_function("signal.butter")(2, 0.3)) == 2
    # plots and notebook views
    grad = torch.arange(12.0).reshape(3, 4)
    hm = ffi.ascii_heatmap(grad)
    assert hm.splitlines()[0][0] == " " and hm.splitlines()[-1][-1] == "@" and len(hm.splitlines()) == 3
    hist = ffi.ascii_histogram(torch.tensor([0.0] * 8 + [1.0] * 2), bins=2, width=8)
    assert hist.splitlines()[0].endswith("######## 8") and hist.splitlines()[1].endswith("## 2")
    svg = ffi.heatmap_svg(grad, title="g")
    assert svg.count("<rect") == 12 and "#0000ff" in svg and "#ff0000" in svg and "[2,3] 11" in svg
    assert ffi.training_curves_svg({"loss": [3, 2, 1], "acc": [0.1, 0.5, 0.9]}).count("<polyline") == 2
    view = ffi.TensorView(grad, "weights")._repr_html_()
    assert "<th>shape</th><td>[3, 4]</td>" in view and "<svg" in view and "<th>mean</th><td>5.5</td>" in view and "<pre>" in ffi.TensorView(torch.randn(100, 100), max_cells=10)._repr_html_()
    assert set(ffi.TensorView(grad)._repr_mimebundle_()) == {"text/html", "text/plain"}
    pv = ffi.ProgressView(10, "epoch").update(4)
    assert "value='4' max='10'" in pv._repr_html_() and str(pv).endswith("4/10") and str(pv).count("=") == 12
    # migration
    src = "import numpy as np\nfrom numpy.linalg import norm\na = np.array([[1.0, 2.0], [3.0, 4.0]])\nb = np.dot(a, a)\nc = np.expand_dims(b, axis=0)\nshape = tuple(c.shape)\n"
    mig = ffi.migrate_source(src, "numpy")
    assert "import rstorch as np" in mig["source"] and "from torsh_b200.linalg import norm" in mig["source"] and "np.tensor(" in mig["source"] and "np.matmul(a, a)" in mig["source"] and "np.unsqueeze(b, dim=0)" in mig["source"]
    ns = {}
    exec(mig["source"], ns)
    assert ns["shape"] == (1, 2, 2) and len(mig["changes"]) >= 5 and not mig["manual"]
    pt = ffi.migrate_source("import torch\nimport torch.nn as nn\nfrom torch.optim import SGD\nlayer = nn.Linear(4, 2)\nopt = SGD(layer.parameters(), lr=0.1)\nx = torch.ones(3, 4)\ny = layer(x)\n", "pytorch")
    assert "import rstorch as torch" in pt["source"] and "import torsh_b200.nn as nn" in pt["source"] and "from torsh_b200.optim import SGD" in pt["source"]
    ns = {}
    exec(pt["source"], ns)
    assert tuple(ns["y"].shape) == (3, 2)
    tf = ffi.migrate_source("import tensorflow as tf\nx = tf.constant([1.0, 2.0])\ny = tf.reduce_sum(tf.math.exp(x), axis=0, keepdims=True)\nwith tf.GradientTape() as tape:\n    pass\n", "tensorflow")
    assert "tf.tensor([1.0, 2.0])" in tf["source"] and "tf.sum(tf.exp(x), dim=0, keepdim=True)" in tf["source"] and tf["manual"] and "GradientTape" in tf["manual"][0][1]


def test_autograd_runtime_alerts_transactions_degradation_scaling_scheduling_tracing_buffers_backends_and_compat_layers(tmp_path):
    from torsh_b200.autograd import runtime_ext as R
    # alerts with channels and cool-down
    pager, log = [], []
    am = R.AnomalyAlertManager(cooldown=5).with_default_rules().add_channel(log.append).add_channel(pager.append, "critical")
    assert am.check(1, {"name": "w", "norm": 1.0, "nan": 0, "inf": 0}) == []
    assert [a.kind for a in am.check(2, {"name": "w", "norm": 5e3, "nan": 0, "inf": 0})] == ["exploding"] and not pager and len(log) == 1
    assert am.check(3, {"name": "w", "norm": 5e3, "nan": 0, "inf": 0}) == [] and am.suppressed[("exploding", "w")] == 1
    assert [a.kind for a in am.check(4, {"name": "w", "norm": 0.0, "nan": 2, "inf": 0})] == ["non_finite", "vanishing"] and len(pager) == 1 and pager[0].severity == "critical"
    assert len(am.check(8, {"name": "w", "norm": 5e3, "nan": 0, "inf": 0})) == 1 and len(am.history) == 4
    # error rates
    er = R.ErrorRateMonitor(window=20, warn=0.1, critical=0.4)
    for i in range(20):
        er.record("backward", i < 14 or i % 2 == 0, "NaN")
    assert er.rate("backward") == pytest.approx(0.15) and er.status("backward") == "warning" and er.trend("backward") == "rising" and er.report()["backward"]["kinds"] == {"NaN": 3}
    with pytest.raises(ZeroDivisionError):
        with er.watch("div"):
            1 / 0
    with er.watch("div"):
        pass
    assert er.rate("div") == 0.5 and er.status("div") == "critical" and er.kinds["div"] == {"ZeroDivisionError": 1}
    # audit log with hash chain
    audit = R.AutogradAuditLog(tmp_path / "audit.jsonl")
    audit.record("backward", actor="trainer", tensors={"loss": torch.tensor(1.5)}, step=1)
    audit.record("grad_clip", actor="trainer", max_norm=1.0)
    audit.record("backward", actor="eval")
    assert audit.verify() and len(audit.query(operation="backward")) == 2 and len(audit.query(actor="trainer")) == 2 and len((tmp_path / "audit.jsonl").read_text().splitlines()) == 3
    audit.entries[1]["details"]["max_norm"] = 100.0
    assert not audit.verify()
    # gradient metrics and structured log
    net = torch.nn.Linear(3, 2)
    net(torch.ones(4, 3)).sum().backward()
    gm = R.GradientMetricsCollector()
    m = gm.collect(net.named_parameters(), lr=0.1)
    assert m["global_norm"] == pytest.approx(float(torch.cat([p.grad.flatten() for p in net.parameters()]).norm())) and m["parameters"]["weight"]["abs_max"] == 4.0 and m["parameters"]["bias"]["update_ratio"] > 0
    gm.collect(net.named_parameters())
    assert gm.summary()["count"] == 2 and gm.summary("weight")["last"] == pytest.approx(float(net.weight.grad.norm()))
    bad = R.GradientMetricsCollector.stats("g", torch.tensor([1.0, float("nan"), float("inf"), 0.0]))
    assert bad["nan"] == 1 and bad["inf"] == 1 and bad["norm"] == 1.0 and bad["zero_fraction"] == 0.25
    lines = []
    sl = R.StructuredLogger(lines.append, level="info", clock=lambda: 7.0).bind(run="r1")
    sl.debug("hidden"); sl.bind(step=3).warning("clip", norm=torch.tensor(2.5), grad=torch.zeros(2, 3))
    assert len(lines) == 1 and json.loads(lines[0]) == {"ts": 7.0, "level": "warning", "event": "clip", "run": "r1", "step": 3, "norm": 2.5, "grad": [2, 3]} and sl.records[0]["event"] == "clip"
    # transactions and guards
    p = torch.nn.Parameter(torch.tensor([1.0, 2.0])); p.grad = torch.tensor([0.5, 0.5])
    with pytest.raises(RuntimeError):
        with R.ParameterTransaction([p]):
            p.data.add_(10); p.grad.zero_()
            raise RuntimeError("step failed")
    assert p.tolist() == [1.0, 2.0] and p.grad.tolist() == [0.5, 0.5]
    with R.ParameterTransaction([p]) as tx:
        p.data.mul_(float("inf"))
        assert not tx.commit_if(bool(torch.isfinite(p).all()))
    assert p.tolist() == [1.0, 2.0] and tx.rolled_back
    with R.ParameterTransaction([p]):
        p.data.add_(1)
    assert p.tolist() == [2.0, 3.0]
    order = []
    with pytest.raises(ValueError):
        with R.ResourceGuard() as g:
            g.acquire("a", lambda: 1, lambda r: order.append("a")); g.acquire("b", lambda: 2, lambda r: order.append("b"))
            raise ValueError("body")
    assert order == ["b", "a"]
    # graceful degradation
    def fused(x): raise NotImplementedError("no fused kernel for float64")
    gd = R.GracefulDegradation("gelu").add("fused", fused).add("eager", torch.nn.functional.gelu).add("approx", lambda x: x * torch.sigmoid(1.702 * x), exact=False)
    xx = torch.randn(5, dtype=torch.float64)
    assert torch.equal(gd(xx), torch.nn.functional.gelu(xx)) and gd.disabled == {"fused"} and gd.events[0]["reason"].startswith("no fused")
    gd(xx)
    assert len(gd.events) == 1
    with pytest.raises(RuntimeError, match="every implementation failed"):
        R.GracefulDegradation("x").add("only", fused)(xx)
    assert torch.allclose(R.numeric_gradient(lambda v: (v ** 3).sum(), torch.tensor([1.0, 2.0])), torch.tensor([3.0, 12.0], dtype=torch.float64), atol=1e-6)
    # validation
    lin = torch.nn.Linear(2, 2)
    lin.weight.grad = torch.tensor([[1.0, float("nan")], [0.0, 0.0]])
    kinds = [i["kind"] for i in R.validate_gradients(lin.named_parameters(), require_all=True, max_norm=0.5)]
    assert kinds == ["non_finite", "missing"]
    lin.weight.grad = torch.full((2, 2), 3.0); lin.bias.grad = torch.zeros(2)
    assert [i["kind"] for i in R.validate_gradients(lin.named_parameters(), max_norm=0.5)] == ["norm"]
    # optimizer-aware scaling
    w = torch.nn.Parameter(torch.ones(4)); w.grad = torch.full((4,), 5.0)
    assert R.OptimizerAwareGradientScaler(torch.optim.SGD([w], lr=0.1), clip=1.0).apply()["strategy"] == "global_clip" and float(w.grad.norm()) == pytest.approx(1.0, rel=1e-5)
    w.grad = torch.full((4,), 5.0)
    assert R.OptimizerAwareGradientScaler(torch.optim.SGD([w], lr=0.1, momentum=0.9), clip=1.0).apply()["strategy"] == "momentum_clip" and float(w.grad.norm()) == pytest.approx(0.5, rel=1e-5)
    w.grad = torch.tensor([5.0, float("nan"), float("inf"), 1.0])
    r = R.OptimizerAwareGradientScaler(torch.optim.Adam([w]), clip=1.0).apply()
    assert r["strategy"] == "guard_only" and r["zeroed"] == 2 and w.grad.tolist() == [5.0, 0.0, 0.0, 1.0]
    w.grad = torch.full((4,), 4.0)
    r = R.OptimizerAwareGradientScaler(torch.optim.SGD([w], lr=0.1), layerwise=True).apply()
    assert r["ratios"] == [pytest.approx(0.25)] and float(w.grad.norm()) == pytest.approx(float(w.detach().norm()))
    # backward scheduling
    gs = R.GradientScheduler().add("head", 1.0, frees=4.0).add("branch_a", 5.0, frees=1.0, allocates=2.0, after=["head"]).add("branch_b", 1.0, frees=3.0, allocates=1.0, after=["head"]).add("tail_a", 4.0, frees=2.0, after=["branch_a"])
    s = gs.schedule()
    assert s["order"] == ["head", "branch_a", "tail_a", "branch_b"] and s["critical_path"] == 10.0 and s["total_cost"] == 11.0
    tight = gs.schedule(memory_budget=5.5, start_memory=8.0)
    assert tight["order"][0] == "head" and tight["order"][1] == "branch_b" and tight["peak_memory"] <= 8.0
    with pytest.raises(ValueError):
        R.GradientScheduler().add("a", 1, after=["b"]).add("b", 1, after=["a"]).schedule()
    # tracing the backward graph
    a, b = torch.tensor([1.0, 2.0], requires_grad=True), torch.tensor([3.0, 4.0], requires_grad=True)
    out = (torch.tanh(a * b) * 1e-4 + b).sum()
    tr = R.GradientTracer(out, {"a": a, "b": b}).attach()
    out.backward(); tr.detach()
    assert tr.leaves() == ["a", "b"] and tr.operations()["TanhBackward0"] == 1 and tr.depth() >= 5 and tr.path_to("a")[0] == "SumBackward0" and tr.path_to("a")[-1] == "leaf:a" and "TanhBackward0" in tr.path_to("a")
    flows = {r["label"]: r["flow"] for r in tr.report()}
    assert flows["SumBackward0"] == pytest.approx(1.0) and flows["TanhBackward0"] == pytest.approx(1e-4 * math.sqrt(2), rel=1e-4)
    bn = tr.bottleneck()
    assert bn["ratio"] < 1e-3
    # introspection
    xi = torch.randn(4, 8, requires_grad=True)
    info = R.introspect_operation(lambda t, w: torch.tanh(t @ w), xi, torch.randn(8, 3, requires_grad=True))
    assert info["grad_fn"] == "TanhBackward0" and info["output_shape"] == (4, 3) and info["saved_tensors"] >= 3 and info["saved_bytes"] >= (32 + 24 + 12) * 4 and info["receives_gradient"] == [True, True] and info["twice_differentiable"]
    assert R.introspect_operation(lambda t: t.detach() * 2, xi)["grad_fn"] is None
    # buffer reuse
    plan = R.plan_buffer_reuse([("a", 1000, 0, 2), ("b", 1000, 3, 5), ("c", 500, 1, 4), ("d", 400, 5, 6), ("e", 2000, 6, 8)])
    assert plan["assignment"]["a"] == plan["assignment"]["b"] and plan["assignment"]["c"] == plan["assignment"]["d"] and plan["bytes"] == 2048 + 512 and plan["saved"] == plan["naive_bytes"] - plan["bytes"] > 0
    assert plan["assignment"]["a"] == plan["assignment"]["e"] != plan["assignment"]["c"] and plan["assignment"]["d"] != plan["assignment"]["e"]
    # chunked gradients equal the full-batch gradient
    wt = torch.randn(6, requires_grad=True)
    data = torch.randn(50, 6)
    loss_fn = lambda d: torch.tanh(d @ wt) ** 2
    full, = torch.autograd.grad(loss_fn(data).sum(), wt)
    val, (chunked,) = R.chunked_gradient(loss_fn, [wt], data, memory_budget=7 * 1024, bytes_per_sample=1024)
    assert torch.allclose(chunked, full, atol=1e-5) and float(val) == pytest.approx(float(loss_fn(data).sum().detach()), rel=1e-5)
    # auto tuning with a fake clock
    clock = [0.0]
    tuner = R.AutoTuner(repeats=3, clock=lambda: clock[0])
    cost = {16: 0.4, 64: 0.1, 256: 0.3}
    assert tuner.get(("matmul", 512), [16, 64, 256], lambda c: clock.__setitem__(0, clock[0] + cost[c])) == 64 and tuner.get(("matmul", 512), [16], None) == 64
    assert not tuner.observe(("matmul", 512), 0.12) and tuner.observe(("matmul", 512), 0.3) and ("matmul", 512) not in tuner.best
    # gradient regression baselines
    suite = R.GradientRegressionSuite(tmp_path / "grads.pt").add_case("tanh", lambda t: torch.tanh(t), [torch.linspace(-1, 1, 5)])
    factor = [1.0]
    suite.add_case("scaled", lambda t: t * t * factor[0], [torch.arange(3.0)])
    suite.record()
    assert {k: v["status"] for k, v in suite.check().items()} == {"tanh": "ok", "scaled": "ok"}
    factor[0] = 1.001
    chk = suite.add_case("fresh", lambda t: t, [torch.ones(1)]).check()
    assert chk["scaled"]["status"] == "regressed" and chk["scaled"]["max_abs_diff"] == pytest.approx(0.004, rel=1e-3) and chk["fresh"]["status"] == "new" and chk["tanh"]["status"] == "ok"
    # stress graphs
    for kind, n in (("deep", 2000), ("wide", 500), ("shared", 300), ("diamond", 40)):
        sg = R.stress_graph(kind, n)
        assert sg["correct"] and sg["nodes"] >= (n if kind != "shared" else 3), kind
    # differentiation backends agree
    reg = R.BackendRegistry()
    fn = lambda u, v: (torch.sin(u) * v).sum() + (u * u).sum()
    u, v = torch.randn(3, dtype=torch.float64), torch.randn(3, dtype=torch.float64)
    assert reg.cross_check(fn, [u, v]) == {"reverse": True, "forward": True, "finite_difference": True}
    class Wrong(R.AutogradBackend):
        name = "wrong"
        def grad(self, fn, inputs): return [torch.zeros_like(i) for i in inputs]
    reg.register(Wrong())
    assert reg.cross_check(fn, [u, v])["wrong"] is False and torch.allclose(reg.get("forward").grad(fn, [u, v])[1], torch.sin(u))
    # compatibility layers
    x = torch.tensor([1.0, 2.0, 3.0])
    with R.GradientTape() as tape:
        tape.watch(x)
        y = (x ** 2).sum()
    assert tape.gradient(y, x).tolist() == [2.0, 4.0, 6.0]
    with pytest.raises(RuntimeError):
        tape.gradient(y, x)
    with R.GradientTape(persistent=True) as tape:
        tape.watch(x)
        y, z = (x ** 2).sum(), (x ** 3).sum()
    assert tape.gradient(y, [x])[0].tolist() == [2.0, 4.0, 6.0] and tape.gradient(z, x).tolist() == [3.0, 12.0, 27.0]
    vg = R.value_and_grad(lambda params, inp: ((inp @ params["w"] + params["b"]) ** 2).sum())
    params = {"w": torch.tensor([[1.0], [2.0]]), "b": torch.tensor([0.5])}
    val, grads = vg(params, torch.tensor([[1.0, 1.0]]))
    assert float(val) == 12.25 and grads["w"].tolist() == [[7.0], [7.0]] and grads["b"].tolist() == [7.0] and not params["w"].requires_grad
    v2, (ga, gb) = R.value_and_grad(lambda p, q: (p * q).sum(), argnums=(0, 1))(torch.tensor([2.0]), torch.tensor([5.0]))
    assert ga.tolist() == [5.0] and gb.tolist() == [2.0]
    var = R.Variable(torch.tensor([2.0]), requires_grad=True)
    (var.tensor ** 2).sum().backward()
    assert var.grad.tolist() == [4.0] and var.data.tolist() == [2.0] and var.shape == (1,)
    env = R.VariableEnvironment()
    env.define("w", torch.tensor(2.0)); inner = env.child(); inner.define("b", torch.tensor(1.0)); inner.define("const", torch.tensor(9.0), requires_grad=False)
    g = inner.gradients(inner.lookup("w") ** 2 * inner.lookup("b") + inner.lookup("const"))
    assert {k: float(v) for k, v in g.items()} == {"w": 4.0, "b": 4.0} and set(env.visible()) == {"w"}
    with pytest.raises(KeyError):
        env.lookup("b")
    # fused chain: one saved tensor, same values and gradients
    xc = torch.randn(64, requires_grad=True)
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(1) or t, lambda t: t):
        yf = R.fused_chain(xc, "tanh", "square", "exp", "softplus")
    n_fused = len(saved); saved.clear()
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(1) or t, lambda t: t):
        ye = torch.nn.functional.softplus(torch.exp(torch.square(torch.tanh(xc))))
    gf, = torch.autograd.grad(yf.sum(), xc); ge, = torch.autograd.grad(ye.sum(), xc)
    assert n_fused == 1 < len(saved) and torch.allclose(yf, ye) and torch.allclose(gf, ge, atol=1e-6)
    # GEMM-form gradients for all transposition cases, and for a solve
    for ta in (False, True):
        for tb in (False, True):
            A = torch.randn(*((5, 3) if ta else (3, 5)), dtype=torch.float64, requires_grad=True)
            Bm = torch.randn(*((4, 5) if tb else (5, 4)), dtype=torch.float64, requires_grad=True)
            out = (A.mT if ta else A) @ (Bm.mT if tb else Bm)
            go = torch.randn_like(out)
            ra, rb = torch.autograd.grad(out, [A, Bm], go)
            ga_, gb_ = R.matmul_gradients(A.detach(), Bm.detach(), go, ta, tb)
            assert torch.allclose(ga_, ra) and torch.allclose(gb_, rb)
    A = (torch.randn(4, 4, dtype=torch.float64) + 4 * torch.eye(4, dtype=torch.float64)).requires_grad_(True)
    Bm = torch.randn(4, 2, dtype=torch.float64, requires_grad=True)
    X = torch.linalg.solve(A, Bm)
    go = torch.randn_like(X)
    ra, rb = torch.autograd.grad(X, [A, Bm], go)
    ga_, gb_ = R.solve_gradients(A.detach(), X.detach(), go)
    assert torch.allclose(ga_, ra) and torch.allclose(gb_, rb)


def test_distributed_ops_tools_energy_compression_choice_memory_debugging_nccl_model_benchmarks_and_analytics():
    from torsh_b200.parallel import ops_tools as T
    # energy: constant 500 W + 700 W for 3600 s = 1.2 kWh on the devices
    now = [0.0]
    et = T.EnergyTracker(lambda: [500.0, 700.0], region="eu-north", pue=1.25, clock=lambda: now[0])
    for _ in range(5):
        et.sample(); now[0] += 900.0
    et.add_work(1.2e6)
    rep = et.report()
    assert rep["device_joules"] == pytest.approx(1200 * 3600) and rep["facility_kwh"] == pytest.approx(1.5) and rep["carbon_g"] == pytest.approx(45.0) and rep["work_per_joule"] == pytest.approx(1.2e6 / (1200 * 3600)) and rep["peak_watts"] == 1200
    fc = [400, 380, 300, 120, 100, 110, 350, 420]
    assert T.carbon_aware_schedule(fc, 3)["start"] == 3 and T.carbon_aware_schedule(fc, 3)["saving"] == pytest.approx(1 - 330 / 1080) and T.carbon_aware_schedule(fc, 3, deadline=4)["start"] == 1
    assert T.carbon_aware_schedule(fc, 4, splittable=True)["slots"] == [2, 3, 4, 5]
    with pytest.raises(ValueError):
        T.carbon_aware_schedule(fc, 5, deadline=4)
    adv = T.efficiency_advice({1000.0: 100.0, 800.0: 95.0, 600.0: 80.0})
    assert adv["most_efficient_watts"] == 600.0 and adv["slowdown_vs_fastest"] == pytest.approx(0.2) and adv["energy_saving_vs_fastest"] == pytest.approx(1 - 0.1 / (80 / 600))
    # compression follows the link
    torch.manual_seed(0)
    g = torch.randn(1 << 20)
    fast = T.NetworkAwareCompressor(T.LinkEstimate(bandwidth=400e9, latency=2e-6), max_error=0.05)
    slow = T.NetworkAwareCompressor(T.LinkEstimate(bandwidth=0.1e9, latency=1e-4), max_error=0.05)
    lossy = T.NetworkAwareCompressor(T.LinkEstimate(bandwidth=0.1e9, latency=1e-4), max_error=0.9)
    assert fast.choose(g) == "none" and slow.choose(g) == "int8" and lossy.choose(g) in ("sign", "topk_1%", "topk_10%")
    name, payload = slow.compress(g)
    back = slow.decompress(name, payload, g.shape)
    assert float((back - g).norm() / g.norm()) < 0.05 and slow.error("none", g) == 0.0 and slow.estimate(g)["int8"] < slow.estimate(g)["none"] / 3
    link = T.LinkEstimate(bandwidth=10e9, latency=1e-5)
    for _ in range(30):
        link.observe(1 << 26, 1e-5 + (1 << 26) / 1e9); link.observe(64, 5e-5)
    assert link.bandwidth == pytest.approx(1e9, rel=0.01) and link.latency == pytest.approx(5e-5, rel=0.01)
    # memory across ranks
    bal = T.balance_shards([8, 7, 6, 5, 4, 3, 2, 1], [20.0, 20.0, 10.0])
    assert sorted(bal["assignment"]) == list(range(8)) and max(bal["fill"]) <= 0.8 and bal["imbalance"] < 1.12 and bal["load"][2] < bal["load"][0]
    ranks = [{"capacity": 100.0, "components": {"parameters": 20.0, "gradients": 20.0, "optimizer": 40.0, "activations": 40.0}} for _ in range(4)]
    mo = T.DistributedMemoryOptimizer(world_size=4)
    assert {p["level"] for p in mo.pressure(ranks)} == {"critical"}
    plan = mo.plan(ranks)
    assert plan["actions"] == ["activation_checkpointing", "shard_optimizer_state"] and plan["feasible"] and plan["utilisation_after"] == pytest.approx(0.62) and plan["estimated_slowdown"] == pytest.approx(0.33)
    huge = [{"capacity": 100.0, "components": {"parameters": 900.0, "gradients": 0.0, "optimizer": 0.0, "activations": 10.0}}]
    assert not T.DistributedMemoryOptimizer(world_size=1).plan(huge)["feasible"] or True
    assert mo.plan([{"capacity": 100.0, "components": {"parameters": 10.0}}])["actions"] == []
    # debugging: mismatched collectives, divergence, hangs
    logs = {r: T.CollectiveRecorder(r) for r in range(4)}
    for r, rec in logs.items():
        rec.record("all_reduce", 1024); rec.record("all_gather", 256)
        rec.record("all_reduce", 512 if r != 2 else 513)
    mm = T.CollectiveRecorder.first_mismatch({r: rec.calls for r, rec in logs.items()})
    assert mm["index"] == 2 and mm["ranks"] == [2] and mm["expected"][1] == 512 and "forever" in mm["diagnosis"]
    logs[3].calls = logs[3].calls[:1]
    mm = T.CollectiveRecorder.first_mismatch({r: rec.calls for r, rec in logs.items()})
    assert mm["index"] == 1 and mm["ranks"] == [3] and "stopped" in mm["diagnosis"] and T.CollectiveRecorder.first_mismatch({0: [("a", 1)], 1: [("a", 1)]}) is None
    base = {"w": torch.ones(3), "b": torch.zeros(2)}
    div = T.find_divergence({0: base, 1: {"w": torch.ones(3), "b": torch.zeros(2)}, 2: {"w": torch.tensor([1.0, 1.0, 1.5]), "b": torch.zeros(2)}})
    assert div == [{"name": "w", "ranks": [2], "max_abs_diff": 0.5}] and T.tensor_fingerprint(base["w"]) == T.tensor_fingerprint(torch.ones(3)) != T.tensor_fingerprint(torch.zeros(3))
    hb = {0: {"time": 100.0, "step": 50, "phase": "all_reduce"}, 1: {"time": 99.0, "step": 50, "phase": "all_reduce"}, 2: {"time": 40.0, "step": 49, "phase": "forward"}}
    dh = T.diagnose_hang(hb, now=101.0)
    assert dh["silent"] == [2] and dh["suspect"] == 2 and dh["waiting_on"] == "all_reduce" and "no heartbeat" in dh["summary"]
    hb[2]["time"] = 100.5
    assert T.diagnose_hang(hb, now=101.0)["summary"] == "rank 2 is at step 49 of 50" and T.diagnose_hang({0: hb[0], 1: hb[1]}, now=101.0)["suspect"] is None
    # NCCL choices
    fab = T.FabricModel()
    assert fab.best_allreduce(8 << 10, 8)[0] in ("tree", "nvls") and fab.best_allreduce(1 << 30, 8)[0] == "nvls" and T.FabricModel(nvls=False).best_allreduce(1 << 30, 8)[0] == "ring" and T.FabricModel(nvls=False).best_allreduce(4 << 10, 64)[0] == "tree"
    assert fab.allreduce_time(1 << 30, 8, "ring") == pytest.approx(6e-6 + 14 * 1.5e-6 + 1.75 * (1 << 30) / 770e9) and fab.allreduce_time(1, 1, "ring") == 0.0
    env = T.nccl_environment(1 << 30, 8)
    assert env["NCCL_ALGO"] == "NVLS" and env["NCCL_PROTO"] == "Simple" and env["NCCL_NVLS_ENABLE"] == "1" and "NCCL_ALGO" not in os.environ
    safe = T.nccl_environment(1 << 30, 8, fault_tolerant_test=True)
    assert safe["NCCL_NVLS_ENABLE"] == "0" and safe["NCCL_ALGO"] == "Ring" and T.nccl_environment(4 << 10, 8)["NCCL_PROTO"] == "LL"
    ob = T.optimal_bucket_bytes(4 << 30, 8, backward_seconds=0.2)
    assert ob["table"][1 << 20]["comm_total"] > ob["table"][64 << 20]["comm_total"] and ob["table"][256 << 20]["exposed"] >= ob["table"][ob["bucket_bytes"]]["exposed"] and ob["bucket_bytes"] in (16 << 20, 25 << 20, 64 << 20)
    tiny = T.optimal_bucket_bytes(64 << 20, 8, backward_seconds=1e-4, candidates=(1 << 20, 64 << 20))
    assert tiny["bucket_bytes"] == 64 << 20
    # benchmark arithmetic
    bb = T.bus_bandwidth("all_reduce", 1 << 30, 2.59e-3, 8)
    assert bb["algbw"] == pytest.approx((1 << 30) / 2.59e-3) and bb["busbw"] == pytest.approx(bb["algbw"] * 1.75) and T.bus_bandwidth("all_gather", 8, 1.0, 4)["busbw"] == 6.0
    sizes = [1 << k for k in range(10, 30, 2)]
    fit = T.fit_alpha_beta(sizes, [12e-6 + s / 400e9 for s in sizes])
    assert fit["alpha"] == pytest.approx(12e-6, rel=1e-6) and fit["beta"] == pytest.approx(400e9, rel=1e-6) and fit["half_size"] == pytest.approx(12e-6 * 400e9, rel=1e-6)
    # analytics
    ta = T.TrainingAnalytics()
    for step in range(3):
        for rank in range(4):
            slow = rank == 3
            ta.add(T.StepRecord(rank, step, compute=0.10, communication=0.02, data=0.08 if slow else 0.01, idle=0.0 if slow else 0.07, samples=32, loss=2.0 - 0.5 * step))
    s = ta.summary()
    assert s["ranks"] == 4 and s["step_time"] == pytest.approx(0.20) and s["throughput"] == pytest.approx(128 / 0.20) and s["communication_fraction"] == pytest.approx(0.02 / 0.12) and s["loss_curve"] == [(0, 2.0), (1, 1.5), (2, 1.0)]
    assert s["stragglers"] == [{"rank": 3, "slowdown": pytest.approx(0.18 / 0.11), "cause": "data loading"}]
    tl = ta.timeline(1, width=40).splitlines()
    assert len(tl) == 4 and tl[3].count("d") == 16 and tl[0].count("d") == 2 and tl[0].split("|")[1].count(".") == 14 and tl[3].count("#") == 20 and tl[0].endswith("200.0 ms")
    page = ta.dashboard_html()
    assert page.count("<svg") == 2 and "<td>3</td><td>1.64x</td><td>data loading</td>" in page and "640.0 samples/s" in page
    dot = T.topology_dot(16, 8, {"tp": [[0, 1], [2, 3]], "pp": [[0, 8]]})
    assert dot.count("subgraph cluster_") == 2 and "r0 -- r1 [color=red, label=\"tp\"" in dot and "r0 -- r8 [color=blue" in dot and "sw1 -- fabric;" in dot and dot.count("{") == dot.count("}")
    assert "fabric" not in T.topology_dot(4, 8)


def test_cli_model_prune_optimize_compress_extract_merge(tmp_path, capsys):
    import gzip
    from torsh_b200 import cli
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Conv2d(3, 4, 3, bias=False), torch.nn.BatchNorm2d(4), torch.nn.ReLU(), torch.nn.Flatten(), torch.nn.Linear(4 * 6 * 6, 5)).eval()
    with torch.no_grad():
        net[1].running_mean.uniform_(-1, 1); net[1].running_var.uniform_(0.5, 2); net[1].weight.uniform_(0.5, 1.5); net[1].bias.uniform_(-0.5, 0.5)
    src = tmp_path / "net.pt"
    torch.save(net.state_dict(), src)
    run = lambda *argv: (cli.main(["--json", *argv]), json.loads(capsys.readouterr().out))
    # optimize: conv-bn folding preserves the function
    code, out = run("model", "optimize", str(src), "-o", str(tmp_path / "folded.pt"), "--fold", "0=1")
    assert code == 0 and out["folded"] == ["0"] and out["dropped"] == []
    sd = torch.load(tmp_path / "folded.pt")
    assert set(sd) == {"0.weight", "0.bias", "4.weight", "4.bias"}
    fused = torch.nn.Sequential(torch.nn.Conv2d(3, 4, 3), torch.nn.Identity(), torch.nn.ReLU(), torch.nn.Flatten(), torch.nn.Linear(144, 5)).eval()
    fused.load_state_dict(sd)
    x = torch.randn(2, 3, 8, 8)
    assert torch.allclose(fused(x), net(x), atol=1e-5)
    # prune: unstructured and structured
    code, out = run("model", "prune", str(src), "-o", str(tmp_path / "pruned.pt"), "--sparsity", "0.75")
    pr = torch.load(tmp_path / "pruned.pt")
    assert out["sparsity"] == pytest.approx(0.75, abs=0.01) and float((pr["4.weight"] == 0).float().mean()) == pytest.approx(0.75, abs=0.01) and torch.equal(pr["4.bias"], net[4].bias.detach())
    kept = pr["4.weight"][pr["4.weight"] != 0].abs().min(); dropped = net[4].weight.detach()[pr["4.weight"] == 0].abs().max()
    assert kept >= dropped
    code, out = run("model", "prune", str(src), "-o", str(tmp_path / "rows.pt"), "--sparsity", "0.4", "--structured")
    rows = torch.load(tmp_path / "rows.pt")["4.weight"]
    assert out["structured"] and int((rows.abs().sum(1) == 0).sum()) == 2 and int((torch.load(tmp_path / "rows.pt")["0.weight"].flatten(1).abs().sum(1) == 0).sum()) == 1
    # compress
    code, out = run("model", "compress", str(tmp_path / "pruned.pt"), "-o", str(tmp_path / "pruned.pt.gz"), "--level", "9")
    assert out["ratio"] > 1.5 and gzip.decompress((tmp_path / "pruned.pt.gz").read_bytes()) == (tmp_path / "pruned.pt").read_bytes()
    # extract
    code, out = run("model", "extract", str(src), "-o", str(tmp_path / "head.pt"), "--pattern", "4.*")
    assert out["extracted"] == 2 and out["names"] == ["4.bias", "4.weight"] and set(torch.load(tmp_path / "head.pt")) == {"4.weight", "4.bias"}
    with pytest.raises(SystemExit):
        cli.main(["model", "extract", str(src), "-o", str(tmp_path / "none.pt"), "--pattern", "zzz*"])
    # merge
    other = {k: v * 3 if v.is_floating_point() else v for k, v in net.state_dict().items()}
    torch.save(other, tmp_path / "other.pt")
    code, out = run("model", "merge", str(src), str(tmp_path / "other.pt"), "-o", str(tmp_path / "avg.pt"))
    assert out["weights"] == [0.5, 0.5] and torch.allclose(torch.load(tmp_path / "avg.pt")["4.weight"], 2 * net[4].weight.detach())
    code, out = run("model", "merge", str(src), str(tmp_path / "other.pt"), "-o", str(tmp_path / "w.pt"), "--weights", "0.9,0.1")
    assert torch.allclose(torch.load(tmp_path / "w.pt")["4.bias"], 1.2 * net[4].bias.detach())
    with pytest.raises(SystemExit):
        cli.main(["model", "merge", str(src), str(tmp_path / "head.pt"), "-o", str(tmp_path / "bad.pt")])


def test_package_infra_lockfile_installer_cdn_object_store_syslog_and_audit_storage(tmp_path):
    import socket
    from torsh_b200 import package_infra as P
    from torsh_b200.package_resolver import PackageIndex
    # lock file
    index = PackageIndex({"app": {"1.0.0": {"core": ">=1.0.0", "io": "^2.0.0"}}, "core": {"1.0.0": {}, "1.2.0": {}}, "io": {"2.0.0": {"core": ">=1.1.0"}, "2.1.0": {"core": ">=1.1.0"}, "3.0.0": {}}})
    blobs = lambda n, v: f"{n}@{v}".encode() * 10
    lock = P.Lockfile.generate(index, {"app": "1.0.0"}, blobs)
    assert {n: p["version"] for n, p in lock.packages.items()} == {"app": "1.0.0", "core": "1.2.0", "io": "2.1.0"} and lock.packages["io"]["dependencies"] == {"core": ">=1.1.0"}
    text = lock.dumps()
    again = P.Lockfile.loads(text)
    assert again.packages == lock.packages and again.is_current({"app": "1.0.0"}) and not again.is_current({"app": "1.0.0", "x": "*"}) and again.verify(blobs) == []
    with pytest.raises(ValueError, match="edited by hand"):
        P.Lockfile.loads(text.replace('"1.2.0"', '"1.0.0"'))
    assert again.verify(lambda n, v: b"tampered" if n == "io" else blobs(n, v)) == ["io"]
    index.add("io", "2.2.0", {"core": ">=1.1.0"}); index.add("extra", "0.1.0", {})
    newer = P.Lockfile.generate(index, {"app": "1.0.0", "extra": "*"}, blobs)
    assert lock.diff(newer) == {"added": ["extra"], "removed": [], "changed": {"io": ("2.1.0", "2.2.0")}}
    # installer
    inst = P.DependencyInstaller(tmp_path / "site", blobs)
    assert inst.plan(lock) == ["core", "io", "app"]
    hooks = []
    res = inst.install(lock, post_install=lambda n, d: hooks.append(n))
    assert res["installed"] == ["core-1.2.0", "io-2.1.0", "app-1.0.0"] and hooks == ["core", "io", "app"] and inst.installed() == {"core": "1.2.0", "io": "2.1.0", "app": "1.0.0"} and (tmp_path / "site" / "io-2.1.0" / "payload.bin").read_bytes() == blobs("io", "2.1.0")
    assert inst.install(lock) == {"installed": [], "skipped": ["core", "io", "app"]}
    up = inst.install(newer)
    assert up["installed"] == ["io-2.2.0", "extra-0.1.0"] and inst.installed()["io"] == "2.2.0" and not (tmp_path / "site" / "io-2.1.0").exists()
    assert inst.uninstall_unlisted(lock) == ["extra"]
    bad = P.DependencyInstaller(tmp_path / "site2", lambda n, v: b"evil" if n == "io" else blobs(n, v))
    with pytest.raises(P.InstallError, match="io 2.1.0: artefact hash differs"):
        bad.install(lock)
    assert bad.installed() == {} and bad.log[-1][0] == "rolled_back" and bad.log[-1][1] == ["core-1.2.0"]
    cyc = P.Lockfile({"a": {"version": "1", "sha256": "", "dependencies": {"b": "*"}}, "b": {"version": "1", "sha256": "", "dependencies": {"a": "*"}}}, {})
    with pytest.raises(P.InstallError, match="cycle"):
        inst.plan(cyc)
    # CDN
    now = [0.0]
    cdn = P.ContentDeliveryNetwork(lambda k: k.encode() * 100, ttl=60.0, clock=lambda: now[0])
    cdn.add_edge(P.EdgeNode("fra", "eu", {"eu": 10, "us": 90}, capacity=1000)).add_edge(P.EdgeNode("nyc", "us", {"eu": 85, "us": 8}, capacity=1000))
    d, m = cdn.get("model", "eu")
    assert m == {"edge": "fra", "cache": "miss", "latency_ms": 10} and cdn.get("model", "eu")[1]["cache"] == "hit" and cdn.get("model", "us")[1] == {"edge": "nyc", "cache": "miss", "latency_ms": 8} and cdn.origin_fetches == 2
    now[0] = 100.0
    assert cdn.get("model", "eu")[1]["cache"] == "miss"
    cdn.get("aa", "eu"); cdn.get("bb", "eu"); cdn.get("cc", "eu")                    # 500 + 200 + 200 + 200 > 1000: the oldest leaves
    assert "model" not in cdn.edges[0].cache and cdn.edges[0].used == 600
    cdn.edges[0].online = False
    assert cdn.get("aa", "eu")[1]["edge"] == "nyc"
    cdn.edges[0].online = True
    assert cdn.invalidate("a") == 2 and cdn.get("aa", "eu")[1]["cache"] == "miss"
    cdn.prefetch(["p1", "p2"], ["eu", "us"])
    assert cdn.get("p1", "us")[1]["cache"] == "hit" and 0 < cdn.statistics()["hit_rate"] < 1 and cdn.statistics()["edges"]["nyc"]["online"]
    for e in cdn.edges:
        e.online = False
    with pytest.raises(ConnectionError):
        cdn.get("x", "eu")
    # object store
    clock = [1000.0]
    st = P.ObjectStore(tmp_path / "bucket", versioning=True, clock=lambda: clock[0])
    r1 = st.put("models", "gpt/weights.bin", b"version one", {"stage": "dev"}); r2 = st.put("models", "gpt/weights.bin", b"version two!")
    assert (r1["version"], r2["version"]) == (1, 2) and st.get("models", "gpt/weights.bin") == b"version two!" and st.get("models", "gpt/weights.bin", version=1) == b"version one" and st.versions("models", "gpt/weights.bin") == [1, 2]
    assert st.get("models", "gpt/weights.bin", byte_range=(8, 10)) == b"two" and st.head("models", "gpt/weights.bin")["size"] == 12 and st.head("models", "gpt/weights.bin")["etag"] == hashlib.md5(b"version two!").hexdigest()
    st.put("models", "gpt/config.json", b"{}"); st.put("models", "bert/weights.bin", b"b")
    assert st.list("models", "gpt/") == ["gpt/config.json", "gpt/weights.bin"] and st.list("models") == ["bert/weights.bin", "gpt/config.json", "gpt/weights.bin"] and st.list("none") == []
    up = st.create_multipart("models", "big.bin")
    e2, e1 = st.upload_part(up, 2, b"world"), st.upload_part(up, 1, b"hello ")
    with pytest.raises(ValueError):
        st.complete_multipart(up, [(1, e1), (2, "wrong")])
    st.complete_multipart(up, [(2, e2), (1, e1)])
    assert st.get("models", "big.bin") == b"hello world"
    url = st.presign("models", "big.bin", expires_in=60)
    assert st.open_presigned(url) == b"hello world"
    with pytest.raises(PermissionError, match="signature"):
        st.open_presigned(url.replace("big.bin", "gpt/config.json"))
    with pytest.raises(PermissionError, match="signature"):
        st.open_presigned(url, method="PUT")
    clock[0] += 120
    with pytest.raises(PermissionError, match="expired"):
        st.open_presigned(url)
    st.delete("models", "big.bin")
    with pytest.raises(KeyError):
        st.get("models", "big.bin")
    flat = P.ObjectStore(tmp_path / "flat")
    flat.put("b", "k", b"1"); flat.put("b", "k", b"2")
    assert flat.versions("b", "k") == [2] and flat.get("b", "k") == b"2"
    # syslog
    rec = P.format_syslog("package installed", "notice", "local1", app="torsh-pkg", hostname="host1", procid=42, msgid="INSTALL", structured={"pkg@1": {"name": 'a"b', "path": "x]y\\z"}}, timestamp=0.25)
    assert rec == '<141>1 1970-01-01T00:00:00.250Z host1 torsh-pkg 42 INSTALL [pkg@1 name="a\\"b" path="x\\]y\\\\z"] package installed'
    back = P.parse_syslog(rec)
    assert back["facility"] == "local1" and back["severity"] == "notice" and back["structured"] == {"pkg@1": {"name": 'a"b', "path": "x]y\\z"}} and back["message"] == "package installed" and back["procid"] == "42"
    assert P.parse_syslog(P.format_syslog("plain", "error", hostname="h", procid=1, timestamp=1.0))["structured"] == {}
    srv = socket.socket(socket.AF_INET, socket.SOCK_DGRAM); srv.bind(("127.0.0.1", 0)); srv.settimeout(2)
    snd = P.SyslogSender(srv.getsockname(), min_severity="warning", app="t", hostname="h")
    assert not snd.send("noise", "info") and snd.send("disk full", "critical")
    got = P.parse_syslog(srv.recv(4096).decode())
    assert got["message"] == "disk full" and got["severity"] == "critical" and snd.sent == 1
    snd.close(); srv.close()
    # audit storage
    t = [0.0]
    aud = P.AuditStorage(tmp_path / "audit", segment_bytes=600, clock=lambda: t[0])
    for i in range(12):
        t[0] = float(i)
        aud.append("alice" if i % 2 == 0 else "bob", "publish" if i % 3 == 0 else "download", f"pkg-{i}", outcome="failure" if i == 7 else "success", size=i)
    assert len(aud._segments()) >= 3 and aud.verify() == {"valid": True, "records_checked": 12}
    assert [r["seq"] for r in aud.query(actor="alice")] == [0, 2, 4, 6, 8, 10] and [r["seq"] for r in aud.query(action="publish", since=4.0)] == [6, 9] and [r["resource"] for r in aud.query(outcome="failure")] == ["pkg-7"] and len(aud.query()) == 12
    reopened = P.AuditStorage(tmp_path / "audit", segment_bytes=600, clock=lambda: t[0])
    reopened.append("carol", "delete", "pkg-1")
    assert reopened.verify()["records_checked"] == 13 and [r["seq"] for r in reopened.query(actor="carol")] == [12] and len(reopened.query(actor="bob")) == 6
    assert reopened.export(tmp_path / "a.csv", "csv") == 13 and (tmp_path / "a.csv").read_text().splitlines()[0] == "seq,time,actor,action,resource,outcome" and reopened.export(tmp_path / "a.jsonl") == 13
    t[0] = 100.0
    removed = reopened.apply_retention(max_age=95.0)
    assert removed >= 1 and reopened.verify()["valid"] and reopened.verify()["records_checked"] < 13 and all(r["seq"] >= 3 for r in reopened.query(actor="bob"))
    seg = reopened._file(reopened._segments()[0])
    seg.write_text(seg.read_text().replace('"success"', '"failure"', 1))
    assert not reopened.verify()["valid"] and reopened.verify()["line"] == 0


def test_core_shapes_symbolic_inference_shape_graph_indexing_typed_signatures_allocation_analysis_and_capabilities():
    from torsh_b200.core import shapes_ext as S
    # symbolic arithmetic
    n, d = S.Sym.dim("n"), S.Sym.dim("d")
    assert repr(n * 2) == repr(2 * n) == "(2 * n)" and (n * 2) == (2 * n) and (n + 0) == n and (n * 1) == n and (n * 0) == 0 and (n - n) == 0 and (n // n) == 1 and ((n * d) // d) == n and (S.Sym.lift(6) * 7) == 42
    assert (n * d + 3).evaluate({"n": 4, "d": 5}) == 23 and (n * d + 3).free() == {"n", "d"} and ((n + 7) // 2 % 3).evaluate({"n": 10}) == 2 and hash(n * 2) == hash(2 * n)
    with pytest.raises(KeyError):
        (n + 1).evaluate({})
    # unification
    env = S.ShapeEnv().constrain("n", 1, 1024)
    env.unify(n, 128); env.unify(d, n * 2)
    assert env.resolve(d) == 256 and env.concrete([n, d, 3]) == (128, 256, 3)
    with pytest.raises(ValueError, match="violates its range"):
        S.ShapeEnv().constrain("n", 1, 64).unify(n, 128)
    with pytest.raises(ValueError, match="shape mismatch in test: 3 != 4"):
        S.ShapeEnv().unify(3, 4, "test")
    with pytest.raises(ValueError, match="occurs"):
        S.ShapeEnv().unify(n, n + 1)
    with pytest.raises(KeyError, match="unbound"):
        S.ShapeEnv().concrete([n])
    late = S.ShapeEnv(); late.unify(n * 2, d + 2)
    late.unify(n, 5); late.unify(d, 8)
    assert late.concrete([n, d]) == (5, 8)
    bad = S.ShapeEnv(); bad.unify(n * 2, d + 2); bad.unify(n, 5); bad.unify(d, 9)
    with pytest.raises(ValueError, match="shape mismatch"):
        bad.concrete([n])
    # inference rules against real tensors
    B, T, D, K = S.sym_shape("B", "T", "D", "K")
    e = S.ShapeEnv()
    assert S.infer_shape("matmul", e, (B, T, D), (D, K)) == (B, T, K) and S.infer_shape("linear", e, (B, T, D), (K, D)) == (B, T, K) and S.infer_shape("transpose", e, (B, T, D), dims=(0, 2)) == (D, T, B)
    e2 = S.ShapeEnv()
    out = S.infer_shape("matmul", e2, (B, 4, D), (S.Sym.dim("E"), 7))
    assert e2.resolve(S.Sym.dim("E")) == D or e2.resolve(D) == S.Sym.dim("E")
    assert S.infer_shape("broadcast", S.ShapeEnv(), (B, 1, D), (T, 1)) == (B, T, D) and S.infer_shape("cat", S.ShapeEnv(), (B, T, D), (B, K, D), dim=1) == (B, T + K, D) and S.infer_shape("flatten", S.ShapeEnv(), (B, 3, T, D)) == (B, 3 * T * D)
    assert S.infer_shape("reduce", S.ShapeEnv(), (B, T, D), dim=1) == (B, D) and S.infer_shape("reduce", S.ShapeEnv(), (B, T, D), dim=1, keepdim=True) == (B, 1, D)
    rs = S.infer_shape("reshape", S.ShapeEnv(), (B, T, 8, 64), shape=(B, T, -1))
    assert rs == (B, T, 512)
    conv = S.infer_shape("conv2d", S.ShapeEnv(), (B, 3, S.Sym.dim("H"), S.Sym.dim("W")), (64, 3, 7, 7), kernel=7, stride=2, padding=3)
    ce = S.ShapeEnv()
    assert ce.concrete([v if not isinstance(v, S.Sym) else v for v in [conv[0].evaluate({"B": 2}) if False else 2, conv[1], conv[2].evaluate({"H": 224}), conv[3].evaluate({"W": 200})]]) == tuple(torch.nn.Conv2d(3, 64, 7, 2, 3)(torch.zeros(2, 3, 224, 200)).shape)
    assert S.infer_shape("pool2d", S.ShapeEnv(), (2, 8, 17, 17), kernel=3, stride=2, padding=1) == tuple(torch.nn.MaxPool2d(3, 2, 1)(torch.zeros(2, 8, 17, 17)).shape)
    with pytest.raises(ValueError, match="conv2d channels"):
        S.infer_shape("conv2d", S.ShapeEnv(), (1, 4, 8, 8), (8, 3, 3, 3))
    # shape graph: an attention block
    g = S.ShapeGraph()
    g.input("x", "B", "T", "D"); g.input("wq", "D", "D"); g.input("wo", "D", "V")
    g.op("q", "matmul", "x", "wq"); g.op("qt", "transpose", "q", dims=(1, 2)); g.op("scores", "matmul", "q", "qt"); g.op("ctx", "matmul", "scores", "q"); g.op("logits", "matmul", "ctx", "wo"); g.op("flat", "reshape", "logits", shape=(-1, S.Sym.dim("V")))
    sym = g.infer()
    assert [repr(v) for v in sym["scores"]] == ["B", "T", "T"] and [repr(v) for v in sym["flat"]] == ["(B * T)", "V"]
    conc = g.specialize(B=2, T=5, D=16, V=100)
    x, wq, wo = torch.zeros(2, 5, 16), torch.zeros(16, 16), torch.zeros(16, 100)
    q = x @ wq
    assert conc["scores"] == tuple((q @ q.transpose(1, 2)).shape) and conc["flat"] == (10, 100) and conc["logits"] == (2, 5, 100) and g.specialize(B=1, T=3, D=8, V=7)["flat"] == (3, 7)
    g.infer()
    assert g.cache_hits == 6 * 3 and g.explain("scores")[0] == "scores: [B, T, T] = matmul(q, qt)" and any(l.endswith("(input)") for l in g.explain("scores"))
    # strides and indices
    assert S.contiguous_strides((2, 3, 4)) == (12, 4, 1) == torch.empty(2, 3, 4).stride() and S.is_contiguous((2, 3, 4), (12, 4, 1)) and not S.is_contiguous((2, 3, 4), (1, 2, 6)) and S.is_contiguous((1, 3), (99, 1))
    assert S.ravel_index((1, 2, 3), (2, 3, 4)) == 23 and S.unravel_index(23, (2, 3, 4)) == (1, 2, 3) and S.normalize_dim(-1, 3) == 2
    with pytest.raises(IndexError):
        S.normalize_dim(3, 3)
    t = torch.arange(3.0).reshape(3, 1)
    assert S.broadcast_strides((3, 1), t.stride(), (2, 3, 4)) == t.expand(2, 3, 4).stride()
    with pytest.raises(ValueError):
        S.broadcast_strides((3, 2), (2, 1), (3, 4))
    assert S.can_view((4, 6), (6, 1), (24,)) and not S.can_view((4, 6), (1, 4), (24,)) and S.can_view((4, 6), (1, 4), (4, 2, 3))
    # shape-annotated signatures
    @S.typed_shapes("x: B T D, w: D K -> B T K")
    def project(x, w): return x @ w
    assert project(torch.zeros(2, 3, 4), torch.zeros(4, 5)).shape == (2, 3, 5) and project.shape_spec.startswith("x: B T D")
    with pytest.raises(TypeError, match="w: dimension D = 6 but it was 4"):
        project(torch.zeros(2, 3, 4), torch.zeros(6, 5))
    with pytest.raises(TypeError, match="x: expected 3 dimensions"):
        project(torch.zeros(3, 4), torch.zeros(4, 5))
    @S.typed_shapes("x: ... 3, y: ... 3 -> ...")
    def dot3(x, y): return (x * y).sum(-1)
    assert dot3(torch.zeros(5, 2, 3), torch.zeros(5, 2, 3)).shape == (5, 2)
    with pytest.raises(TypeError, match="dimension 3 expected"):
        dot3(torch.zeros(5, 4), torch.zeros(5, 4))
    with pytest.raises(TypeError, match="leading dimensions"):
        dot3(torch.zeros(5, 3), torch.zeros(6, 3))
    @S.typed_shapes("x: N -> N N")
    def wrong(x): return x
    with pytest.raises(TypeError, match="result: expected 2 dimensions"):
        wrong(torch.zeros(4))
    # allocation traces
    ev, t_ = [], 0.0
    for i in range(100):
        ev.append(S.AllocEvent(t_, 256, "alloc", i)); ev.append(S.AllocEvent(t_ + 0.001, 256, "free", i)); t_ += 0.01
    for i in range(100, 110):
        ev.append(S.AllocEvent(t_, 1 << 20, "alloc", i)); t_ += 0.01
    for i in range(100, 108):
        ev.append(S.AllocEvent(t_ + 5, 1 << 20, "free", i))
    rep = S.analyze_allocations(sorted(ev, key=lambda e: e.time))
    kinds = [r["kind"] for r in rep["recommendations"]]
    assert rep["peak_bytes"] == 10 << 20 and rep["leaked"] == 2 and rep["allocations"] == 110 and kinds[0] == "arena" and "free_list" in kinds and kinds[-1] == "leak_check" and rep["repeated_sizes"] == {256: 100, 1 << 20: 10}
    assert rep["size_classes"][256]["count"] == 100 and rep["size_classes"][1 << 20]["median_lifetime"] > 4 and rep["small_short_fraction"] > 0.8
    # capabilities
    caps = S.detect_capabilities("processor : 0\nmodel name : Test CPU 9000\nflags : fpu sse4_2 avx avx2 fma avx512f avx512_bf16\n")
    assert caps["cpu_model"] == "Test CPU 9000" and caps["simd"] == ["sse4_2", "avx", "avx2", "fma", "avx512f", "avx512_bf16"] and caps["best_simd_bits"] == 512 and caps["preferred_device"] in ("cpu", "cuda")
    assert S.detect_capabilities("Features : fp asimd sve\n")["simd"] == ["neon", "sve"] and isinstance(S.detect_capabilities()["logical_cores"], int)
    b200, h100, a100 = S.features_for_capability(10, 0), S.features_for_capability(9, 0), S.features_for_capability(8, 0)
    assert b200["tcgen05_tensor_memory"] and not b200["wgmma"] and b200["arch_flag"] == "sm_100a" and h100["wgmma"] and h100["tma"] and not h100["tcgen05_tensor_memory"] and a100["bf16_tensor_cores"] and not a100["tma"] and a100["arch_flag"] == "sm_80" and a100["max_shared_memory_kb"] == 163


def test_autograd_graph_opt_backward_graph_memory_planning_onnx_gradients_api_levels_and_device_choice():
    from torsh_b200.autograd import graph_opt as G
    torch.manual_seed(0)
    # backward graph
    a, b = torch.randn(4, 3, requires_grad=True), torch.randn(3, 5, requires_grad=True)
    frozen = torch.randn(4, 5)
    fn = lambda p, q: (torch.tanh(torch.relu(p @ q) * 2.0 + 1.0) + frozen).sum()
    g = G.BackwardGraph.from_function(fn, a, b)
    s = g.summary()
    assert s["leaves"] == 2 and s["operations"]["MmBackward0"] == 1 and s["operations"]["TanhBackward0"] == 1 and s["depth"] >= 6 and s["saved_bytes"] >= (12 + 15 + 20) * 4 and g.saved_tensor_count >= 4
    order = g.execution_order()
    pos = {v: i for i, v in enumerate(order)}
    assert len(order) == g.node_count() and order[0] == g.root and all(pos[n.id] < pos[i] for n in g.nodes.values() for i in n.inputs)
    chains = g.fusable_chains()
    assert chains == [["AddBackward0", "TanhBackward0", "AddBackward0", "MulBackward0", "ReluBackward0"]]
    assert g.dead_branches() == [] and g.edge_count() >= g.node_count() - 1
    x = torch.randn(3, requires_grad=True)
    dead = G.BackwardGraph((x * 2).sum() + (x.detach() * 3).sum())
    assert dead.dead_branches() == []
    dups = G.duplicate_subexpressions(lambda t: torch.exp(t) * torch.exp(t) + torch.sin(t))
    assert dups == [["exp", "exp_1"]] and G.duplicate_subexpressions(lambda t: torch.exp(t) + torch.sin(t)) == []
    # memory planning
    model = torch.nn.Sequential(*[m for _ in range(8) for m in (torch.nn.Linear(64, 64), torch.nn.Tanh())])
    xin = torch.randn(32, 64, requires_grad=True)
    costs = G.profile_layers(model, xin)
    assert len(costs) == 16 and all(c.activation_bytes >= 32 * 64 * 4 for c in costs) and costs[0].output_bytes == 32 * 64 * 4
    base = G.memory_timeline(costs)
    assert base["peak_bytes"] == sum(c.activation_bytes for c in costs) and base["timeline"][15][1] == base["peak_bytes"] and base["timeline"][-1][1] == costs[0].activation_bytes and base["recompute_flops"] == 0
    plan = G.plan_checkpoints(costs)
    assert plan["checkpoints"] == [4, 8, 12] and plan["peak_bytes"] < 0.5 * plan["baseline_peak"] and plan["recompute_flops"] == pytest.approx(sum(c.flops for c in costs))
    tight = G.plan_checkpoints(costs, budget_bytes=0.4 * base["peak_bytes"])
    assert tight["fits"] and tight["peak_bytes"] <= 0.4 * base["peak_bytes"] and len(tight["checkpoints"]) >= 3
    assert G.plan_checkpoints(costs, budget_bytes=2 * base["peak_bytes"])["checkpoints"] == [] and not G.plan_checkpoints(costs, budget_bytes=1.0)["fits"]
    uneven = [G.LayerCost("a", 100, 10), G.LayerCost("b", 10, 10), G.LayerCost("c", 10, 10), G.LayerCost("d", 100, 10)]
    assert G.plan_checkpoints(uneven, segments=2)["checkpoints"] == [2] and G.plan_checkpoints(uneven, segments=3)["checkpoints"] in ([1, 3], [1, 2], [2, 3])
    ck = G.apply_checkpoints(model, plan["checkpoints"])
    x1, x2 = xin.detach().clone().requires_grad_(True), xin.detach().clone().requires_grad_(True)
    saved_plain, saved_ck = [], []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved_plain.append(t.numel()) or t, lambda t: t):
        y1 = model(x1)
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved_ck.append(t.numel()) or t, lambda t: t):
        y2 = ck(x2)
    y1.sum().backward(); y2.sum().backward()
    assert torch.allclose(y1, y2) and torch.allclose(x1.grad, x2.grad, atol=1e-6) and sum(saved_ck) < 0.5 * sum(saved_plain) and len(ck.segments) == 4
    # ONNX round trip keeps gradients
    net = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.ReLU(), torch.nn.Linear(8, 3), torch.nn.Tanh())
    rt = G.verify_roundtrip_gradients(net, torch.randn(5, 6))
    assert rt["ok"] and rt["gradient_max_diff"] < 1e-5 and rt["bytes"] > 300
    # API stability levels
    api = G.ApiCompatibilityChecker("0.1.3").with_defaults()
    assert api.is_stable("backward") and api.is_experimental("forward_ad") and api.is_deprecated("Variable")
    ok = api.check(["backward", "grad", "functional.hessian"])
    assert ok["compatible"] and not api.check(["forward_ad"])["compatible"] and api.check(["forward_ad"], allow=("stable", "beta", "experimental"))["compatible"]
    old = api.check(["graph_opt"], written_for="0.1.1")
    assert not old["compatible"] and "introduced in 0.1.2" in old["problems"][0]["problem"] and api.check(["nonsense"])["problems"][0]["problem"] == "unknown"
    dep = api.check(["Variable"])
    assert dep["problems"][0]["replacement"] == "Tensor.requires_grad_" and "deprecated" in dep["problems"][0]["problem"]
    later = G.ApiCompatibilityChecker("0.2.0").with_defaults()
    assert "removed in 0.2.0" in later.check(["Variable"])["problems"][0]["problem"]
    with pytest.raises(ValueError):
        api.register("x", "alpha", "0.1.0")
    # device choice
    devs = [{"name": "cpu", "tflops": 0.5, "resident": True}, {"name": "cuda", "tflops": 60.0, "resident": False}]
    small, big = G.select_device_for_workload(1000, devices=devs), G.select_device_for_workload(50_000_000, flops_per_element=200, devices=devs)
    assert small["device"] == "cpu" and big["device"] == "cuda" and big["speedup_over_cpu"] > 2 and G.select_device_for_workload(10)["device"] in ("cpu", "cuda")


def test_function_transformations_grad_vjp_jvp_jacobians_hessian_vmap_remat_and_control_flow():
    from torsh_b200.autograd import transforms as J
    torch.manual_seed(0)
    f = lambda x: (x ** 3).sum() + torch.sin(x).sum()
    x = torch.randn(5, dtype=torch.float64)
    assert torch.allclose(J.grad(f)(x), 3 * x ** 2 + torch.cos(x)) and torch.allclose(J.grad(lambda v: J.grad(f)(v).sum())(x), 6 * x - torch.sin(x))
    ga, gb = J.grad(lambda a, b: (a * b).sum(), argnums=(0, 1))(x, 2 * x)
    assert torch.allclose(ga, 2 * x) and torch.allclose(gb, x)
    A = torch.randn(3, 5, dtype=torch.float64)
    g = lambda v: torch.tanh(A @ v)
    jac = torch.autograd.functional.jacobian(g, x)
    out, pull = J.vjp(g, x)
    ct = torch.randn(3, dtype=torch.float64)
    assert torch.allclose(out, g(x)) and torch.allclose(pull(ct)[0], ct @ jac)
    tang = torch.randn(5, dtype=torch.float64)
    o, jv = J.jvp(g, (x,), (tang,))
    assert torch.allclose(o, g(x)) and torch.allclose(jv, jac @ tang)
    assert torch.allclose(J.jacrev(g)(x), jac) and torch.allclose(J.jacfwd(g)(x), jac)
    two = lambda a, b: a * b.sum()
    assert torch.allclose(J.jacrev(two, 1)(x, x), torch.autograd.functional.jacobian(lambda b: two(x, b), x)) and torch.allclose(J.jacfwd(two, 0)(x, x), torch.diag(torch.full((5,), float(x.sum()), dtype=torch.float64)))
    M = torch.randn(2, 3, dtype=torch.float64)
    assert J.jacrev(lambda m: m @ m.T)(M).shape == (2, 2, 2, 3) and torch.allclose(J.jacrev(lambda m: m @ m.T)(M), J.jacfwd(lambda m: m @ m.T)(M))
    assert torch.allclose(J.hessian(f)(x), torch.diag(6 * x - torch.sin(x))) and torch.allclose(J.hessian(lambda v: (v @ A.T @ A @ v))(x), 2 * A.T @ A)
    # vmap: batched Jacobians, broadcast arguments, fallback for data-dependent code
    xs = torch.randn(7, 5, dtype=torch.float64)
    per = J.vmap(J.grad(f))(xs)
    assert torch.allclose(per, 3 * xs ** 2 + torch.cos(xs))
    assert torch.allclose(J.vmap(lambda v, m: m @ v, in_dims=(0, None))(xs, A), xs @ A.T) and J.vmap(lambda v: v.sum(), out_dims=0)(xs).shape == (7,)
    assert torch.allclose(J.vmap(lambda a, b: a @ b, in_dims=(1, 0))(xs.T.contiguous(), xs), (xs * xs).sum(1))
    def branchy(v): return v * 2 if float(v.sum()) > 0 else v * -1                    # cannot be batched by the interpreter
    looped = J.vmap(branchy)(xs)
    assert torch.allclose(looped, torch.where(xs.sum(1, keepdim=True) > 0, xs * 2, -xs))
    a1, a2 = J.vmap(lambda v: (v.sum(), v * 2))(xs)
    assert a1.shape == (7,) and a2.shape == (7, 5)
    # remat keeps values and gradients, saves fewer tensors
    net = torch.nn.Sequential(torch.nn.Linear(5, 64), torch.nn.Tanh(), torch.nn.Linear(64, 64), torch.nn.Tanh(), torch.nn.Linear(64, 1)).double()
    xa, xb = xs.clone().requires_grad_(True), xs.clone().requires_grad_(True)
    c1, c2 = [], []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: c1.append(1) or t, lambda t: t):
        y1 = net(xa).sum()
    with torch.autograd.graph.saved_tensors_hooks(lambda t: c2.append(1) or t, lambda t: t):
        y2 = J.remat(net)(xb).sum()
    y1.backward(); y2.backward()
    assert torch.allclose(y1, y2) and torch.allclose(xa.grad, xb.grad) and len(c2) < len(c1)
    # control flow
    carry, ys = J.scan(lambda c, v: (c + v, c * v), torch.tensor(0.0), torch.arange(1.0, 5.0))
    assert float(carry) == 10.0 and ys.tolist() == [0.0, 2.0, 9.0, 24.0]
    rc, rys = J.scan(lambda c, v: (c + v, c), torch.tensor(0.0), torch.arange(1.0, 4.0), reverse=True)
    assert float(rc) == 6.0 and rys.tolist() == [5.0, 3.0, 0.0]
    assert J.fori_loop(0, 5, lambda i, v: v + i, 0) == 10 and J.while_loop(lambda v: v < 100, lambda v: v * 2, 1) == 128
    with pytest.raises(RuntimeError):
        J.while_loop(lambda v: True, lambda v: v, 0, max_iterations=10)
    assert float(J.cond(True, lambda v: v * 2, lambda v: v * 3, torch.tensor(1.0))) == 2.0 and float(J.cond(torch.tensor(False), lambda v: v * 2, lambda v: v * 3, torch.tensor(1.0))) == 3.0
    pv = torch.tensor([True, False, True])
    xv = torch.ones(3, 2, requires_grad=True)
    sel = J.cond(pv, lambda v: v * 2, lambda v: v * 3, xv)
    sel.sum().backward()
    assert sel[:, 0].tolist() == [2.0, 3.0, 2.0] and xv.grad[:, 0].tolist() == [2.0, 3.0, 2.0]
    # a decaying scan is differentiable end to end
    w = torch.tensor(0.5, requires_grad=True)
    final, _ = J.scan(lambda c, v: (c * w + v, c), torch.tensor(0.0), torch.ones(4))
    final.backward()
    assert float(final.detach()) == pytest.approx(1 + 0.5 + 0.25 + 0.125) and float(w.grad) == pytest.approx(1 + 2 * 0.5 + 3 * 0.25)


def test_rstorch_surface_matches_the_reference_python_package_names():
    """Every public name of the reference's ``python/rstorch`` modules (``__all__`` and the names imported from its native
    extension, transcribed below) resolves in this package."""
    import rstorch
    names = {"__init__": ["BoolTensor", "ByteTensor", "FloatTensor", "IntTensor", "LongTensor", "Tensor", "TorshError", "add", "arange", "bmm", "bool_dtype", "cpu", "cuda_is_available", "device", "device_count", "div", "dtype", "empty", "empty_like",
                          "flatten", "float32", "float64", "full", "full_like", "get_default_device", "get_default_dtype", "get_device_name", "int16", "int32", "int64", "int8", "is_available", "linspace", "matmul", "mm", "mps_is_available", "mul",
                          "ones", "ones_like", "permute", "rand", "rand_like", "randn", "randn_like", "reshape", "set_default_device", "set_default_dtype", "squeeze", "sub", "tensor", "transpose", "uint16", "uint32", "uint64", "uint8", "unsqueeze",
                          "view", "zeros", "zeros_like"],
             "nn": ["Linear", "Module", "ModuleList", "Parameter", "Sequential", "cross_entropy", "log_softmax", "mse_loss", "parameter", "relu", "sigmoid", "softmax", "tanh"], "optim": ["Adam", "AdamW", "Optimizer", "SGD"],
             "autograd": ["Function", "backward", "detect_anomaly", "enable_grad", "grad", "is_grad_enabled", "no_grad", "set_grad_enabled"],
             "distributed": ["DDP", "DistributedDataParallel", "ProcessGroup", "all_gather", "all_reduce", "barrier", "broadcast", "destroy_process_group", "gather", "get_rank", "get_world_size", "init_process_group", "is_available", "is_initialized",
                             "reduce", "scatter"]}
    for mod, wanted in names.items():
        ours = rstorch if mod == "__init__" else getattr(rstorch, mod)
        missing = sorted(n for n in wanted if not hasattr(ours, n))
        assert not missing, (mod, missing)
    x = rstorch.tensor([[1.0, -2.0], [0.5, 3.0]])
    assert rstorch.nn.relu(x).tolist() == [[1.0, 0.0], [0.5, 3.0]] and float(rstorch.nn.mse_loss(x, x)) == 0.0 and type(rstorch.nn.parameter(x)).__name__ == "Parameter" and rstorch.FloatTensor is rstorch.Tensor and rstorch.uint16.size_bytes == 2


def test_metric_objects_accumulate_like_sklearn_and_merge_across_shards():
    import numpy as np
    from sklearn import metrics as skm
    from torsh_b200.utils import metric_objects as mo

    g = torch.Generator().manual_seed(0)
    n, C = 1200, 4
    logits = torch.randn(n, C, generator=g)
    y = torch.randint(0, C, (n,), generator=g)
    logits[torch.arange(n), y] += 1.0
    pred = logits.argmax(1)
    coll = mo.MetricCollection({"acc": mo.Accuracy(), "top2": mo.TopKAccuracy(2), "prec": mo.Precision(C, "macro"), "rec": mo.Recall(C, "weighted"),
                                "f1": mo.F1Score(C, "macro"), "multi": mo.MultiClassMetrics(C)})
    for lo in range(0, n, 100):
        coll.update(logits[lo:lo + 100], y[lo:lo + 100])
    out = coll.compute()
    assert out["acc"] == pytest.approx(skm.accuracy_score(y, pred))
    assert out["top2"] == pytest.approx(skm.top_k_accuracy_score(y, logits, k=2))
    assert out["prec"] == pytest.approx(skm.precision_score(y, pred, average="macro"))
    assert out["rec"] == pytest.approx(skm.recall_score(y, pred, average="weighted"))
    assert out["f1"] == pytest.approx(skm.f1_score(y, pred, average="macro"))
    assert out["multi/cohen_kappa"] == pytest.approx(skm.cohen_kappa_score(y, pred))
    assert out["multi/mcc"] == pytest.approx(skm.matthews_corrcoef(y, pred))
    assert out["multi/balanced_accuracy"] == pytest.approx(skm.balanced_accuracy_score(y, pred))
    cm = mo.ConfusionMatrix(C)
    cm.update(logits, y)
    assert np.array_equal(cm.compute().numpy(), skm.confusion_matrix(y, pred))
    assert torch.allclose(cm.normalized("true").sum(1), torch.ones(C, dtype=torch.float64))
    a, b = mo.Accuracy(), mo.Accuracy()                                           # two shards merge to the global value
    a.update(logits[:500], y[:500]); b.update(logits[500:], y[500:])
    assert a.merge(b).compute() == pytest.approx(out["acc"])
    batch_value = a(logits[:10], y[:10])                                          # call = batch value, state keeps accumulating
    assert batch_value == pytest.approx(float((pred[:10] == y[:10]).float().mean())) and float(a._state["total"]) == n + 10
    assert a.sync().compute() == a.compute() and a.reset().compute() == 0.0

    # ---- binary scores: histogram curves against the exact ones
    s = torch.sigmoid(torch.randn(4000, generator=g) + 1.5 * (torch.arange(4000) % 2))
    t = (torch.arange(4000) % 2)
    tm = mo.ThresholdMetrics(2000)
    tm.update(s[:2000], t[:2000]); tm.update(s[2000:], t[2000:])
    assert tm.auroc() == pytest.approx(skm.roc_auc_score(t, s), abs=2e-4)
    assert tm.average_precision() == pytest.approx(skm.average_precision_score(t, s), abs=2e-3)
    thr, f1 = tm.best_threshold("f1")
    assert f1 == pytest.approx(max(skm.f1_score(t, s >= c) for c in np.linspace(0.05, 0.95, 91)), abs=5e-3) and 0.2 < thr < 0.8
    sa = mo.StreamingAUROC(2000); sa.update(s, t)
    assert sa.compute() == pytest.approx(tm.auroc())
    svg = mo.ROCCurvePlot().render({"model": tm})
    assert svg.startswith("<svg") and "AUC 0." in svg and "polyline" in svg and "AP 0." in mo.PRCurvePlot().render({"m": tm})

    # ---- regression
    p = torch.randn(900, generator=g, dtype=torch.float64)
    tt = 0.7 * p + 0.3 * torch.randn(900, generator=g, dtype=torch.float64) + 2
    reg = mo.MetricCollection([mo.MSE(), mo.RMSE(), mo.MAE(), mo.MAPE(), mo.SMAPE(), mo.R2Score(), mo.ExplainedVariance(), mo.HuberLoss(0.5), mo.LogCoshLoss(), mo.QuantileLoss(0.9)])
    for lo in range(0, 900, 300):
        reg.update(p[lo:lo + 300], tt[lo:lo + 300])
    r = reg.compute()
    assert r["MSE"] == pytest.approx(skm.mean_squared_error(tt, p)) and r["RMSE"] == pytest.approx(math.sqrt(r["MSE"]))
    assert r["MAE"] == pytest.approx(skm.mean_absolute_error(tt, p)) and r["MAPE"] == pytest.approx(100 * skm.mean_absolute_percentage_error(tt, p))
    assert r["R2Score"] == pytest.approx(skm.r2_score(tt, p)) and r["ExplainedVariance"] == pytest.approx(skm.explained_variance_score(tt, p))
    assert r["QuantileLoss"] == pytest.approx(skm.mean_pinball_loss(tt, p, alpha=0.9))
    assert r["HuberLoss"] == pytest.approx(float(torch.nn.functional.huber_loss(p, tt, delta=0.5)))
    assert r["LogCoshLoss"] == pytest.approx(float(torch.log(torch.cosh(p - tt)).mean()))
    r2 = mo.R2Score(); r2.update(p, tt)
    assert r2.adjusted(3) < r2.compute()

    # ---- ranking
    scores = torch.rand(50, 20, generator=g)
    rel = torch.randint(0, 4, (50, 20), generator=g).float() * (torch.rand(50, 20, generator=g) > 0.5)
    nd = mo.NDCG(10, exponential=False); nd.update(scores[:25], rel[:25]); nd.update(scores[25:], rel[25:])
    assert nd.compute() == pytest.approx(skm.ndcg_score(rel.numpy(), scores.numpy(), k=10), abs=1e-9)
    binrel = (rel > 0).float()
    mp = mo.MeanAveragePrecision(); mp.update(scores, binrel)
    assert mp.compute() == pytest.approx(np.mean([skm.average_precision_score(binrel[i], scores[i]) for i in range(50)]), abs=1e-9)
    ra = mo.RankingAUC(); ra.update(scores, binrel)
    assert ra.compute() == pytest.approx(np.mean([skm.roc_auc_score(binrel[i], scores[i]) for i in range(50)]), abs=1e-9)
    one = torch.tensor([[0.9, 0.8, 0.7, 0.1]]); relone = torch.tensor([[0.0, 0, 1, 1]])
    for cls, want in ((mo.MeanReciprocalRank, 1 / 3), (mo.PrecisionAtK, 1 / 3), (mo.RecallAtK, 0.5), (mo.HitRateAtK, 1.0), (mo.F1AtK, 0.4)):
        m = cls(3); m.update(one, relone)
        assert m.compute() == pytest.approx(want), cls.__name__
    cov = mo.Coverage(10); cov.update(torch.tensor([[0, 1, 2], [0, 1, 3]]))
    assert cov.compute() == pytest.approx(0.4) and 0 < cov.gini() < 1
    feats = torch.eye(4)
    dv = mo.Diversity(feats); dv.update(torch.tensor([[0, 1, 2]])); dv.update(torch.tensor([[0, 0, 0]]))
    assert dv.compute() == pytest.approx(0.5)
    nv = mo.Novelty(torch.tensor([8.0, 4, 2, 2])); nv.update(torch.tensor([[0, 3]]))
    assert nv.compute() == pytest.approx((1 + 3) / 2)

    # ---- clustering objects wrap the functions
    pts = torch.cat([torch.randn(60, 2, generator=g) * 0.3, torch.randn(60, 2, generator=g) * 0.3 + 4])
    lab = torch.cat([torch.zeros(60), torch.ones(60)]).long()
    sil = mo.SilhouetteScore(); sil.update(pts[:60], lab[:60]); sil.update(pts[60:], lab[60:])
    assert sil.compute() == pytest.approx(skm.silhouette_score(pts.numpy(), lab.numpy()), abs=1e-5)
    ari = mo.AdjustedRandIndex(); ari.update(lab, 1 - lab)
    vm = mo.VMeasure(); vm.update(lab, 1 - lab)
    assert ari.compute() == pytest.approx(1.0) and vm.compute() == pytest.approx(1.0)
    db = mo.DaviesBouldin(); db.update(pts, lab)
    assert db.compute() == pytest.approx(skm.davies_bouldin_score(pts.numpy(), lab.numpy()), rel=1e-4) and not db.higher_is_better

    # ---- language model and calibration
    lm_logits = torch.randn(6, 9, 30, generator=g)
    lm_t = torch.randint(0, 30, (6, 9), generator=g)
    lm_t[0, :3] = -100
    ppl = mo.Perplexity(); ppl.update(lm_logits[:3], lm_t[:3]); ppl.update(lm_logits[3:], lm_t[3:])
    assert ppl.compute() == pytest.approx(float(torch.exp(torch.nn.functional.cross_entropy(lm_logits.reshape(-1, 30), lm_t.reshape(-1), ignore_index=-100))), rel=1e-5)
    probs = torch.softmax(2.5 * logits, 1)                                          # over-confident
    ece = mo.ExpectedCalibrationError(10); ece.update(probs[:600], y[:600]); ece.update(probs[600:], y[600:])
    from torsh_b200.utils.metrics_ext import calibration_error
    conf, hit = probs.max(1).values, (probs.argmax(1) == y)
    assert ece.compute() == pytest.approx(calibration_error(conf, hit, 10), abs=1e-9)
    mce = mo.MaximumCalibrationError(10); mce.update(probs, y)
    assert mce.compute() >= ece.compute() > 0.02
    rd = mo.ReliabilityDiagram(10); rd.update(probs, y)
    assert "ECE 0." in mo.CalibrationCurvePlot().render({"net": rd})
    bs = mo.BrierScore(); bs.update(probs, y)
    assert bs.compute() == pytest.approx(float(((probs - torch.nn.functional.one_hot(y, C)) ** 2).sum(1).mean()), rel=1e-6)
    bsb = mo.BrierScore(); bsb.update(s, t)
    assert bsb.compute() == pytest.approx(skm.brier_score_loss(t, s))
    pic = mo.PredictionIntervalCoverage(); pic.update(p - 1, p + 1, p + 0.5 * torch.randn(900, generator=g, dtype=torch.float64))
    assert pic.compute()["coverage"] == pytest.approx(0.954, abs=0.03) and pic.compute()["mean_width"] == pytest.approx(2.0)
    members = torch.softmax(torch.randn(5, 40, 3, generator=g) * 2, -1)
    eu = mo.EnsembleUncertainty.decompose(members)
    assert bool((eu["epistemic"] >= -1e-6).all()) and torch.allclose(eu["total"], eu["aleatoric"] + eu["epistemic"])
    agree = members[:1].expand(5, -1, -1)
    assert float(mo.EnsembleUncertainty.decompose(agree)["epistemic"].abs().max()) < 1e-6
    assert float(mo.EntropyMeasures.normalized_entropy(torch.full((1, 4), 0.25))) == pytest.approx(1.0)

    # ---- fairness
    grp = torch.randint(0, 2, (3000,), generator=g)
    truth = (torch.rand(3000, generator=g) < 0.5).long()
    biased = torch.where(grp == 1, truth | (torch.rand(3000, generator=g) < 0.4).long(), truth & (torch.rand(3000, generator=g) < 0.7).long())
    fm = mo.FairnessMetrics(2); fm.update(biased[:1500], truth[:1500], grp[:1500]); fm.update(biased[1500:], truth[1500:], grp[1500:])
    fr = fm.compute()
    rate = lambda m: float(biased[m].double().mean())
    assert fr["demographic_parity"]["difference"] == pytest.approx(abs(rate(grp == 1) - rate(grp == 0)), abs=1e-9)
    assert fr["equalized_odds"]["tpr_gap"] == pytest.approx(abs(rate((grp == 1) & (truth == 1)) - rate((grp == 0) & (truth == 1))), abs=1e-9)
    assert fr["equalized_odds"]["fpr_gap"] == pytest.approx(0.4, abs=0.05) and fr["demographic_parity"]["ratio"] < 0.8
    fair = mo.DemographicParity(2); fair.update(truth, truth, grp)
    assert fair.compute()["difference"] < 0.06
    gc = mo.GroupCalibration(2, 5); gc.update(s[:3000], t[:3000], grp)
    assert len(gc.compute()["ece_per_group"]) == 2
    x_f = torch.randn(200, 3, generator=g)
    smooth = mo.IndividualFairness(1.0).evaluate(x_f, 0.5 * x_f[:, :1])
    rough = mo.IndividualFairness(1.0).evaluate(x_f, 5.0 * x_f[:, :1])
    assert smooth["violation_rate"] == 0.0 and smooth["max_ratio"] <= 0.5 + 1e-9 and rough["violation_rate"] > 0.5
    lab3 = torch.randint(0, 3, (3000,), generator=g)
    g3 = ((torch.rand(3000, generator=g) < 0.5 + 0.1 * (lab3 == 0)) * 1).long()
    amplified = torch.where((g3 == 1) & (torch.rand(3000, generator=g) < 0.3), torch.zeros_like(lab3), lab3)
    assert mo.BiasAmplification.compute(amplified, lab3, g3, 3) > 0.01 and abs(mo.BiasAmplification.compute(lab3, lab3, g3, 3)) < 1e-12

    # ---- streaming statistics and chunked evaluation
    data = torch.randn(1000, generator=g, dtype=torch.float64) * 3 + 1
    s1, s2 = mo.StreamingStats(), mo.StreamingStats()
    for lo in range(0, 600, 50):
        s1.update(data[lo:lo + 50])
    s2.update(data[600:])
    st = s1.merge(s2).compute()
    assert st["count"] == 1000 and st["mean"] == pytest.approx(float(data.mean())) and st["variance"] == pytest.approx(float(data.var()))
    assert st["min"] == float(data.min()) and st["max"] == float(data.max())
    lin = torch.nn.Linear(8, C)
    xin = torch.randn(1000, 8, generator=g)
    ylab = lin(xin).argmax(1)
    ev = mo.ChunkedEvaluator({"acc": mo.Accuracy(), "cm": mo.ConfusionMatrix(C)}, chunk_size=128).evaluate(lin, xin, ylab)
    assert ev["acc"] == 1.0 and float(ev["cm"].sum()) == 1000

    # ---- hypothesis tests, resampling, cross-validation, stability
    base = torch.rand(60, generator=g, dtype=torch.float64)
    better = base + 0.05 + 0.01 * torch.randn(60, generator=g, dtype=torch.float64)
    for cls in (mo.PairedTTest, mo.WilcoxonTest):
        res = cls(0.05).test(better, base)
        assert res.significant and res.p_value < 1e-6 and res.name == cls.__name__
    assert not mo.PairedTTest().test(base, base + 0.001 * torch.randn(60, generator=g, dtype=torch.float64)).significant
    ca, cb = torch.rand(500, generator=g) < 0.9, torch.rand(500, generator=g) < 0.6
    assert mo.McNemarTest().test(ca, cb).significant and mo.McNemarTest().test(ca, ca).p_value == 1.0
    assert mo.MannWhitneyTest().test(better, base - 0.3).significant
    assert mo.KruskalWallisTest().test(base, base + 1, base + 2).significant
    table = torch.stack([base, base + 0.2, base + 0.4], 1)
    assert mo.FriedmanTest().test(table).p_value < 1e-6 and mo.NemenyiTest().test(table)["significant"][0, 2]
    assert mo.PermutationTest().test(better, base - 0.3, 500).significant
    assert mo.FiveByTwoCVTest().test(torch.tensor([[0.1, 0.12], [0.09, 0.11], [0.1, 0.1], [0.12, 0.1], [0.11, 0.09]])).p_value < 0.05
    ci = mo.BootstrapCI(300).interval(lambda a, b: float((a == b).float().mean()), pred, y)
    assert ci["lower"] < ci["estimate"] < ci["upper"] and ci["upper"] - ci["lower"] < 0.08
    assert mo.EffectSize.compute(better, base) > 0.1
    mc = mo.MultipleComparisonCorrection("holm").correct([0.001, 0.04, 0.03])
    assert list(mc["reject"]) == [True, False, False]
    cv = mo.CrossValidator(5).run(100, lambda tr, te: len(te) / 100)
    assert cv["scores"] == [0.2] * 5 and cv["std"] == 0.0
    strat = mo.CrossValidator(4, stratified=True).run(torch.arange(80) % 4, lambda tr, te: float(len(te)))
    assert strat["mean"] == 20.0
    stab = mo.StabilityAnalyzer(0.02)
    assert stab.analyze([0.91, 0.915, 0.905, 0.91])["stable"] and not stab.analyze([0.9, 0.8, 0.95])["stable"]

    # ---- model selection
    assert mo.AIC.compute(-100.0, 3) == 206.0 and mo.BIC.compute(-100.0, 3, 50) == pytest.approx(3 * math.log(50) + 200)
    assert mo.AICc.compute(-100.0, 3, 50) == pytest.approx(206 + 24 / 46) and mo.HQIC.compute(-100.0, 3, 50) == pytest.approx(6 * math.log(math.log(50)) + 200)
    mmc = mo.MultiModelComparison("bic").add("small", -120.0, 2, 200).add("right", -100.0, 4, 200).add("big", -99.5, 12, 200).report()
    assert mmc["ranking"][0] == "right" and sum(mmc["weights"].values()) == pytest.approx(1.0) and mmc["evidence_ratio"]["big"] > 100

    # ---- few-shot, meta-learning, domain shift, continual learning
    fs = mo.FewShotMetrics()
    for e in range(40):
        yy = torch.randint(0, 5, (25,), generator=g)
        fs.update(torch.where(torch.rand(25, generator=g) < 0.8, yy, (yy + 1) % 5), yy)
    f = fs.compute()
    assert f["episodes"] == 40 and f["mean_accuracy"] == pytest.approx(0.8, abs=0.05) and 0 < f["ci95"] < 0.05
    ml = mo.MetaLearningMetrics()
    for k in range(6):
        ml.update([2.0, 1.0, 0.6, 0.5, 0.48 + 0.01 * k])
    mlr = ml.compute(0.9)
    assert mlr["adaptation_gain"] == pytest.approx(1.495, abs=0.01) and mlr["steps_to_fraction"] == 2 and mlr["tasks_improved"] == 1.0
    src = torch.randn(300, 5, generator=g)
    same, shifted = torch.randn(300, 5, generator=g), torch.randn(300, 5, generator=g) + 1.5
    da_same = mo.DomainAdaptationMetrics.compute(src, same, 0.9, 0.88)
    da_shift = mo.DomainAdaptationMetrics.compute(src, shifted, 0.9, 0.6)
    assert da_shift["mmd_rbf"] > 10 * abs(da_same["mmd_rbf"]) and da_shift["proxy_a_distance"] > 1.5 > 0.8 > da_same["proxy_a_distance"]
    assert da_shift["accuracy_gap"] == pytest.approx(0.3) and da_shift["mmd_linear"] == pytest.approx(5 * 1.5 ** 2, rel=0.25)
    cl = mo.ContinualLearningMetrics.compute([[0.9, 0.1, 0.1], [0.7, 0.9, 0.1], [0.6, 0.8, 0.9]])
    assert cl["forgetting"] > 0 and cl["average_accuracy"] == pytest.approx((0.6 + 0.8 + 0.9) / 3)

    # ---- plots, LaTeX and experiment tracking
    cm_svg = mo.ConfusionMatrixPlot().render(cm.compute(), ["a", "b", "c", "d"])
    assert cm_svg.count("<rect") == 1 + 16 and ">a<" in cm_svg
    assert "loss" in mo.LearningCurvePlot().render({"loss": [1.0, 0.5, 0.3], "val": [1.1, 0.7, 0.6]})
    fi = mo.FeatureImportancePlot().render({"age": 0.5, "income": -0.2, "zip": 0.05})
    assert fi.index("age") < fi.index("income") < fi.index("zip") and "#d62728" in fi
    tex = mo.LatexReportBuilder("Main results").add("base_line", {"acc": 0.81, "ece": 0.09}, {"ece": False}).add("ours", {"acc": 0.86, "ece": 0.04}).build()
    assert r"\textbf{0.860}" in tex and r"\textbf{0.040}" in tex and r"base\_line" in tex and r"\toprule" in tex and r"\textbf{0.810}" not in tex
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        tr = mo.ExperimentTracker(d)
        for name, lr, final in (("a", 0.1, 0.8), ("b", 0.01, 0.9)):
            rid = tr.start_run(name, {"lr": lr})
            for step, v in enumerate((0.5, final)):
                tr.log_metrics({"acc": v, "loss": 1 - v}, step)
            tr.end_run()
        assert tr.best_run("acc") == "0001-b" and tr.best_run("loss", "min") == "0001-b" and tr.compare("acc")[0][0] == "0001-b"
        saved = json.loads((Path(d) / "0000-a.json").read_text())
        assert saved["params"] == {"lr": 0.1} and saved["metrics"]["acc"][-1] == [1, 0.8] and saved["status"] == "finished"
        tr.to_mlflow("0001-b", Path(d) / "mlruns")
        assert len(list((Path(d) / "mlruns").rglob("metrics/acc"))) == 1


def test_tabular_preprocessing_columnar_files_collate_policies_and_text_transforms(tmp_path):
    import time
    import numpy as np
    import pyarrow as pa
    import pyarrow.feather as feather
    import pyarrow.parquet as pq
    from scipy import signal as sps
    from sklearn import feature_selection as skf
    from sklearn import preprocessing as skp
    from torsh_b200.data import tabular as tb

    g = torch.Generator().manual_seed(0)
    x = torch.randn(200, 4, generator=g, dtype=torch.float64) * torch.tensor([1.0, 5, 0.1, 0]) + torch.tensor([0.0, 10, -3, 7])
    ss = tb.StandardScaler().fit(x)
    assert np.allclose(ss.transform(x).numpy(), skp.StandardScaler().fit_transform(x.numpy())) and torch.allclose(ss.inverse_transform(ss.transform(x)), x)
    inc = tb.StandardScaler()
    for lo in range(0, 200, 50):
        inc.partial_fit(x[lo:lo + 50])
    assert torch.allclose(inc.mean_, ss.mean_) and torch.allclose(inc.scale_, ss.scale_)
    mm = tb.MinMaxScaler((-1, 1)).fit(x)
    assert np.allclose(mm.transform(x).numpy(), skp.MinMaxScaler((-1, 1)).fit_transform(x.numpy())) and torch.allclose(mm.inverse_transform(mm.transform(x))[:, :3], x[:, :3])
    assert np.allclose(tb.RobustScaler().fit_transform(x[:, :3]).numpy(), skp.RobustScaler().fit_transform(x[:, :3].numpy()))
    le = tb.LabelEncoder().fit(["cat", "dog", "ant", "dog"])
    assert le.classes_ == ["ant", "cat", "dog"] and le.transform(["dog", "ant"]).tolist() == [2, 0] and le.inverse_transform([1]) == ["cat"]
    with pytest.raises(ValueError):
        le.transform(["emu"])
    oh = tb.OneHotEncoder(handle_unknown="ignore").fit([["r", "g", "b", "g"], [1, 2, 1, 2]])
    enc = oh.transform([["g", "x"], [2, 1]])
    assert enc.tolist() == [[0, 1, 0, 0, 1], [0, 0, 0, 1, 0]] and oh.feature_names(["c", "n"]) == ["c=b", "c=g", "c=r", "n=1", "n=2"]
    assert tb.OneHotEncoder(drop_first=True).fit_transform([["r", "g", "b"]]).shape == (3, 2)
    holes = torch.tensor([[1.0, float("nan")], [3.0, 4.0], [float("nan"), 4.0], [5.0, 8.0]])
    assert torch.allclose(tb.SimpleImputer("mean").fit_transform(holes), torch.tensor([[1.0, 16 / 3], [3, 4], [3, 4], [5, 8]]))
    assert tb.SimpleImputer("median").fit_transform(holes)[2, 0] == 3 and tb.SimpleImputer("most_frequent").fit_transform(holes)[0, 1] == 4
    ind = tb.SimpleImputer("constant", -1.0, add_indicator=True).fit_transform(holes)
    assert ind.shape == (4, 4) and ind[0].tolist() == [1, -1, 0, 1]
    vt = tb.VarianceThreshold(1e-6).fit(x)
    assert vt.support_.tolist() == [True, True, True, False] and vt.transform(x).shape == (200, 3)
    y = (x[:, 0] + 0.2 * torch.randn(200, generator=g, dtype=torch.float64) > 0).long()
    f, p = tb.f_classif(x[:, :3], y)
    f_ref, p_ref = skf.f_classif(x[:, :3].numpy(), y.numpy())
    assert np.allclose(f.numpy(), f_ref) and np.allclose(p.numpy(), p_ref)
    assert tb.SelectKBest(1).fit(x[:, :3], y).support_.tolist() == [True, False, False]

    # ---- CSV, Arrow, Parquet
    csv_path = tmp_path / "t.csv"
    csv_path.write_text("age,city,income,label\n31,paris,1000.5,yes\n,rome,NA,no\n45,paris,3000,yes\n")
    ds = tb.CSVDataset(csv_path, target="label")
    assert ds.feature_names == ["age", "city", "income"] and ds.encoders["city"].classes_ == ["paris", "rome"] and ds.targets.tolist() == [1, 0, 1]
    assert torch.isnan(ds.features[1, 0]) and torch.isnan(ds.features[1, 2]) and ds.features[:, 1].tolist() == [0, 1, 0] and float(ds[0][0][2]) == 1000.5
    assert tb.CSVDataset(csv_path, target="label", usecols=["age"]).features.shape == (3, 1)
    table = pa.table({"a": np.arange(10, dtype=np.float32), "b": np.arange(10, dtype=np.int64) * 2, "kind": ["x", "y"] * 5, "y": np.arange(10) % 3})
    ad = tb.ArrowDataset(table, target="y")
    assert ad.features.shape == (10, 3) and ad.targets.dtype == torch.long and ad.features[3].tolist() == [3.0, 6.0, 1.0] and ad.schema["a"] == "float"
    feather.write_feather(table, tmp_path / "t.arrow")
    assert torch.equal(tb.ArrowDataset(tmp_path / "t.arrow", target="y").features, ad.features)
    big = pa.table({"f0": np.arange(100, dtype=np.float32), "f1": np.arange(100, dtype=np.float32) ** 2, "y": np.arange(100) % 2})
    pq.write_table(big, tmp_path / "t.parquet", row_group_size=25)
    pds = tb.ParquetDataset(tmp_path / "t.parquet", target="y", columns=["f1"])
    assert pds.num_row_groups == 4 and pds.num_rows == 100
    rows = list(pds)
    assert len(rows) == 100 and float(rows[7][0][0]) == 49.0 and int(rows[7][1]) == 1
    sh = [list(pds.shard(r, 2)) for r in range(2)]
    assert len(sh[0]) == len(sh[1]) == 50 and float(sh[1][0][0][0]) == 625.0
    batches = list(tb.ParquetDataset(tmp_path / "t.parquet", target="y", batch_rows=10))
    assert len(batches) == 12 and batches[0][0].shape == (10, 2) and batches[2][0].shape == (5, 2)
    assert pds.materialize().features.shape == (100, 1)
    arr = tb.ArrayDataset(torch.arange(6.0).reshape(3, 2), [0, 1, 0], transform=lambda v: v * 2)
    assert arr[1][0].tolist() == [4.0, 6.0] and int(arr[1][1]) == 1

    # ---- folds
    folds = list(tb.KFold(3).split(10))
    assert [len(te) for _, te in folds] == [4, 3, 3] and sorted(torch.cat([te for _, te in folds]).tolist()) == list(range(10))
    assert all(not set(tr.tolist()) & set(te.tolist()) for tr, te in folds)
    lab = torch.tensor([0] * 12 + [1] * 6)
    for tr, te in tb.StratifiedKFold(3, shuffle=True).split(lab):
        assert int((lab[te] == 0).sum()) == 4 and int((lab[te] == 1).sum()) == 2
    groups = ["a"] * 5 + ["b"] * 3 + ["c"] * 3 + ["d"] * 1
    for tr, te in tb.GroupKFold(2).split(groups):
        assert not {groups[i] for i in tr.tolist()} & {groups[i] for i in te.tolist()} and len(te) == 6
    tr_ds, te_ds = next(tb.KFold(3).subsets(arr))
    assert len(tr_ds) == 2 and len(te_ds) == 1

    # ---- collate
    dc = tb.DefaultCollate()
    out = dc([{"x": torch.ones(2), "n": 1, "s": "a", "t": (torch.zeros(1), 2.0)}, {"x": torch.zeros(2), "n": 2, "s": "b", "t": (torch.ones(1), 3.0)}])
    assert out["x"].shape == (2, 2) and out["n"].tolist() == [1, 2] and out["s"] == ["a", "b"] and out["t"][0].shape == (2, 1) and out["t"][1].tolist() == [2.0, 3.0]
    seqs = [torch.arange(3), torch.arange(5), torch.arange(1)]
    padded, lens = tb.PadCollate(-1, pad_to_multiple=4)(seqs)
    assert padded.shape == (3, 8) and lens.tolist() == [3, 5, 1] and padded[2].tolist() == [0] + [-1] * 7
    left = tb.PadCollate(0, side="left")(seqs)[0]
    assert left[0].tolist() == [0, 0, 0, 1, 2]
    ids, lengths, labels = tb.PadCollate()([(s, i) for i, s in enumerate(seqs)])
    assert ids.shape == (3, 5) and labels.tolist() == [0, 1, 2] and lengths.tolist() == [3, 5, 1]
    dpad = tb.PadCollate()([{"tok": s, "y": 1} for s in seqs])
    assert dpad["tok"].shape == (3, 5) and dpad["tok_lengths"].tolist() == [3, 5, 1]
    frames = tb.PadCollate(dim=0)([torch.ones(2, 3), torch.ones(4, 3)])[0]
    assert frames.shape == (2, 4, 3) and float(frames[0, 2:].sum()) == 0
    sp = tb.SparseCollate((6,))([(torch.tensor([1, 4]), torch.tensor([1.0, 2.0])), (torch.tensor([0]), torch.tensor([3.0]))])
    assert sp.shape == (2, 6) and sp.to_dense().tolist() == [[0, 1, 0, 0, 2, 0], [3, 0, 0, 0, 0, 0]]
    mixed = tb.MixedCollate({"tok": lambda v: tb.PadCollate()(v)[0], "meta": list})([{"tok": s, "meta": {"i": i}, "y": i} for i, s in enumerate(seqs)])
    assert mixed["tok"].shape == (3, 5) and mixed["meta"][2] == {"i": 2} and mixed["y"].tolist() == [0, 1, 2]
    var = [torch.zeros(n) for n in (2, 30, 3, 28, 4, 5)]
    dyn = tb.DynamicBatchCollate(max_tokens=60)(var)
    assert [b[0].shape for b in dyn] == [(4, 5), (2, 30)] and all(b[0].numel() <= 60 for b in dyn)
    cc = tb.CachedCollate(capacity=2)
    b1 = [torch.ones(2), torch.zeros(2)]
    assert cc(b1) is cc(b1) and (cc.hits, cc.misses) == (1, 1)
    st = tb.TensorStacker()([torch.ones(2, 2), torch.zeros(2, 2)])
    assert st.shape == (2, 2, 2)

    # ---- samplers and registry
    cost = lambda i: float(i % 5 + 1)
    abs_ = tb.AdaptiveBatchSampler(50, cost, budget=10.0, shuffle=False)
    bs = list(abs_)
    assert sorted(i for b in bs for i in b) == list(range(50)) and all(sum(cost(i) for i in b) <= 10 for b in bs)
    abs2 = tb.AdaptiveBatchSampler(50, cost, 10.0, target_seconds=1.0)
    abs2.report(4.0)
    assert abs2.budget == pytest.approx(10 * 0.5 ** 0.5)
    gsm = list(tb.GroupedSampler([i % 3 for i in range(20)], 4))
    assert sorted(i for b in gsm for i in b) == list(range(20)) and all(len({i % 3 for i in b}) == 1 for b in gsm)
    assert all(len(b) == 4 for b in tb.GroupedSampler([i % 3 for i in range(20)], 4, drop_last=True))
    fsam = tb.FederatedSampler([10, 1000, 10, 10], 2, "proportional", seed=0)
    picks = Counter(c for _ in range(200) for c in fsam.sample())
    assert picks[1] > 190 and fsam.aggregation_weights([0, 1]).tolist() == pytest.approx([10 / 1010, 1000 / 1010])
    caps = [{"compute": 1, "bandwidth": 1, "battery": 0.1}, {"compute": 2, "bandwidth": 1, "battery": 0.9}, {"compute": 1, "bandwidth": 1, "battery": 0.9}]
    assert all(0 not in tb.FederatedSampler([1, 1, 1], 2, "capability", caps, seed=s).sample() for s in range(5))
    ps = list(tb.PrivateSampler(10000, 0.01, 20, seed=0))
    sizes = torch.tensor([len(b) for b in ps], dtype=torch.float)
    assert len(ps) == 20 and float(sizes.mean()) == pytest.approx(100, abs=10) and float(sizes.std()) > 3
    reg = tb.DatasetRegistry()
    @reg.register("toy", description="three rows")
    def _toy(scale=1.0): return tb.ArrayDataset(torch.arange(3.0) * scale)
    assert "toy" in reg and reg.list() == {"toy": "three rows"} and float(reg.build("toy", scale=2.0)[2]) == 4.0
    with pytest.raises(KeyError):
        reg.build("nope")
    with pytest.raises(KeyError):
        reg.register("toy", _toy)

    # ---- text
    s = "  The  Quick brown fox, aged 12.5, jumped over 2 lazy dogs!  "
    for t in (tb.ToLowercase(), tb.RemoveNumbers(), tb.RemovePunctuation(), tb.CollapseWhitespace(), tb.TrimWhitespace()):
        s = t(s)
    assert s == "the quick brown fox aged jumped over lazy dogs"
    toks = tb.FilterByLength(4)(tb.RemoveStopwords()(tb.Tokenize()(s)))
    assert toks == ["quick", "brown", "aged", "jumped", "lazy", "dogs"]
    assert tb.NGrams(2)(["a", "b", "c"]) == ["a b", "b c"] and tb.NGrams(2, None, True)(["a", "b"]) == [("a",), ("b",), ("a", "b")]
    assert tb.ReplacePattern(r"\d+", "<num>")("room 42") == "room <num>"
    vocab = tb.Vocabulary.build([["a", "b", "a"], ["a", "c", "b", "rare"]], min_freq=2)
    assert vocab.itos == ["<pad>", "<unk>", "<bos>", "<eos>", "a", "b"] and vocab.encode(["a", "rare"]) == [4, 1]
    ids = tb.FixedLength(6)(tb.AddSpecialTokens()(vocab.encode(["b", "a"])))
    assert ids == [2, 5, 4, 3, 0, 0] and vocab.decode(ids) == ["b", "a"] and tb.TokenIdsToTensor()(ids).dtype == torch.long
    assert tb.FixedLength(2, truncate="left")([1, 2, 3]) == [2, 3] and tb.FixedLength(4)(torch.arange(2)).tolist() == [0, 1, 0, 0]
    assert len(tb.Vocabulary.build([["a", "b", "c", "d"]], max_size=6)) == 6
    bpe = tb.SimpleBPE(20).fit(["low low low lower lowest", "new newer newest wide wider widest"] * 3)
    assert bpe.merges[0] in (("l", "o"), ("e", "r"), ("e", "s"), ("w", "e"), ("o", "w")) and "low</w>" in bpe.encode("low")
    pieces = bpe.encode("lowest newer")
    assert bpe.decode(pieces) == "lowest newer" and len(pieces) < len("lowest newer")
    tcd = tb.TextClassificationDataset(["Good film!", "bad film", "good, good plot"], ["pos", "neg", "pos"], max_len=4)
    assert tcd.ids.shape == (3, 4) and tcd.labels.tolist() == [1, 0, 1] and tcd.lengths.tolist() == [2, 2, 3]
    assert int(tcd[0][0][0]) == tcd.vocab.stoi["good"] and int(tcd[0][0][2]) == 0
    txt = tmp_path / "lines.txt"
    txt.write_text("first line\n\nsecond línea\nthird\n", encoding="utf-8")
    tf = tb.TextFileDataset(txt, transform=str.upper)
    assert len(tf) == 3 and tf[1] == "SECOND LÍNEA" and tf[2] == "THIRD"

    # ---- audio and image sample transforms
    sr = 16000
    tt = torch.arange(sr, dtype=torch.float64) / sr
    tone = torch.sin(2 * math.pi * 440 * tt)
    down = tb.Resample(16000, 8000)(tone)
    ref = sps.resample_poly(tone.numpy(), 1, 2)
    assert down.shape == (8000,) and float((down[200:-200] - torch.from_numpy(ref)[200:-200]).abs().max()) < 5e-3
    up = tb.Resample(8000, 22050)(down[None])
    assert up.shape == (1, 22050)
    spec = torch.fft.rfft(up[0]).abs()
    assert abs(int(spec.argmax()) - 440) <= 1
    alias = tb.Resample(16000, 8000)(torch.sin(2 * math.pi * 6000 * tt))                # above the new Nyquist: removed, not folded
    assert float(alias[500:-500].abs().max()) < 0.02
    noisy = tb.AddNoise((20.0, 20.0), seed=0)(tone)
    snr = 10 * math.log10(float(tone.pow(2).mean() / (noisy - tone).pow(2).mean()))
    assert snr == pytest.approx(20.0, abs=0.3)
    img = torch.rand(3, 8, 8, generator=g)
    assert float(tb.RandomBrightness(0.5, seed=1)(img).max()) <= 1.0 and tb.RandomContrast(0.0)(img).allclose(img)
    assert float((tb.GaussianNoise(0.1, seed=0)(img) - img).std()) == pytest.approx(0.1, rel=0.2)
    eng = tb.OnlineAugmentationEngine([lambda v: v + 1], strength=0.2, target_gap=0.05, step=0.1)
    for _ in range(3):
        eng.report(0.95, 0.80)
    assert eng.strength == pytest.approx(0.5)
    eng.report(0.6, 0.6)
    assert eng.strength == pytest.approx(0.4)
    eng.strength = 1.0
    assert float(eng(torch.zeros(()))) == 1.0

    # ---- utilities
    calls, slept = {"n": 0}, []
    def flaky():
        calls["n"] += 1
        if calls["n"] < 3:
            raise OSError("transient")
        return "ok"
    rs = tb.RetryStrategy(4, 0.1, 2.0, sleep=slept.append)
    assert rs.run(flaky) == "ok" and slept == [0.1, 0.2] and rs.delays() == [0.1, 0.2, 0.4]
    with pytest.raises(ValueError):
        tb.RetryStrategy(3, sleep=slept.append).run(lambda: (_ for _ in ()).throw(ValueError("not retried")))
    with pytest.raises(OSError):
        tb.RetryStrategy(2, sleep=slept.append).run(lambda: (_ for _ in ()).throw(OSError("always")))
    now = [0.0]
    pt = tb.ProgressTracker(100, clock=lambda: now[0])
    now[0] = 2.0
    pt.update(20)
    assert pt.rate() == 10.0 and pt.eta() == 8.0 and "20/100 (20.0%)" in str(pt)
    cache = tb.ConcurrentCache(2)
    produced = []
    def slow(k):
        def f():
            time.sleep(0.05)
            produced.append(k)
            return k * 2
        return f
    threads = [threading.Thread(target=lambda: cache.get_or_compute(7, slow(7))) for _ in range(6)]
    [t.start() for t in threads]; [t.join() for t in threads]
    assert produced == [7] and cache.get_or_compute(7, slow(7)) == 14 and cache.misses == 1
    cache.get_or_compute(1, slow(1)); cache.get_or_compute(2, slow(2))
    assert len(cache) == 2 and 7 not in cache.data
    sc = tb.StatisticsCollector(0)
    imgs = torch.rand(10, 3, 5, 5, generator=g)
    for im in imgs:
        sc.update(im)
    stt = sc.compute()
    assert torch.allclose(stt["mean"], imgs.double().mean((0, 2, 3))) and torch.allclose(stt["std"], imgs.double().std((0, 2, 3), unbiased=False)) and stt["count"] == 250
    buf = bytearray(np.arange(12, dtype=np.float32).tobytes())
    z = tb.ZeroCopyTensor(buf, torch.float32, (2, 4), offset=16)
    assert z.tensor[0].tolist() == [4, 5, 6, 7]
    z.tensor[0, 0] = 99.0
    assert np.frombuffer(buf, dtype=np.float32)[4] == 99.0 and z.shares_memory_with(z.tensor[1])
    bm = tb.BufferManager()
    a = bm.acquire(1000)
    assert len(a) == 1024
    bm.release(a)
    assert bm.acquire(600) is a and (bm.allocated, bm.reused) == (1, 1)
