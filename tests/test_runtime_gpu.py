"""Native device runtime on a B200: pools, streams, events, CUDA-graph cache."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_info_and_occupancy():
    from torsh_b200.core import runtime as rt
    info = rt.device_info()
    assert info.sm_count >= 100 and info.capability[0] >= 10 and info.tmem_columns == 512
    assert info.smem_per_block_optin >= 200 * 1024 and info.total_memory > 100 << 30
    n, lim = rt.occupancy(192, 128, 200 * 1024)
    assert n == 1 and lim == "shared memory"
    n, lim = rt.occupancy(256, 32, 0)
    assert n >= 4


def test_device_and_pinned_pool_roundtrip():
    from torsh_b200.core import runtime as rt
    pool = rt.DeviceMemoryPool
    base = pool.stats()
    buf = pool.alloc(3 << 20)
    t = buf.tensor((1 << 18,), torch.float32)
    t.fill_(2.5)
    assert t.sum().item() == 2.5 * (1 << 18)
    s1 = pool.stats()
    assert s1["allocated_bytes"] - base["allocated_bytes"] == 4 << 20
    p0 = buf.ptr
    del t
    buf.free()
    again = pool.alloc(4 << 20)
    assert again.ptr == p0 and pool.stats()["cache_hits"] > base["cache_hits"]
    again.free()
    assert pool.empty_cache() >= 4 << 20 and pool.pressure() == "low"
    pin = rt.PinnedBuffer(1 << 20)
    h = pin.tensor((1 << 18,), torch.float32)
    h.copy_(torch.arange(1 << 18, dtype=torch.float32))
    d = torch.empty(1 << 18, device="cuda")
    pin.copy_to_device_async(d)
    torch.cuda.synchronize()
    assert torch.equal(d.cpu(), torch.arange(1 << 18, dtype=torch.float32))
    pin.free()


def test_stream_pool_events_and_graph_cache():
    from torsh_b200.core import runtime as rt
    from torsh_b200.ops import elementwise as ew
    sp = rt.StreamPool(2)
    hi, lo = sp.get(rt.HIGH), sp.get(rt.LOW)
    assert sp.priority(hi) <= sp.priority(lo)
    raws = {sp.get_raw(rt.NORMAL) for _ in range(6)}
    assert len(raws) == 2                                  # round robin over a pool of two
    x = torch.randn(1 << 20, device="cuda")
    y = torch.empty_like(x)
    e0, e1 = rt.Event(True), rt.Event(True)
    hi.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(hi):
        e0.record(hi)
        ew.unary_raw("relu", x, out=y)
        e1.record(hi)
    e1.synchronize()
    assert e1.query() and e0.elapsed_ms(e1) > 0 and torch.equal(y, torch.relu(x))
    e0.release(); e1.release()
    e2 = rt.Event(True)
    assert rt.Event.pool_stats()["reused"] >= 1
    e2.release()
    # capture two of this library's kernels into a cached graph and replay it on new data
    gc = rt.GraphCache()
    key = gc.key("relu-then-square", tuple(x.shape))
    z = torch.empty_like(x)
    if not gc.has(key):
        gc.capture(key, lambda: (ew.unary_raw("relu", x, out=y), ew.unary_raw("square", y, out=z)))
    assert gc.has(key) and gc.node_count(key) == 2
    x.copy_(torch.randn_like(x))
    gc.launch(key)
    torch.cuda.synchronize()
    assert torch.allclose(z, torch.relu(x) ** 2)
    assert gc.stats()["entries"] >= 1
    gc.clear()


def test_bounded_wait_reports_timeout_and_context_survives():
    """A flag that nothing sets: the wait gives up after its limit, records the error in the status word, the host
    turns it into KernelTimeout, and the next launches on the same context work."""
    import ctypes

    from torsh_b200 import _native as nv
    from torsh_b200.ops import elementwise as ew
    lib = nv.require_cuda()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    st = nv.status_word()
    st.zero_()
    lib.tb_wait_probe.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    # satisfied wait: no error
    flag.fill_(5)
    nv.check(lib.tb_wait_probe(flag.data_ptr(), 5, 50_000_000, st.data_ptr(), waited.data_ptr(), nv.stream_ptr()), "wait_probe")
    nv.check_status()
    # a flag nobody sets, 50 ms limit
    flag.zero_()
    nv.check(lib.tb_wait_probe(flag.data_ptr(), 1, 50_000_000, st.data_ptr(), waited.data_ptr(), nv.stream_ptr()), "wait_probe")
    with pytest.raises(nv.KernelTimeout, match="peer"):
        nv.check_status()
    assert 45e6 < waited.item() < 500e6
    nv.check_status()                                   # the status word was reset
    x = torch.randn(1024, device="cuda")
    assert torch.equal(ew.unary_raw("relu", x), torch.relu(x))
    assert lib.tb_wait_probe(flag.data_ptr(), 1, 2_000_000_000, st.data_ptr(), None, nv.stream_ptr()) != 0   # > 1 s refused


def test_unified_buffer_is_visible_from_host_and_device():
    import torch
    from torsh_b200.core import runtime as rt
    n = 1 << 20
    buf = rt.UnifiedBuffer(n * 4)
    host = buf.host_view((n,), torch.float32)
    host.copy_(torch.arange(n, dtype=torch.float32))
    buf.advise(rt.UnifiedBuffer.READ_MOSTLY)
    buf.prefetch()                                       # pages move to the GPU ahead of the copy
    dev = torch.empty(n, device="cuda")
    buf.copy_to(dev)
    torch.cuda.synchronize()
    assert torch.equal(dev.cpu(), torch.arange(n, dtype=torch.float32))
    buf.prefetch(-1)
    torch.cuda.synchronize()
    assert float(host[12345]) == 12345.0
    del host
    buf.free()


def test_device_side_index_checks_report_through_the_status_word():
    """With the checks on, a token id outside the vocabulary and a class target outside [0, C) leave code 108 in the
    status word (the kernels skip the access either way, nothing traps); with the checks off the same calls stay silent."""
    from torsh_b200 import _native as nv
    from torsh_b200.ops import elementwise as ew
    from torsh_b200.ops import softmax as sm
    dev = torch.device("cuda", torch.cuda.current_device())
    wte = torch.randn(64, 32, device=dev, dtype=torch.bfloat16)
    good = torch.randint(0, 64, (2, 8), device=dev)
    bad = good.clone()
    bad[1, 3] = 64
    logits = torch.randn(16, 40, device=dev, dtype=torch.bfloat16)
    tgt_bad = torch.randint(0, 40, (16,), device=dev)
    tgt_bad[5] = 41
    torch.cuda.synchronize()
    nv.check_status()
    nv.enable_kernel_checks(True)
    try:
        ew.embedding(good, wte, None)
        torch.cuda.synchronize()
        nv.check_status()                                    # in-range ids: silent
        out = ew.embedding(bad, wte, None)
        torch.cuda.synchronize()
        with pytest.raises(nv.KernelCheckFailed, match="108"):
            nv.check_status()
        assert torch.equal(out[1, 3], wte[0])                # the bad id was clamped, not followed
        sm.cross_entropy(logits, tgt_bad)
        torch.cuda.synchronize()
        with pytest.raises(nv.KernelCheckFailed):
            nv.check_status()
    finally:
        nv.enable_kernel_checks(False)
    ew.embedding(bad, wte, None)
    sm.cross_entropy(logits, tgt_bad)
    torch.cuda.synchronize()
    nv.check_status()                                        # checks off: the same calls leave no code


def test_graphed_step_replays_a_training_step():
    """A small ResNet training step captured by GraphedStep gives the same parameters as the same steps run eagerly."""
    import copy
    from torsh_b200.engine import GraphedStep
    from torsh_b200.models import create_model
    from torsh_b200.optim.fused import SGD
    torch.manual_seed(0)
    base = create_model("resnet18").cuda().train()
    base.use_kernels = True
    x = torch.randn(8, 3, 64, 64, device="cuda").to(torch.bfloat16)
    y = torch.randint(0, 1000, (8,), device="cuda")
    results = []
    for graphed in (False, True):
        model = copy.deepcopy(base)
        opt = SGD(model.parameters(), lr=1e-3, momentum=0.9, zero_grad_in_step=True)   # small steps: the comparison stays well conditioned

        def step(x, y):
            loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            opt.step()
            return loss
        gs = GraphedStep(step, [torch.empty_like(x), torch.empty_like(y)], warmup=2, enabled=graphed)
        losses = [float(gs(x, y).detach()) for _ in range(6)]
        assert (gs.graph is not None) == graphed and gs.error is None
        results.append((losses, [p.detach().float().clone() for p in model.parameters()]))
    (l0, p0), (l1, p1) = results
    # The loss falls from about 7 to about 1 over the six steps; a skipped, doubled or stale step would shift the whole
    # sequence. Two eager runs already differ in the third digit (fp32 atomics in the weight gradients), so the
    # comparison is by tolerance, and only weight matrices are compared (biases start at zero: no scale to relate to).
    assert l0[0] > 2 * l0[-1]
    assert all(abs(a - b) <= 5e-2 * max(abs(a), 1.0) for a, b in zip(l0, l1))
    for a, b in zip(p0, p1):
        if a.dim() >= 2:
            assert ((a - b).norm() / a.norm().clamp(min=1e-6)).item() < 0.15
