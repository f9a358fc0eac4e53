"""CPU tests of the API breadth: optimizers, schedulers, autograd utilities, data, formats, fault tolerance, MoE."""
import math

import pytest
import torch


def test_reference_optimizer_arithmetic():
    """AdamW / SGD / LAMB against hand-written restatements of the reference formulas."""
    from torsh_b200 import optim as O
    torch.manual_seed(0)
    w0, g = torch.randn(7), torch.randn(7)
    # AdamW: decay, moments, both bias corrections, eps outside the sqrt of v-hat
    p = torch.nn.Parameter(w0.clone()); p.grad = g.clone()
    O.AdamW([p], lr=0.1, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01).step()
    w = w0 - 0.1 * 0.01 * w0
    m, v = 0.1 * g, 0.001 * g * g
    exp = w - 0.1 * (m / 0.1) / ((v / 0.001).sqrt() + 1e-8)
    assert torch.allclose(p.data, exp, atol=1e-6)
    # SGD nesterov with weight decay, buffer starting at zero
    p = torch.nn.Parameter(w0.clone()); p.grad = g.clone()
    O.SGD([p], lr=0.1, momentum=0.9, weight_decay=0.1, nesterov=True).step()
    d = g + 0.1 * w0
    buf = d.clone()
    assert torch.allclose(p.data, w0 - 0.1 * (d + 0.9 * buf), atol=1e-6)
    with pytest.raises(ValueError):
        O.SGD([p], lr=0.1, momentum=0.0, nesterov=True)
    # LAMB: coupled decay before the moments, trust ratio clamped to <= 1
    p = torch.nn.Parameter(w0.clone()); p.grad = g.clone()
    O.LAMB([p], lr=0.1, weight_decay=0.01).step()
    gg = g + 0.01 * w0
    u = ((0.1 * gg) / 0.1) / (((0.001 * gg * gg) / 0.001).sqrt() + 1e-6)
    trust = min(w0.norm().item() / u.norm().item(), 1.0)
    assert torch.allclose(p.data, w0 - 0.1 * trust * u, atol=1e-6)


@pytest.mark.parametrize("name", ["Lion", "AdaBelief", "AdaBound", "Yogi", "LARS", "FTRL", "SophiaG", "ScheduleFreeSGD",
                                  "Prodigy", "Adagrad", "RMSprop", "NAdam", "RAdam", "Adamax", "Adadelta"])
def test_optimizer_zoo_descends(name):
    from torsh_b200 import optim as O
    w = torch.nn.Parameter(torch.tensor([3.0, -2.0]))
    kw = {"Lion": dict(lr=1e-2), "LARS": dict(lr=0.5, eta=0.1), "FTRL": dict(lr=0.5), "Adadelta": dict(lr=5.0),
          "ScheduleFreeSGD": dict(lr=0.1), "Prodigy": {}}.get(name, dict(lr=5e-2))
    opt = getattr(O, name)([w], **kw)
    start = (w ** 2).sum().item()
    for _ in range(150):
        opt.zero_grad()
        (w ** 2).sum().backward()
        opt.step()
    assert (w ** 2).sum().item() < 0.6 * start


def test_lr_schedulers():
    from torsh_b200 import optim as O
    from torsh_b200.optim import lr_scheduler as S
    def lrs(make, n):
        opt = O.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
        s = make(opt)
        out = []
        for _ in range(n):
            out.append(opt.get_lr()[0])
            s.step()
        return out
    assert lrs(lambda o: S.StepLR(o, 2, 0.5), 5) == [1.0, 1.0, 0.5, 0.5, 0.25]
    assert lrs(lambda o: S.MultiStepLR(o, [1, 3], 0.1), 4) == pytest.approx([1.0, 0.1, 0.1, 0.01])
    c = lrs(lambda o: S.CosineAnnealingLR(o, 10), 11)
    assert c[5] == pytest.approx(0.5) and c[10] == pytest.approx(0.0, abs=1e-9)
    w = lrs(lambda o: S.PolynomialDecayWithWarmup(o, 4, 10), 10)
    assert w[:4] == pytest.approx([0.25, 0.5, 0.75, 1.0]) and w[-1] < w[4]
    oc = lrs(lambda o: S.OneCycleLR(o, max_lr=1.0, total_steps=20), 20)
    assert max(oc) == pytest.approx(1.0, abs=1e-6) and oc[0] == pytest.approx(0.04) and oc[-1] < 1e-3
    opt = O.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    p = S.ReduceLROnPlateau(opt, factor=0.5, patience=1)
    for m in (1.0, 1.0, 1.0, 1.0):
        p.step(m)
    assert opt.get_lr()[0] == 0.5


def test_autograd_utilities():
    from torsh_b200 import autograd as A
    a = torch.nn.Parameter(torch.ones(4)); a.grad = torch.full((4,), 3.0)
    n = A.clip_grad_norm([a], 1.0)
    assert n.item() == pytest.approx(6.0) and a.grad.norm().item() == pytest.approx(1.0, rel=1e-4)
    A.clip_grad_value([a], 0.1)
    assert a.grad.max().item() <= 0.1 + 1e-7
    x = torch.randn(3, dtype=torch.double, requires_grad=True)
    assert A.gradcheck(lambda t: (t ** 3).sum(), (x,))
    ng = A.numerical_gradient(lambda t: (t ** 2).sum(), torch.tensor([1.0, -2.0]))
    assert torch.allclose(ng, torch.tensor([2.0, -4.0], dtype=torch.double), atol=1e-5)
    assert A.CheckpointScheduler(A.CheckpointStrategy.SQRT).plan(9) == [False, True, True] * 3
    assert A.has_nan_or_inf(torch.tensor([1.0, float("nan")])) and not A.has_nan_or_inf(torch.ones(2))
    with A.no_grad():
        assert not A.is_grad_enabled()


def test_distributed_sampler_contiguous_blocks():
    from torsh_b200.data import DistributedSampler
    parts = [DistributedSampler(10, 4, r, shuffle=False).indices() for r in range(4)]
    assert parts[0] == [0, 1, 2] and parts[3] == [9, 0, 1]                     # wrap-around padding, contiguous blocks
    sh = [DistributedSampler(10, 2, r, shuffle=True) for r in range(2)]
    assert sorted(sh[0].indices() + sh[1].indices()) == list(range(10))
    assert sh[0].indices() == DistributedSampler(10, 2, 0, shuffle=True, seed=42).indices()
    d = DistributedSampler(10, 4, 0, shuffle=False, drop_last=True)
    assert len(d) == 2 and d.indices() == [0, 1]


def test_dataloader_config_and_prefetch():
    from torsh_b200.data import DataLoader, DataLoaderConfig, PrefetchToDevice, SyntheticTokenDataset
    ds = SyntheticTokenDataset(100, 8, 10)
    dl = DataLoader(ds, DataLoaderConfig(batch_size=4, drop_last=False))
    batches = list(PrefetchToDevice(dl, "cpu"))
    assert [b[0].shape[0] for b in batches] == [4, 4, 2] and torch.equal(batches[0][0][0, 1:], batches[0][1][0, :-1])


def test_model_state_and_checkpoint_roundtrip(tmp_path):
    from torsh_b200 import nn, optim
    from torsh_b200.serialize import checkpoint as ck, model_state as ms
    m = nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2))
    st = ms.model_state(m, {"hidden": 3, "name": "mlp", "p": 0.5, "flag": True, "dims": [4, 3, 2]})
    ms.save_json(st, tmp_path / "a.json"); ms.save_binary(st, tmp_path / "a.bin"); ms.save_safetensors(st, tmp_path / "a.st")
    for back in (ms.load_json(tmp_path / "a.json"), ms.load_binary(tmp_path / "a.bin"), ms.load_safetensors(tmp_path / "a.st")):
        m2 = nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2))
        ms.load_model_state(m2, back)
        assert all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), m2.state_dict().values()))
        assert back["config"]["dims"] == [4, 3, 2] and back["metadata"]["version"] == "1.0.0"
    o = optim.AdamW(m.parameters())
    m(torch.randn(2, 4)).sum().backward(); o.step()
    mgr = ck.CheckpointManager(tmp_path / "ck", max_to_keep=2)
    for s in range(4):
        mgr.save(m, o, epoch=0, global_step=s, metric=1.0 / (s + 1))
    assert sorted(p.name for p in (tmp_path / "ck").iterdir()) == ["model_best.torsh", "model_epoch_0_step_2.torsh", "model_epoch_0_step_3.torsh"]
    c = mgr.load()
    m3 = nn.Sequential(nn.Linear(4, 3), nn.ReLU(), nn.Linear(3, 2)); o3 = optim.AdamW(m3.parameters())
    ck.restore_into(c, m3, o3)
    assert torch.equal(m3[0].weight, m[0].weight) and o3.state[m3[0].weight]["step"] == 1
    dm = ck.DistributedCheckpointManager(tmp_path / "d", rank=1, world_size=2)
    dm.save(10, 1, {"flat": torch.arange(8.0)})
    (tmp_path / "d" / "checkpoint_step_12_rank_1.json").write_text("{corrupt")
    assert dm.latest_step() == 12
    from torsh_b200.core.error import TorshDistributedError
    with pytest.raises(TorshDistributedError):
        dm.load()
    assert torch.equal(dm.load(10)["model_state"]["flat"], torch.arange(8.0))


def test_module_state_dict_rules():
    from torsh_b200 import nn
    from torsh_b200.core.error import TorshError
    m = nn.Sequential(nn.Linear(2, 2), nn.BatchNorm1d(2))
    sd = m.torsh_state_dict()
    assert set(sd) == {"0.weight", "0.bias", "1.weight", "1.bias"}        # parameters only, no running stats
    with pytest.raises(TorshError, match="missing"):
        m.load_torsh_state_dict({"0.weight": sd["0.weight"]}, strict=True)
    m.load_torsh_state_dict({"0.weight": sd["0.weight"]}, strict=False)
    with pytest.raises(TorshError, match="ShapeMismatch"):
        m.load_torsh_state_dict({**sd, "0.bias": torch.zeros(3)})
    assert m.num_parameters() == 10 and m.freeze().num_parameters(trainable_only=True) == 0


def test_retry_circuit_breaker_health_and_injection():
    from torsh_b200.core.error import TorshDistributedError
    from torsh_b200.parallel import fault_tolerance as ft
    now = [0.0]
    cb = ft.CircuitBreaker(failure_threshold=2, success_threshold=2, timeout_s=10, clock=lambda: now[0])
    cb.record_failure(); assert cb.allow()
    cb.record_failure(); assert cb.state is ft.CircuitState.OPEN and not cb.allow()
    now[0] = 11; assert cb.allow() and cb.state is ft.CircuitState.HALF_OPEN
    cb.record_success(); cb.record_success(); assert cb.state is ft.CircuitState.CLOSED
    inj = ft.FaultInjector(); inj.add(ft.FaultKind.NETWORK_FAILURE, 1.0, max_count=2)
    calls = []
    ex = ft.RetryExecutor(ft.RetryConfig(max_attempts=3, initial_delay_s=0.0), sleep=lambda s: None)
    assert ex.execute(inj.wrap(lambda: calls.append(1) or "ok")) == "ok" and ex.stats["retries"] == 2
    inj.add(ft.FaultKind.PROCESS_CRASH, 1.0)                               # not retryable: fails at once
    with pytest.raises(TorshDistributedError, match="ProcessFailure"):
        ft.RetryExecutor(sleep=lambda s: None).execute(inj.wrap(lambda: None))
    hc = ft.HealthChecker(timeout_s=5, clock=lambda: now[0])
    hc.heartbeat(0); now[0] += 6; hc.heartbeat(1)
    assert hc.unhealthy() == [0]


def test_elastic_manager_detects_dead_and_new_workers():
    from torsh_b200.parallel import fault_tolerance as ft
    from torsh_b200.parallel.store import MemoryStore
    st = MemoryStore()
    for r in (0, 1):
        st.set(f"hb/{r}", repr(1000.0).encode())
    saved = []
    mgr = ft.ElasticTrainingManager(st, 0, 2, ft.ElasticConfig(max_workers=4, heartbeat_timeout_s=10), on_checkpoint=lambda: saved.append(1))
    assert mgr.check_scaling_needs(now=1005.0) is None
    st.set("hb/0", repr(1020.0).encode())                                      # rank 1 went silent
    assert mgr.check_scaling_needs(now=1021.0) is ft.ScalingEvent.WORKER_FAILURE and saved == [1]
    assert mgr.state is ft.ElasticState.SCALING
    mgr.complete_scaling()
    assert mgr.world_size == 1 and mgr.state is ft.ElasticState.STABLE and mgr.generation == 1
    st.set("hb/1", repr(1030.0).encode()); st.set("hb/0", repr(1030.0).encode())
    assert mgr.check_scaling_needs(now=1031.0) is ft.ScalingEvent.WORKER_JOIN


def test_compression_and_error_feedback():
    from torsh_b200.parallel import compression as C
    torch.manual_seed(0)
    g = torch.randn(64, 32)
    for comp, tol in ((C.TopK(0.25), None), (C.Quantization(8), 0.02), (C.SignSGD(), None), (C.Ternary(), None), (C.PowerSGD(8), None)):
        back = comp.decompress(comp.compress(g), g.shape)
        assert back.shape == g.shape
        if tol:
            assert (back - g).abs().max() < tol * (g.max() - g.min())
    ef = C.ErrorFeedback(C.TopK(0.1))
    total = torch.zeros_like(g)
    for _ in range(30):
        _, approx = ef.compress("w", g)
        total += approx
    assert ((total / 30 - g).norm() / g.norm()).item() < 0.35                   # residuals are eventually transmitted


def test_moe_router_capacity_and_layer():
    from torsh_b200.parallel.expert_parallel import ExpertParallelismConfig, MoELayer, TopKRouter
    torch.manual_seed(0)
    cfg = ExpertParallelismConfig(num_experts=4, top_k=2, capacity_factor=1.0)
    r = TopKRouter(16, cfg)
    x = torch.randn(32, 16)
    idx, w, keep, slot, aux = r(x)
    assert r.capacity(32) == 16 and idx.shape == (32, 2) and torch.allclose(w.sum(-1), torch.ones(32))
    for e in range(4):
        assert ((idx == e) & keep).sum().item() <= 16
    layer = MoELayer(16, 32, cfg)
    y, aux = layer(x.requires_grad_(True))
    (y.sum() + aux).backward()
    assert y.shape == x.shape and layer.w1.grad is not None and layer.router.gate.grad is not None


def test_ring_all_reduce_host_oracle():
    from torsh_b200.parallel.collectives import ring_all_reduce_host
    bufs = [torch.arange(10.0) * (r + 1) for r in range(3)]
    ring_all_reduce_host(bufs)
    for b in bufs:
        assert torch.equal(b, torch.arange(10.0) * 6)


def test_models_forward_shapes():
    from torsh_b200 import models as M
    assert M.VisionTransformer(M.ViTConfig.vit_tiny())(torch.randn(2, 3, 32, 32)).shape == (2, 10)
    ids = torch.randint(0, 1000, (2, 16))
    assert M.BertForMaskedLM(M.BertConfig.tiny())(ids).shape == (2, 16, 1000)
    assert M.EncoderDecoderModel(M.Seq2SeqConfig.tiny())(ids, ids).shape == (2, 16, 1000)
    assert M.ResNet.resnet18(7)(torch.randn(1, 3, 64, 64)).shape == (1, 7)
    lm = M.LlamaModel(M.LlamaConfig.tiny())
    assert lm(ids).shape == (2, 16, 1024) and "resnet50" in M.list_models()


def test_extra_layers_amp_and_second_order_optimizers():
    import warnings

    import torch

    import torsh_b200 as tb
    from torsh_b200 import nn
    from torsh_b200.optim import mixed_precision as mp
    from torsh_b200.optim import second_order as so
    torch.manual_seed(0)
    x = torch.randn(4, 8, 10, 10)
    for layer in (nn.DepthwiseSeparableConv2d(8, 16), nn.WeightStandardizedConv2d(8, 16, 3, padding=1), nn.BatchRenorm2d(8),
                  nn.VirtualBatchNorm2d(8), nn.SwitchableNorm2d(8), nn.StochasticDepth(0.5), nn.DropBlock2d(0.2, 3),
                  nn.MBConvBlock(8, 8), nn.DenseBlock(8, 4, 2)):
        y = layer(x)
        assert y.shape[0] == 4 and torch.isfinite(y).all(), type(layer).__name__
        layer.eval()
        assert torch.isfinite(layer(x)).all()
    assert nn.GlobalAvgPool2d()(x).shape == (4, 8) and nn.GlobalMaxPool2d()(x).shape == (4, 8)
    sn = nn.SwitchableNorm2d(8)
    with torch.no_grad():
        sn.mean_w.copy_(torch.tensor([-50.0, -50.0, 50.0])); sn.var_w.copy_(sn.mean_w)     # pure batch-norm mixture
    assert torch.allclose(sn(x), torch.nn.functional.batch_norm(x, None, None, training=True), atol=1e-4)
    q, k, v = torch.randn(2, 5, 6), torch.randn(2, 7, 6), torch.randn(2, 7, 6)
    out, att = nn.AdditiveAttention(6, 6, 12)(q, k, v)
    assert out.shape == (2, 5, 6) and torch.allclose(att.sum(-1), torch.ones(2, 5))
    assert nn.MultiplicativeAttention(6, 6)(q, k, v)[0].shape == (2, 5, 6)
    assert nn.CrossAttention(16, 6, heads=4)(torch.randn(2, 5, 16), k).shape == (2, 5, 16)
    fa = nn.FlexAttention(16, heads=2, pattern="sliding_window", window=3)
    m = fa.mask(6, "cpu")
    assert m[5, 3] and not m[5, 2] and not m[2, 3] and fa(torch.randn(2, 6, 16)).shape == (2, 6, 16)
    assert nn.RelativePositionBias(4)(5, 7).shape == (4, 5, 7)
    assert nn.interpolate_positions(torch.arange(8.0)[:, None].expand(8, 3), 15)[7].allclose(torch.full((3,), 3.5))
    xm, ym = nn.mixup(x, torch.tensor([0, 1, 2, 3]), 0.4, num_classes=4)
    assert xm.shape == x.shape and torch.allclose(ym.sum(1), torch.ones(4))
    xc, yc = nn.cutmix(x, torch.tensor([0, 1, 2, 3]), 1.0, num_classes=4)
    assert xc.shape == x.shape and torch.allclose(yc.sum(1), torch.ones(4))
    # loss scaling: overflow skips the step and halves the scale, clean steps grow it back
    lin = torch.nn.Linear(4, 2)
    opt = torch.optim.SGD(lin.parameters(), lr=0.1)
    sc = mp.GradScaler(init_scale=1024.0, growth_interval=2)
    taken = []
    for i in range(4):
        opt.zero_grad()
        sc.scale(lin(torch.ones(2, 4)).sum()).backward()
        assert torch.allclose(lin.bias.grad, torch.full((2,), 2.0 * sc.get_scale()))
        if i == 1:
            lin.weight.grad[0, 0] = float("inf")
        w_before = lin.weight.detach().clone()
        taken.append(sc.step(opt))
        assert torch.equal(lin.weight, w_before) == (not taken[-1])
    assert taken == [True, False, True, True] and sc.get_scale() == 1024.0 and sc.stats["backoffs"] == 1
    half = torch.nn.Linear(4, 2).to(torch.bfloat16)
    mo = mp.MixedPrecisionOptimizer(half.parameters(), torch.optim.SGD, mp.BF16Config(), lr=0.1)
    half(torch.ones(2, 4, dtype=torch.bfloat16)).sum().backward()
    assert mo.step() and mo.masters[0].dtype == torch.float32 and half.weight.dtype == torch.bfloat16
    # curvature-aware optimizers reduce a least-squares loss
    X = torch.randn(64, 8); Y = X @ torch.randn(8, 3)

    def fit(make, steps=60, graph=False, closure=False):
        torch.manual_seed(1)
        m = torch.nn.Linear(8, 3)
        o = make(m)
        l0 = ((m(X) - Y) ** 2).mean().item()
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            for _ in range(steps):
                if closure:
                    o.step(lambda: ((m(X) - Y) ** 2).mean())
                    continue
                o.zero_grad()
                ((m(X) - Y) ** 2).mean().backward(create_graph=graph)
                o.step()
        return ((m(X) - Y) ** 2).mean().item() / l0
    assert fit(lambda m: so.Shampoo(m.parameters(), lr=0.3, update_freq=1)) < 1e-3
    assert fit(lambda m: so.AdaHessian(m.parameters(), lr=0.1), graph=True) < 1e-2
    assert fit(lambda m: so.KFAC(m, lr=0.5, damping=0.1)) < 1e-6
    assert fit(lambda m: so.NewtonCG(m.parameters()), steps=4, closure=True) < 1e-8
    assert fit(lambda m: so.YellowFin(m.parameters(), lr=0.01), steps=200) < 0.05
    assert tb.optim.ElasticAveragingSGD and tb.optim.DistributedOptimizer and tb.optim.AsyncSGD


def test_trust_region_and_natural_gradient_reach_quadratic_minimum():
    from torsh_b200.optim import NaturalGradient, TrustRegion
    torch.manual_seed(0)
    A = torch.randn(6, 6)
    A = A @ A.T + torch.eye(6)
    b = torch.randn(6)
    xs = torch.linalg.solve(A, b)
    best = float(0.5 * xs @ A @ xs - b @ xs)
    x = torch.zeros(6, requires_grad=True)
    opt = TrustRegion([x], delta=1.0)
    for _ in range(15):
        loss = opt.step(lambda: 0.5 * x @ A @ x - b @ x)
    assert abs(float(loss) - best) < 1e-4
    w = torch.zeros(6, requires_grad=True)
    opt = NaturalGradient([w], lr=0.1, full_below=10)
    first = None
    for _ in range(200):
        opt.zero_grad()
        loss = 0.5 * w @ A @ w - b @ w
        loss.backward()
        opt.step()
        first = first if first is not None else float(loss.detach())
    assert float(loss.detach()) < first - 0.5 * (first - best)


def test_remaining_nn_layers():
    from torsh_b200 import nn
    torch.manual_seed(0)
    att = nn.LocationBasedAttention(8, 6, 16)
    out, align = att(torch.randn(2, 8), torch.randn(2, 10, 6), torch.randn(2, 10, 5))
    assert out.shape == (2, 5) and torch.allclose(align.sum(-1), torch.ones(2), atol=1e-6)
    xm, ym = nn.Mixup(0.2, 5)(torch.randn(4, 3, 8, 8), torch.randint(0, 5, (4,)))
    assert xm.shape == (4, 3, 8, 8) and torch.allclose(ym.sum(-1), torch.ones(4), atol=1e-6)
    xc, yc = nn.CutMix(1.0, 5)(torch.randn(4, 3, 8, 8), torch.randint(0, 5, (4,)))
    assert torch.allclose(yc.sum(-1), torch.ones(4), atol=1e-6)
    x = torch.randn(1, 5, 2, 8)
    pi = nn.PositionInterpolation(8, 16, 64)
    assert torch.allclose(pi(x).norm(), x.norm(), atol=1e-5)                   # rotations keep the norm
    full = nn.PositionInterpolation(8, 16, 16)
    assert torch.allclose(pi(x, offset=0)[:, 4], full(x[:, 4:5], offset=1)[:, 0], atol=1e-5)   # position 4 / 4 = 1
    ws = nn.WeightStandardization(torch.nn.Conv2d(3, 4, 3))
    assert ws(torch.randn(1, 3, 8, 8)).shape == (1, 4, 6, 6)
    sn = nn.SpectralNorm(torch.nn.Linear(4, 4))
    for _ in range(30):
        sn(torch.randn(2, 4))
    assert abs(float(torch.linalg.matrix_norm(sn.weight.detach(), 2)) - 1.0) < 0.05
    wn = nn.WeightNorm(torch.nn.Linear(4, 3))
    assert wn(torch.randn(2, 4)).shape == (2, 3)
    assert nn.LazyLinear(3)(torch.randn(2, 7)).shape == (2, 3)


def test_amp_context_policy_and_saturation():
    from torsh_b200.optim.mixed_precision import AmpContext, GradientScaler, GradScaler, MixedPrecisionConfig
    assert GradientScaler is GradScaler
    cfg = MixedPrecisionConfig()
    amp = AmpContext(cfg)
    assert amp.dtype_for("matmul") == cfg.dtype and amp.dtype_for("softmax", cfg.dtype) == torch.float32
    assert amp.dtype_for("relu", cfg.dtype) == cfg.dtype and amp.dtype_for("matmul", torch.int64) == torch.int64
    a, b = amp.cast("matmul", torch.ones(2, 2), torch.ones(2, 2))
    assert a.dtype == cfg.dtype and b.dtype == cfg.dtype and amp.stats["casts"] == 2
    half = AmpContext(cfg, overrides={"matmul": torch.float16})
    big = half.cast("matmul", torch.tensor([1e6, -1e6, 1.0]))
    assert big.dtype == torch.float16 and torch.isfinite(big).all() and half.stats["saturated"] == 2


def test_arrow_parquet_roundtrip_and_gated_formats(tmp_path):
    from torsh_b200.core.error import TorshError
    from torsh_b200.serialize import data_science as ds
    ts = {"w": torch.randn(3, 4), "ids": torch.arange(6).reshape(2, 3), "h": torch.randn(5).to(torch.bfloat16)}
    for save, load, ext in ((ds.save_parquet, ds.load_parquet, "parquet"), (ds.save_arrow, ds.load_arrow, "arrow")):
        p = str(tmp_path / f"t.{ext}")
        save(ts, p)
        back = load(p)
        assert all(back[k].dtype == ts[k].dtype and back[k].shape == ts[k].shape and torch.equal(back[k], ts[k]) for k in ts)
    try:
        import h5py  # noqa: F401
    except ImportError:
        with pytest.raises(TorshError):
            ds.save_hdf5(ts, str(tmp_path / "t.h5"))


def test_tensor_runtime_helpers():
    import gc
    from torsh_b200 import tensor_utils as tu
    pool = tu.GlobalMemoryPool(max_per_key=1)
    a = pool.acquire((3, 5))
    ptr = a.tensor.data_ptr()
    assert a.tensor.shape == (3, 5)
    a.release()
    with pool.acquire((4, 4)) as t:                       # 15 and 16 elements share the 16-element class
        assert t.data_ptr() == ptr and t.shape == (4, 4)
    assert pool.stats["hits"] == 1 and pool.stats["misses"] == 1
    cache = tu.LockFreeCache(capacity=2)
    cache.put("a", 1); cache.put("b", 2); cache.put("c", 3)
    assert cache.get("a") is None and cache.get("c") == 3 and len(cache) == 2 and cache.get_or_insert("d", lambda: 4) == 4
    calls = []
    ab = tu.AutoBatcher(lambda b: (calls.append(b.shape[0]), b * 2)[1], max_batch=4, max_wait_s=0.05)
    futs = [ab.submit(torch.full((2,), float(i))) for i in range(6)]
    outs = [f.result(5) for f in futs]
    ab.shutdown()
    assert all(torch.equal(o, torch.full((2,), 2.0 * i)) for i, o in enumerate(outs)) and sum(calls) == 6 and max(calls) <= 4
    ao = tu.AsyncOps(2)
    assert [int(x) for x in ao.map(lambda v: v.sum(), [torch.ones(3), torch.ones(5)])] == [3, 5]
    ao.shutdown()
    log = tu.OperationLog()
    with log.record("matmul", torch.ones(2, 3), torch.ones(3, 4), flops=48):
        torch.ones(2, 3) @ torch.ones(3, 4)
    assert log.summary()["matmul"]["count"] == 1 and log.records[0].shapes == [(2, 3), (3, 4)]
    tr = tu.TensorTracker()
    keep = tr.track(torch.zeros(10), "act")
    tmp = tr.track(torch.zeros(100), "act")
    assert tr.live_bytes("act") == 440
    del tmp
    gc.collect()
    assert tr.live_bytes("act") == 40 and (tr.created, tr.freed) == (2, 1) and keep is not None


def test_distributed_grad_accumulator_and_sync_scheduler():
    import threading
    from torsh_b200.autograd.distributed import DistributedGradAccumulator, GradientSyncScheduler, NetworkHealth
    from torsh_b200.parallel.compression import TopK
    torch.manual_seed(0)
    lin, head = torch.nn.Linear(4, 4), torch.nn.Linear(4, 2)
    acc = DistributedGradAccumulator()
    acc.add_param_group("body", lin.parameters(), priority=5)
    acc.add_param_group("head", head.parameters(), priority=1, compressor=TopK(1.0))
    xs = [torch.randn(3, 4) for _ in range(2)]
    for x in xs:
        head(lin(x)).sum().backward()
        acc.accumulate()
    assert lin.weight.grad is None
    acc.step()
    ref_l, ref_h = torch.nn.Linear(4, 4), torch.nn.Linear(4, 2)
    ref_l.load_state_dict(lin.state_dict()); ref_h.load_state_dict(head.state_dict())
    (sum(ref_h(ref_l(x)).sum() for x in xs) / 2).backward()
    assert torch.allclose(lin.weight.grad, ref_l.weight.grad, atol=1e-6) and torch.allclose(head.bias.grad, ref_h.bias.grad, atol=1e-6)
    assert acc.stats["syncs"] == 2 and acc.stats["compressed"] == 2
    health = NetworkHealth()
    sched = GradientSyncScheduler(max_concurrent=1, health=health)
    gate = threading.Event()
    first = sched.schedule("gate", gate.wait, priority=0)
    hs = [sched.schedule(n, lambda: None, nbytes=1000, priority=p) for n, p in (("low", 9), ("high", 1), ("mid", 5))]
    bad = sched.schedule("bad", lambda: 1 / 0, priority=20)
    gate.set()
    assert first.wait(5) and all(h.wait(5) for h in hs)
    with pytest.raises(ZeroDivisionError):
        bad.wait(5)
    sched.shutdown()
    assert sched.order == ["gate", "high", "mid", "low", "bad"] and health.failures == 1 and health.successes == 4
    slow = NetworkHealth()
    slow.record(10_000_000, 1.0)
    assert slow.should_compress(min_gbs=1.0) and not NetworkHealth().should_compress()


def test_vision_zoo_builds_and_backpropagates():
    from torsh_b200.models import create_model, list_models, vision_zoo as V
    torch.manual_seed(0)
    x = torch.randn(2, 3, 64, 64)
    small = {"alexnet": V.AlexNet(10), "vgg": V.VGG(11, True, 10, width=0.125, hidden=64), "densenet": V.DenseNet((2, 2), 8, 16, 10),
             "mobilenet": V.MobileNetV2(10, 0.25), "efficientnet": V.EfficientNet(10, 0.25, 0.5),
             "convnext": V.ConvNeXt((1, 1, 1, 1), (8, 16, 32, 64), 10),
             "swin": V.SwinTransformer(16, (2, 2), (2, 4), window=4, patch=4, num_classes=10)}
    for name, m in small.items():
        y = m(x)
        assert y.shape == (2, 10), name
        y.sum().backward()
        assert all(p.grad is not None for p in m.parameters() if p.requires_grad), name
    n = lambda m: sum(p.numel() for p in m.parameters())
    assert abs(n(create_model("swin_t")) - 28.29e6) < 0.05e6 and abs(n(create_model("convnext_tiny")) - 28.59e6) < 0.05e6
    assert abs(n(create_model("densenet121")) - 7.98e6) < 0.02e6 and abs(n(create_model("mobilenet_v2")) - 3.50e6) < 0.02e6
    assert {"alexnet", "vgg16_bn", "efficientnet_b0"} <= set(list_models())


def test_sentencepiece_tokenizer_roundtrip():
    pytest.importorskip("sentencepiece")
    from torsh_b200.text import SentencePieceTokenizer
    corpus = ["the quick brown fox jumps over the lazy dog"] * 50 + ["pack my box with five dozen liquor jugs"] * 50
    tok = SentencePieceTokenizer.train(corpus, vocab_size=60)
    ids = tok.encode("the quick brown dog", add_eos=True)
    assert tok.decode(ids) == "the quick brown dog" and max(ids) < tok.vocab_size and "".join(tok.tokenize("lazy dog")).replace("▁", " ").strip() == "lazy dog"


def test_package_ed25519_signature_and_aes_gcm(tmp_path):
    pytest.importorskip("cryptography")
    from torsh_b200 import hub
    sk, pk = hub.generate_signing_key()
    other_sk, other_pk = hub.generate_signing_key()
    pkg = hub.Package("demo", "1.2.3")
    pkg.add_bytes("weights.bin", b"\x00\x01" * 100)
    pkg.add_source("demo.mod", "VALUE = 41 + 1\n")
    enc = bytes(range(32))
    path = str(tmp_path / "demo.tpkg")
    pkg.save(path, signing_key=sk, encryption_key=enc)
    back = hub.Package.load(path, public_key=pk, encryption_key=enc)
    assert back.files["weights.bin"] == b"\x00\x01" * 100 and back.import_module("demo.mod").VALUE == 42
    with pytest.raises(PermissionError):
        hub.Package.load(path, public_key=other_pk, encryption_key=enc)
    with pytest.raises(PermissionError):
        hub.Package.load(path, public_key=pk)                                  # encrypted, no key given
    with pytest.raises(PermissionError):
        hub.Package.load(path, public_key=pk, encryption_key=bytes(32))        # wrong key
    import zipfile
    assert b"VALUE" not in zipfile.ZipFile(path).read("code/demo/mod.py")      # contents are sealed


def test_gradient_free_optimizers_minimise_a_quadratic():
    from torsh_b200.optim import BayesianOptimizer, EvolutionStrategy, NelderMead, RandomSearch
    target = torch.tensor([1.0, -2.0, 0.5])
    f = lambda x: float(((x - target) ** 2).sum())
    nm = NelderMead(torch.zeros(3))
    for _ in range(200):
        v = nm.step(f)
    assert v < 1e-6 and torch.allclose(nm.best_x, target, atol=1e-2)
    es = EvolutionStrategy(torch.zeros(3), sigma=1.0, seed=1)
    for _ in range(120):
        v = es.step(f)
    assert v < 1e-3
    rs = RandomSearch(torch.zeros(3), sigma=0.3, seed=2)
    for _ in range(60):
        v = rs.step(f)
    assert v < 0.1
    bo = BayesianOptimizer([(-3, 3)] * 2, seed=3)
    g = lambda x: float(((x - torch.tensor([1.0, -1.0])) ** 2).sum())
    for _ in range(40):
        v = bo.step(g)
    assert v < 0.15 and bo.best_x.shape == (2,)


def test_vision_extras():
    from torsh_b200.vision import extras as X
    torch.manual_seed(0)
    conv = torch.nn.Conv2d(3, 8, 3, padding=1)
    model = torch.nn.Sequential(conv, torch.nn.ReLU(), torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(8, 5))
    x = torch.randn(2, 3, 16, 16)
    assert X.saliency(model, x).shape == (2, 16, 16)
    cam = X.GradCAM(model, conv)
    m = cam(x)
    cam.close()
    assert m.shape == (2, 16, 16) and float(m.min()) >= 0 and float(m.max()) <= 1.0 + 1e-6
    tgt = torch.tensor([1, 3])
    ig = X.integrated_gradients(model, x, tgt, steps=64)
    diff = model(x).gather(1, tgt[:, None])[:, 0] - model(torch.zeros_like(x)).gather(1, tgt[:, None])[:, 0]
    assert torch.allclose(ig.flatten(1).sum(1), diff.detach(), atol=2e-2)                     # completeness
    video = torch.arange(12.0).view(12, 1, 1, 1).expand(12, 3, 4, 4)
    assert X.sample_frames(video, 4)[:, 0, 0, 0].tolist() == [1.0, 4.0, 7.0, 10.0] and float(X.frame_difference(video).mean()) == 1.0
    assert X.Conv3dClassifier(7, 4)(torch.randn(2, 3, 4, 16, 16)).shape == (2, 7)
    lo = torch.rand(1, 3, 8, 8)
    assert X.SRCNN(2)(lo).shape == (1, 3, 16, 16) and X.ESPCN(3)(lo).shape == (1, 3, 24, 24) and X.psnr(lo, lo) == float("inf")
    feats = torch.nn.Sequential(torch.nn.Conv2d(3, 4, 3, padding=1), torch.nn.ReLU(), torch.nn.Conv2d(4, 4, 3, padding=1), torch.nn.ReLU())
    crit = X.StyleTransferLoss(feats)
    img = torch.rand(1, 3, 8, 8, requires_grad=True)
    total, cl, sl = crit(img, torch.rand(1, 3, 8, 8), torch.rand(1, 3, 8, 8))
    total.backward()
    assert img.grad is not None and float(cl) > 0 and float(sl) > 0
    same, c0, s0 = crit(img.detach(), img.detach(), img.detach())
    assert float(same) < 1e-10


def test_dsr_and_rle_sparse_formats():
    from torsh_b200.sparse import DsrTensor, RleTensor
    d = torch.tensor([[0.0, 2.0, 0.0], [0.0, 0.0, 0.0], [1.0, 0.0, 3.0]])
    dsr = DsrTensor.from_dense(d)
    assert dsr.nnz() == 3 and dsr.get(2, 2) == 3.0 and torch.equal(dsr.to_dense(), d)
    dsr.set(1, 1, 5.0); dsr.set(0, 1, 0.0)
    assert dsr.nnz() == 3 and dsr.get(1, 1) == 5.0 and torch.equal(dsr.to_csr().to_dense(), dsr.to_dense())
    assert torch.allclose(dsr.matmul(torch.ones(3)), dsr.to_dense().sum(1))
    mask = torch.zeros(8, 8, dtype=torch.int64)
    mask[2:5, :] = 7
    rle = RleTensor.from_dense(mask)
    assert rle.values.tolist() == [0, 7, 0] and rle.lengths.tolist() == [16, 24, 24] and torch.equal(rle.to_dense(), mask)
    assert rle.compression_ratio() > 10


def test_weight_gradient_plan_picks_stream_k_only_for_badly_filled_waves():
    from torsh_b200.ops.linear import _wgrad_plan
    # (output rows, output cols, K) -> (tile width, split): -1 = stream-K
    assert _wgrad_plan(4096, 1024, 8192) == (256, -1)        # 128 tiles x 2 splits fill 256 of 296 slots
    assert _wgrad_plan(1024, 1024, 8192) == (256, -1)        # 32 tiles x 4 splits fill 128 of 148
    assert _wgrad_plan(3072, 1024, 8192) == (256, 3)         # 96 x 3 = 288 of 296: uniform splits are fine
    assert _wgrad_plan(50304, 1024, 8192) == (256, 1)        # many tiles per CTA: keep round-robin tiles (L2 reuse)
    assert _wgrad_plan(64, 64, 256)[1] == 1                  # short K: no split at all


def test_tabular_and_audio_datasets(tmp_path):
    from torsh_b200.data import AudioDataset, TabularDataset
    cols = {"age": [20, 30, 40, 50], "income": [1.0, 2.0, 3.0, 4.0], "city": ["a", "b", "a", "c"], "y": [0, 1, 0, 1]}
    ds = TabularDataset(cols, "y", categorical=["city"])
    num, cat, y = ds[2]
    assert len(ds) == 4 and num.shape == (2,) and cat.tolist() == [0] and int(y) == 0 and ds.cardinalities() == [3]
    assert torch.allclose(ds.num.mean(0), torch.zeros(2), atol=1e-6) and torch.allclose(ds.num.std(0, unbiased=False), torch.ones(2), atol=1e-5)
    p = tmp_path / "t.csv"
    p.write_text("age,city,y\n20,a,0\n30,b,1\n")
    assert len(TabularDataset.from_csv(str(p), "y", categorical=["city"])) == 2
    import pyarrow as pa, pyarrow.parquet as pq
    pq.write_table(pa.table(cols), str(tmp_path / "t.parquet"))
    assert TabularDataset.from_parquet(str(tmp_path / "t.parquet"), "y", categorical=["city"]).cardinalities() == [3]
    au = AudioDataset.synthetic(8, classes=3, num_samples=1024, n_fft=256)
    spec, label = au[0]
    assert spec.shape[0] == 129 and 0 <= label < 3
    peak = spec.mean(1).argmax().item() * 8000 / 256
    assert abs(peak - 220.0 * (label + 1)) < 40                               # the spectrogram peaks at the class's tone
    raw = AudioDataset([torch.ones(10)], [1], num_samples=16)
    assert raw[0][0].shape == (16,) and float(raw[0][0][12]) == 0.0


def test_hub_hf_gpt2_import_and_access_control(tmp_path, monkeypatch):
    transformers = pytest.importorskip("transformers")
    from torsh_b200 import hub, models
    torch.manual_seed(0)
    hf = transformers.GPT2LMHeadModel(transformers.GPT2Config(vocab_size=1024, n_positions=128, n_embd=256, n_layer=4, n_head=4,
                                                              resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)).eval()
    ours = models.create_model("gpt2-tiny").eval()
    unused = hub.import_hf_gpt2(hf.state_dict(), ours)
    assert all(("attn.bias" in k or "masked_bias" in k or k == "lm_head.weight") for k in unused)
    ids = torch.randint(0, 1024, (2, 16))
    with torch.no_grad():
        ref = hf(ids).logits
        got = ours(ids)
    got = got[..., :1024] if got.shape[-1] > 1024 else got
    assert torch.allclose(got.float(), ref, atol=2e-4), float((got.float() - ref).abs().max())
    acl = hub.AccessControl(tmp_path / "acl.json")
    acl.grant("alice-token", "write", prefixes=("team-a/",))
    acl.grant("root-token", "admin")
    assert acl.allowed("read", "team-a/gpt2", "alice-token") and acl.allowed("write", "team-a/gpt2", "alice-token")
    assert not acl.allowed("write", "team-b/gpt2", "alice-token") and not acl.allowed("admin", "team-a/x", "alice-token")
    monkeypatch.setenv("TORSH_HUB_TOKEN", "root-token")
    assert hub.AccessControl(tmp_path / "acl.json").allowed("admin", "anything")
    acl.revoke("alice-token")
    with pytest.raises(PermissionError):
        acl.require("read", "team-a/gpt2", "alice-token")


def test_hub_hf_llama_import_matches_transformers_logits():
    transformers = pytest.importorskip("transformers")
    from torsh_b200 import hub
    from torsh_b200.models.llama import LlamaConfig, LlamaModel
    torch.manual_seed(0)
    hc = transformers.LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=64, rms_norm_eps=1e-6,
                                  rope_theta=10000.0, attention_bias=False, tie_word_embeddings=False)
    hf = transformers.LlamaForCausalLM(hc).eval()
    ours = LlamaModel(LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=128, num_layers=2, num_heads=4, max_seq_len=64)).eval()
    assert hub.import_hf_llama(hf.state_dict(), ours) == []
    ids = torch.randint(0, 320, (2, 16))
    with torch.no_grad():
        assert torch.allclose(ours(ids).float(), hf(ids).logits, atol=1e-5)
    gqa = transformers.LlamaForCausalLM(transformers.LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                                                                 num_attention_heads=4, num_key_value_heads=2)).state_dict()
    with pytest.raises(ValueError):
        hub.import_hf_llama(gqa, LlamaModel(LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=128, num_layers=1, num_heads=4, max_seq_len=64)))


def test_hub_hf_bert_import_matches_transformers_hidden_states():
    transformers = pytest.importorskip("transformers")
    from torsh_b200 import hub
    from torsh_b200.models.transformer_zoo import BertConfig, BertModel
    torch.manual_seed(0)
    hc = transformers.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=64,
                                 max_position_embeddings=64, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    hf = transformers.BertModel(hc).eval()
    ours = BertModel(BertConfig(vocab_size=100, hidden_size=32, num_layers=2, num_heads=2, intermediate_size=64,
                                max_position_embeddings=64, dropout=0.0)).eval()
    assert hub.import_hf_bert(hf.state_dict(), ours) == []
    ids = torch.randint(1, 100, (2, 10))
    with torch.no_grad():
        ref, (hidden, pooled) = hf(ids), ours(ids)
    assert torch.allclose(hidden, ref.last_hidden_state, atol=1e-5) and torch.allclose(pooled, ref.pooler_output, atol=1e-5)


def test_hub_hf_vit_import_matches_transformers_logits():
    transformers = pytest.importorskip("transformers")
    from torsh_b200 import hub
    from torsh_b200.models.transformer_zoo import ViTConfig, VisionTransformer
    torch.manual_seed(0)
    hc = transformers.ViTConfig(image_size=32, patch_size=8, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                                intermediate_size=64, num_labels=5, layer_norm_eps=1e-6, hidden_dropout_prob=0.0,
                                attention_probs_dropout_prob=0.0)
    hf = transformers.ViTForImageClassification(hc).eval()
    ours = VisionTransformer(ViTConfig(image_size=32, patch_size=8, hidden_size=32, num_layers=2, num_heads=2, intermediate_size=64,
                                       num_classes=5, layer_norm_eps=1e-6)).eval()
    assert hub.import_hf_vit(hf.state_dict(), ours) == []
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        assert torch.allclose(ours(x), hf(x).logits, atol=1e-5)


def test_resnet_state_dict_is_interchangeable_with_torchvision():
    tv = pytest.importorskip("torchvision")
    from torsh_b200.models import create_model
    torch.manual_seed(0)
    for name in ("resnet18", "resnet50"):
        ref = getattr(tv.models, name)().eval()
        ours = create_model(name).eval()
        assert list(ours.state_dict()) == list(ref.state_dict())
        ours.load_state_dict(ref.state_dict())
        x = torch.randn(2, 3, 64, 64)
        with torch.no_grad():
            assert torch.allclose(ours(x), ref(x), atol=1e-4), name


def test_vision_zoo_reproduces_torchvision_logits():
    tv = pytest.importorskip("torchvision")
    from torsh_b200.models import create_model
    torch.manual_seed(0)
    x = torch.randn(1, 3, 96, 96)
    for name, by_key in (("alexnet", True), ("vgg16_bn", True), ("densenet121", False), ("mobilenet_v2", False),
                         ("efficientnet_b0", False), ("convnext_tiny", False)):
        ref = getattr(tv.models, name)().eval()
        ours = create_model(name).eval()
        if by_key:
            ours.load_state_dict(ref.state_dict())
        else:                               # same tensors in the same order under different names
            mine = ours.state_dict()
            assert [v.numel() for v in mine.values()] == [v.numel() for v in ref.state_dict().values()], name
            # (ConvNeXt's layer scale is [C] here and [C, 1, 1] there; everything else has the same shape)
            ours.load_state_dict({k: v.reshape(mine[k].shape) for k, v in zip(mine.keys(), ref.state_dict().values())})
        with torch.no_grad():
            want = ref(x)
            assert float(want.abs().max()) > 0 and torch.allclose(ours(x), want, atol=1e-4), name


def test_torsh_checkpoint_golden_bytes():
    """The ``.torsh`` payload, built by hand from the bincode "standard" rules (varint lengths, option tag bytes,
    little-endian floats) for the reference's ``ModelCheckpoint`` field order and types
    (``crates/torsh-nn/src/checkpoint.rs:24-113``)."""
    import gzip
    import struct
    from torsh_b200.serialize import checkpoint as ck
    doc = {"state_dict": {"w": [1.0, -2.0]}, "parameter_shapes": {"w": [2, 1]},
           "metadata": {"model_name": "m", "model_version": "v1", "torsh_version": "0.1.3", "timestamp": "2026-01-01T00:00:00+00:00",
                        "epoch": 3, "global_step": None, "best_metric": 0.5, "custom": {"k": "v"}},
           "optimizer_state": {"optimizer_type": "SGD", "learning_rate": 0.1, "momentum_states": {"w": [0.25, 0.5]},
                               "velocity_states": {}, "step_counts": {"w": 300}, "custom_state": {"c": [1.5]}},
           "training_stats": {"train_losses": [1.0], "val_losses": [], "train_accuracies": [], "val_accuracies": [],
                              "learning_rates": [0.1], "epoch_durations": [], "custom_metrics": {"f1": [0.75]}}}
    f32 = lambda *v: struct.pack("<%df" % len(v), *v)
    f64 = lambda *v: struct.pack("<%dd" % len(v), *v)
    s = lambda t: bytes([len(t)]) + t.encode()
    exp = b"".join([
        b"\x01", s("w"), b"\x02", f32(1.0, -2.0),                      # state_dict
        b"\x01", s("w"), b"\x02\x02\x01",                              # parameter_shapes
        s("m"), s("v1"), s("0.1.3"), s("2026-01-01T00:00:00+00:00"),   # metadata strings (timestamp is a String)
        b"\x01\x03", b"\x00", b"\x01", f64(0.5),                       # epoch Some(3), global_step None, best_metric Some
        b"\x01", s("k"), s("v"),                                       # custom
        b"\x01", s("SGD"), f64(0.1),                                   # optimizer_state Some
        b"\x01", s("w"), b"\x02", f32(0.25, 0.5), b"\x00",             # momentum, velocity (empty)
        b"\x01", s("w"), b"\xfb", struct.pack("<H", 300),              # step_counts: 300 needs the u16 varint form
        b"\x01", s("c"), b"\x01", f32(1.5),                            # custom_state: Vec<f32> values
        b"\x01", b"\x01", f64(1.0), b"\x00\x00\x00", b"\x01", f64(0.1), b"\x00",   # training_stats Some: six Vec<f64>
        b"\x01", s("f1"), b"\x01", f64(0.75)])                         # custom_metrics
    blob = ck.encode_checkpoint(doc)
    assert gzip.decompress(blob) == exp
    back = ck.decode_checkpoint(blob)
    assert back["metadata"]["epoch"] == 3 and back["metadata"]["global_step"] is None
    assert back["optimizer_state"]["step_counts"] == {"w": 300} and back["training_stats"]["custom_metrics"] == {"f1": [0.75]}
    assert ck.CheckpointManager.__init__.__defaults__[0] == "model"


def test_flat_adamw_resume_continues_the_loss_curve(tmp_path):
    """Save master weights, moments and step count of the flat fused AdamW (its CPU path), restore into a fresh model and
    optimizer, and get the same losses as the uninterrupted run."""
    from torsh_b200.optim.flat import FlatAdamW, FlatParameters
    from torsh_b200.serialize import checkpoint as ck

    def make():
        torch.manual_seed(3)
        m = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 1))
        return m, FlatAdamW(FlatParameters(m.parameters(), lowp_dtype=torch.float32), lr=1e-2)

    x, y = torch.randn(32, 8, generator=torch.Generator().manual_seed(1)), torch.randn(32, 1, generator=torch.Generator().manual_seed(2))

    def run(m, o, n):
        out = []
        for _ in range(n):
            loss = (m(x) - y).pow(2).mean()
            loss.backward()
            o.step()
            out.append(loss.item())
        return out

    m, o = make()
    full = run(m, o, 8)
    m1, o1 = make()
    first = run(m1, o1, 4)
    mgr = ck.CheckpointManager(tmp_path)
    mgr.save(m1, o1, global_step=4)
    m2, o2 = make()
    run(m2, o2, 1)                      # a different state that the restore must fully replace
    ck.restore_into(mgr.load(), m2, o2)
    assert o2.step_count == 4
    rest = run(m2, o2, 4)
    assert first == full[:4] and all(abs(a - b) < 1e-6 for a, b in zip(rest, full[4:]))
    sd = o1.state_dict()
    m3, o3 = make()
    o3.load_state_dict(sd)
    assert torch.equal(o3.flat.master, o1.flat.master) and torch.equal(o3.flat.lowp, o1.flat.lowp) and o3.step_count == 4


def test_trainer_raises_when_the_device_status_word_is_set():
    """A failed cross-rank wait leaves a code in the device status word; the step's loss handle must raise instead of
    letting training continue (here with host stand-ins for the pinned copies)."""
    from torsh_b200 import _native as nv
    from torsh_b200.engine import PendingLoss, _raise_on_status
    ok = PendingLoss(torch.tensor(1.5), None, torch.zeros(4, dtype=torch.int32), None)
    assert ok.value() == 1.5
    bad = PendingLoss(torch.tensor(1.5), None, torch.tensor([105, 0, 0, 0], dtype=torch.int32), torch.ones(4, dtype=torch.int32))
    with pytest.raises(nv.KernelTimeout, match="peer"):
        bad.value()
    with pytest.raises(nv.KernelTimeout):
        _raise_on_status(101, None)


def test_clip_whisper_wav2vec2_reproduce_transformers_outputs():
    """Random-init Hugging Face models of small size, weights imported, same inputs: the outputs must agree."""
    transformers = pytest.importorskip("transformers")
    from torsh_b200 import hub
    from torsh_b200.models import audio, multimodal
    torch.manual_seed(0)
    # ---- CLIP
    hc = transformers.CLIPConfig(
        text_config=dict(vocab_size=300, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                         max_position_embeddings=16, eos_token_id=299, projection_dim=32),
        vision_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=32,
                           patch_size=8, projection_dim=32), projection_dim=32)
    hf = transformers.CLIPModel(hc).eval()
    ours = multimodal.CLIPModel(multimodal.CLIPConfig.tiny()).eval()
    assert hub.import_hf_clip(hf.state_dict(), ours) == []
    ids = torch.randint(0, 298, (3, 16)); ids[:, 9] = 299
    px = torch.randn(3, 3, 32, 32)
    with torch.no_grad():
        ref = hf(input_ids=ids, pixel_values=px)
        li, lt = ours(ids, px)
    assert torch.allclose(li, ref.logits_per_image, atol=2e-4) and torch.allclose(lt, ref.logits_per_text, atol=2e-4)
    assert torch.allclose(ours.encode_image(px), ref.image_embeds / ref.image_embeds.norm(dim=-1, keepdim=True), atol=1e-5)
    # ---- Whisper encoder
    wc = transformers.WhisperConfig(vocab_size=200, num_mel_bins=16, encoder_layers=2, encoder_attention_heads=4, decoder_layers=1,
                                    decoder_attention_heads=4, decoder_ffn_dim=128, encoder_ffn_dim=128, d_model=64,
                                    max_source_positions=50, max_target_positions=32, pad_token_id=0, bos_token_id=1, eos_token_id=2,
                                    decoder_start_token_id=1)
    hw = transformers.WhisperModel(wc).eval()
    enc = audio.WhisperEncoder(audio.WhisperConfig.tiny()).eval()
    assert hub.import_hf_whisper_encoder(hw.state_dict(), enc) == []
    mel = torch.randn(2, 16, 100)
    with torch.no_grad():
        assert torch.allclose(enc(mel), hw.encoder(mel).last_hidden_state, atol=2e-4)
    assert torch.allclose(audio.sinusoids(50, 64), hw.encoder.embed_positions.weight, atol=1e-6)
    # ---- Wav2Vec2 (base layout: group norm after the first convolution, post-norm encoder)
    vc = transformers.Wav2Vec2Config(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, intermediate_size=128,
                                     conv_dim=(32, 32, 32), conv_kernel=(10, 3, 2), conv_stride=(5, 2, 2), num_conv_pos_embeddings=16,
                                     num_conv_pos_embedding_groups=4, hidden_dropout=0.0, attention_dropout=0.0, feat_proj_dropout=0.0,
                                     layerdrop=0.0, mask_time_prob=0.0, feat_extract_norm="group", do_stable_layer_norm=False)
    hv = transformers.Wav2Vec2Model(vc).eval()
    w2v = audio.Wav2Vec2Model(audio.Wav2Vec2Config.tiny()).eval()
    left = hub.import_hf_wav2vec2(hv.state_dict(), w2v)
    assert all(k.startswith(("masked_spec_embed", "quantizer", "project_")) for k in left)
    wav = torch.randn(2, 4000)
    with torch.no_grad():
        assert torch.allclose(w2v(wav), hv(wav).last_hidden_state, atol=3e-4)
    assert w2v.frames(4000) == w2v(wav).shape[1]


def test_lora_adapters_prefix_and_freezing():
    from torsh_b200.models import fine_tuning as ft
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 8))
    x = torch.randn(5, 16)
    y0 = net(x)
    wrapped = ft.apply_lora(net, target=r"^(0|2)$", rank=4, alpha=8.0)
    assert wrapped == ["0", "2"] and torch.allclose(net(x), y0)                 # B starts at zero: identical function
    s = ft.trainable_summary(net)
    assert s["trainable"] == 4 * 16 + 32 * 4 + 4 * 32 + 8 * 4 and s["fraction"] < 0.5
    opt = torch.optim.SGD([p for p in net.parameters() if p.requires_grad], lr=0.5)
    for _ in range(3):
        loss = (net(x) - 1).pow(2).mean(); opt.zero_grad(); loss.backward(); opt.step()
    assert net[0].base.weight.grad is None and not torch.allclose(net(x), y0)
    y1 = net(x)
    assert ft.merge_lora(net) == 2 and torch.allclose(net(x), y1, atol=1e-5)    # folded into the base weights
    net[0].unmerge()
    assert torch.allclose(net(x), y1, atol=1e-5) and set(ft.lora_state_dict(net)) == {"0.lora_A", "0.lora_B", "2.lora_A", "2.lora_B"}
    # extract: the rank-r factors of a rank-r difference reproduce it
    base = torch.randn(12, 10)
    delta = torch.randn(12, 3) @ torch.randn(3, 10)
    A, B = ft.extract_lora(base, base + delta, rank=3, alpha=6.0)
    assert torch.allclose((6.0 / 3) * B @ A, delta, atol=1e-4)
    # AdaLoRA: pruning singular values removes their contribution
    ada = ft.AdaLoRALinear(torch.nn.Linear(6, 6), rank=4)
    with torch.no_grad():
        ada.lora_E.copy_(torch.tensor([3.0, 0.1, -2.0, 0.01]))
    ada.prune_to(2)
    assert ada.rank_mask.tolist() == [1, 0, 1, 0] and ada.orthogonality_penalty() >= 0
    # adapters start as the identity; prefix encoder shapes
    enc = torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Linear(8, 8))
    z = torch.randn(3, 8)
    z0 = enc(z)
    assert ft.insert_adapters(enc, r"[01]", hidden=8, reduction_factor=2) == ["0", "1"] and torch.allclose(enc(z), z0)
    assert ft.PrefixEncoder(3, 5, 8, reparam_hidden=16)().shape == (3, 5, 8) and ft.PrefixEncoder(3, 5, 8)().shape == (3, 5, 8)
    # layer-wise rates, progressive unfreezing, EWC
    from torsh_b200.models import BertModel, BertConfig
    bert = BertModel(BertConfig.tiny())
    groups = ft.layerwise_lr_groups(bert, 1e-3, 0.5)
    lrs = sorted(g["lr"] for g in groups)
    assert lrs == [1e-3 * 0.25, 1e-3 * 0.5, 1e-3] and sum(len(g["params"]) for g in groups) == len(list(bert.parameters()))
    un = ft.ProgressiveUnfreezer(bert, every=2)
    assert not bert.layers[1].fc1.weight.requires_grad and [un.step() for _ in range(4)] == [None, 1, None, 0]
    assert bert.layers[0].fc1.weight.requires_grad
    assert ft.freeze_parameters(bert, [r"embeddings"], keep=[r"position"]) == 2
    lin = torch.nn.Linear(4, 1)
    ewc = ft.EWCPenalty(lin, lam=2.0)
    lin(torch.ones(1, 4)).sum().backward(); ewc.accumulate()
    with torch.no_grad():
        lin.weight.add_(1.0)
    assert ewc.penalty().item() == pytest.approx(0.5 * 2.0 * 4 * 1.0)            # Fisher = 1 on each weight, moved by 1


def test_model_merging_sharding_surgery_distillation_pruning():
    from torsh_b200.models import model_utils as mu
    mk = lambda v: {"w": torch.full((2, 2), float(v)), "n": torch.tensor(3)}
    M = mu.ModelMerger
    assert M().merge_models([mk(1), mk(3)])["w"][0, 0] == 2 and M().merge_models([mk(1), mk(3)])["n"] == 3
    assert M(mu.MergeStrategy.WEIGHTED_AVERAGE, weights=[0.25, 0.75]).merge_models([mk(0), mk(4)])["w"][0, 0] == 3
    assert M(mu.MergeStrategy.EMA, alpha=0.5).merge_models([mk(0), mk(4), mk(8)])["w"][0, 0] == 5
    assert M(mu.MergeStrategy.MAX_MAGNITUDE).merge_models([mk(1), mk(-3)])["w"][0, 0] == -3
    assert M(mu.MergeStrategy.TASK_ARITHMETIC, base=mk(1), scaling=0.5).merge_models([mk(3), mk(5)])["w"][0, 0] == 1 + 0.5 * (2 + 4)
    with pytest.raises(ValueError):
        M(mu.MergeStrategy.WEIGHTED_AVERAGE, weights=[0.5, 0.6])
    a, b = torch.tensor([1.0, 0.0]), torch.tensor([0.0, 1.0])
    assert torch.allclose(mu.slerp(a, b, 0.5), torch.tensor([0.5 ** 0.5, 0.5 ** 0.5]), atol=1e-6)
    ties = M(mu.MergeStrategy.TIES, base={"w": torch.zeros(4)}, density=0.5).merge_models(
        [{"w": torch.tensor([1.0, -0.1, 2.0, 0.0])}, {"w": torch.tensor([3.0, 0.2, -4.0, 0.1])}])["w"]
    assert ties.tolist() == [2.0, 0.0, -4.0, 0.0]           # small entries trimmed, sign elected by total mass, agreeing entries averaged
    soup = mu.ModelSoup()
    for v in (1, 2, 9):
        soup.add_model(mk(v))
    assert soup.uniform_soup()["w"][0, 0] == 4
    assert soup.greedy_soup(lambda sd: -abs(sd["w"][0, 0].item() - 1.5))["w"][0, 0] == 1.5      # the outlier is left out
    # sharding plans
    net = torch.nn.Sequential(*[torch.nn.Linear(8, 8) for _ in range(4)])
    sh = mu.ModelSharder(mu.ShardingStrategy.PIPELINE, 2)
    parts = sh.shard_model(net)
    assert sorted(parts[0]) == ["0.bias", "0.weight", "1.bias", "1.weight"] and sh.get_stats(parts).balance_ratio() == 1.0
    tp = mu.ModelSharder(mu.ShardingStrategy.TENSOR_PARALLEL, 4).shard_model(net)
    assert tp[0]["0.weight"].shape == (2, 8) and tp[3]["0.bias"].shape == (8,)
    z3 = mu.ModelSharder(mu.ShardingStrategy.ZERO_STAGE3, 3).shard_model(net)
    assert sum(p["0.weight"].numel() for p in z3) == 64
    # surgery
    sg = mu.ModelSurgeon(net)
    sg.replace_layer("1", torch.nn.Linear(8, 8, bias=False), copy_weights=True)
    sg.insert_after("2", torch.nn.ReLU()); sg.remove_layer("3")
    assert isinstance(net[3], torch.nn.Identity) and isinstance(net[2], torch.nn.Sequential) and sg.stats()["operations"] == 3
    donor = torch.nn.Sequential(torch.nn.Linear(8, 8))
    sg.graft("0", donor, "0")
    assert net[0] is donor[0]
    # distillation
    dt = mu.DistillationTrainer(mu.DistillationConfig(mu.DistillationStrategy.MULTI_LEVEL, temperature=2.0, alpha=0.5))
    s, t = torch.randn(4, 5), torch.randn(4, 5)
    out = dt.compute_distillation_loss(s, t, labels=torch.tensor([0, 1, 2, 3]), student_feats={"h": torch.randn(4, 6)},
                                       teacher_feats={"h": torch.randn(4, 6)}, student_attn=[torch.rand(4, 2, 3, 3)], teacher_attn=[torch.rand(4, 2, 3, 3)])
    assert set(out) == {"distillation", "hard", "feature", "attention", "total"} and dt.response_loss(t, t).abs() < 1e-6
    assert dt.relation_loss(s, s) == 0 and mu.compression_ratio(100, 25) == 4
    # pruning
    lin = torch.nn.Sequential(torch.nn.Linear(10, 10))
    st = mu.ModelPruner(mu.PruningConfig(sparsity=0.3)).prune_model(lin)
    assert st["overall_sparsity"] == pytest.approx(0.3) and mu.calculate_sparsity(lin[0].weight) == pytest.approx(0.3)
    lin2 = torch.nn.Sequential(torch.nn.Linear(10, 10))
    pr = mu.ModelPruner(mu.PruningConfig(sparsity=0.5, structured=True))
    pr.prune_model(lin2)
    assert (lin2[0].weight.abs().sum(1) == 0).sum() == 5
    with torch.no_grad():
        lin2[0].weight.add_(1.0)
    pr.apply_masks(lin2)
    assert (lin2[0].weight.abs().sum(1) == 0).sum() == 5
    sched = mu.ModelPruner(mu.PruningConfig(sparsity=0.8, schedule="polynomial", steps=4, power=1.0))
    assert [round(sched.current_sparsity(), 2) for sched.step_count in range(5)] == [0.0, 0.2, 0.4, 0.6, 0.8]
    for method in (mu.PruningMethod.LAMP, mu.PruningMethod.RANDOM):
        l3 = torch.nn.Sequential(torch.nn.Linear(6, 6))
        assert mu.ModelPruner(mu.PruningConfig(sparsity=0.5, method=method)).prune_model(l3)["overall_sparsity"] == pytest.approx(0.5)
    ens = mu.Ensemble([torch.nn.Linear(3, 2), torch.nn.Linear(3, 2)], mode="prob")
    assert torch.allclose(ens(torch.randn(4, 3)).sum(-1), torch.ones(4), atol=1e-6)


def test_int4_int8_and_csr_cpu_paths():
    """The quantised layers and the CSR class give the same answers through their PyTorch fallbacks on a CPU."""
    from torsh_b200 import quantization as Q
    from torsh_b200.sparse import CudaSparseTensor, CooTensor, prune_magnitude
    torch.manual_seed(0)
    lin = torch.nn.Linear(256, 48)
    ql = Q.Int4Linear(lin, group=64)
    x = torch.randn(5, 256)
    w = ql.dequantized_weight()
    assert (w - lin.weight).abs().max() <= 0.5 * ql.scales.max() + 1e-6
    assert torch.allclose(ql(x), x @ w.t() + lin.bias, atol=1e-5)
    q, s = Q.quantize_int8_rowwise(x)
    assert (Q.dequantize_int8_rowwise(q, s) - x).abs().max() <= 0.5 * s.max() + 1e-6
    a = prune_magnitude(torch.randn(40, 60), 0.85)
    sp = CudaSparseTensor.from_dense(a)
    b = torch.randn(60, 9)
    assert torch.allclose(sp @ b, a @ b, atol=1e-5) and torch.equal(sp.to_dense(), a)
    assert torch.equal(CudaSparseTensor.from_coo(CooTensor.from_dense(a)).to_dense(), a)
    assert torch.equal(sp.transpose().to_dense(), a.t()) and sp.nnz == int((a != 0).sum())


def test_lstm_and_grouped_conv_cpu_paths():
    """KernelLSTM shares torch.nn.LSTM's parameters and semantics; the grouped / depthwise front ends agree with
    torch.nn.functional.conv2d on a CPU."""
    from torsh_b200.ops.conv import depthwise_conv2d_nhwc, grouped_conv2d_nhwc
    from torsh_b200.ops.rnn import KernelLSTM
    torch.manual_seed(0)
    ref = torch.nn.LSTM(12, 20, num_layers=2)
    mine = KernelLSTM(12, 20, num_layers=2)
    mine.load_state_dict(ref.state_dict())
    x = torch.randn(7, 3, 12)
    out, (h, c) = mine(x)
    out_r, (h_r, c_r) = ref(x)
    assert torch.allclose(out, out_r, atol=1e-5) and torch.allclose(h, h_r, atol=1e-5) and torch.allclose(c, c_r, atol=1e-5)
    xi = torch.randn(2, 9, 9, 16)
    wd = torch.randn(16, 1, 3, 3)
    yr = torch.nn.functional.conv2d(xi.permute(0, 3, 1, 2), wd, None, 1, 1, groups=16).permute(0, 2, 3, 1)
    assert torch.allclose(depthwise_conv2d_nhwc(xi, wd, None, 1, 1), yr, atol=1e-5)
    wg = torch.randn(8, 4, 3, 3)
    yg = torch.nn.functional.conv2d(xi.permute(0, 3, 1, 2), wg, None, 1, 1, groups=4).permute(0, 2, 3, 1)
    assert torch.allclose(grouped_conv2d_nhwc(xi, wg, None, 1, 1, groups=4), yg, atol=1e-4)


def test_loss_family_values_and_gradients():
    """Every loss of the functional family: closed-form values on small cases, PyTorch parity where a torch loss exists,
    and a finite gradient."""
    import math
    from torsh_b200.nn import losses as L
    torch.manual_seed(0)
    assert len(L.__all__) >= 28
    logits = torch.randn(6, 5, requires_grad=True)
    tgt = torch.tensor([0, 1, 2, 3, 4, 0])
    assert torch.allclose(L.cross_entropy(logits, tgt), torch.nn.functional.cross_entropy(logits, tgt))
    assert torch.allclose(L.cross_entropy_with_label_smoothing(logits, tgt, 0.1),
                          torch.nn.functional.cross_entropy(logits, tgt, label_smoothing=0.1), atol=1e-6)
    assert torch.allclose(L.nll_loss(logits.log_softmax(-1), tgt), L.cross_entropy(logits, tgt))
    x, y = torch.rand(4, 3), (torch.rand(4, 3) > 0.5).float()
    assert torch.allclose(L.binary_cross_entropy_with_logits(torch.logit(x), y), L.binary_cross_entropy(x, y), atol=1e-5)
    assert torch.allclose(L.focal_loss(torch.logit(x), y, alpha=0.5, gamma=0.0), 0.5 * L.binary_cross_entropy(x, y), atol=1e-5)
    a, b = torch.randn(5, 8), torch.randn(5, 8)
    assert torch.allclose(L.mse_loss(a, b), ((a - b) ** 2).mean()) and torch.allclose(L.l1_loss(a, b, "sum"), (a - b).abs().sum())
    assert torch.allclose(L.smooth_l1_loss(a, b, 1.0), L.huber_loss(a, b, 1.0))
    var = torch.rand(5, 8) + 0.1
    assert torch.allclose(L.gaussian_nll_loss(a, b, var), (0.5 * (var.log() + (a - b) ** 2 / var)).mean(), atol=1e-6)
    assert torch.allclose(L.poisson_nll_loss(a, b.abs()), (a.exp() - b.abs() * a).mean(), atol=1e-6)
    lab = torch.tensor([1., -1., 1., -1., 1.])
    assert torch.allclose(L.cosine_embedding_loss(a, a, torch.ones(5)), torch.zeros(()), atol=1e-6)
    assert torch.allclose(L.margin_ranking_loss(a[:, 0], b[:, 0], lab, 0.5), (-lab * (a[:, 0] - b[:, 0]) + 0.5).clamp_min(0).mean())
    assert L.hinge_embedding_loss(a[:, 0].abs(), lab, 1.0) >= 0 and L.multi_margin_loss(logits, tgt) >= 0
    n = torch.randn(5, 8)
    assert torch.allclose(L.triplet_margin_loss(a, b, n), L.triplet_margin_with_distance_loss(a, b, n), atol=1e-5)
    assert torch.allclose(L.contrastive_loss(a, a, torch.ones(5)), torch.zeros(()), atol=1e-9)
    p, q = torch.softmax(torch.randn(4, 6), -1), torch.softmax(torch.randn(4, 6), -1)
    assert torch.allclose(L.kl_div(q.log(), p, "sum"), (p * (p.log() - q.log())).sum(), atol=1e-6)
    js = L.js_divergence(p, q, "none")
    assert (js >= -1e-7).all() and (js <= math.log(2) + 1e-6).all() and torch.allclose(L.js_divergence(p, p), torch.zeros(()), atol=1e-6)
    assert torch.allclose(L.js_divergence(p, q), L.js_divergence(q, p), atol=1e-6)
    assert torch.allclose(L.cross_entropy_continuous(p, p, "sum"), L.entropy_loss(p, "sum"), atol=1e-6)
    u = torch.full((1, 4), 0.25)
    assert torch.allclose(L.entropy_loss(u, "sum"), torch.tensor(math.log(4)), atol=1e-6)
    assert L.mutual_information_loss(torch.full((16,), 3.0), torch.zeros(16)) < -2.9      # critic separates the two sets
    lp = torch.randn(12, 2, 5).log_softmax(-1)
    ctc = L.ctc_loss(lp, torch.tensor([[1, 2], [3, 3]]), torch.tensor([12, 12]), torch.tensor([2, 2]))
    assert torch.isfinite(ctc) and ctc > 0
    assert torch.allclose(L.wasserstein_loss(torch.ones(4), torch.zeros(4)), torch.tensor(-1.0))
    gsamp = torch.randn(3, 2, 4)
    gsamp = gsamp / gsamp.flatten(1).norm(dim=1)[:, None, None]
    assert torch.allclose(L.gradient_penalty_loss(gsamp, 10.0), torch.zeros(()), atol=1e-9)
    assert torch.allclose(L.gradient_penalty_loss(2 * gsamp, 10.0), torch.tensor(10.0), atol=1e-4)
    seq = torch.arange(10.0).reshape(1, 10, 1)
    assert torch.allclose(L.temporal_consistency_loss(seq, 2.0), torch.tensor(2.0))
    pred = torch.randn(2, 4, 7, requires_grad=True)
    tg2 = torch.randint(0, 7, (2, 4))
    att = torch.softmax(torch.randn(2, 4, 5), -1)
    base = L.seq2seq_loss_with_attention(pred, tg2)
    assert torch.allclose(base, torch.nn.functional.cross_entropy(pred.reshape(8, 7), tg2.reshape(8)))
    withreg = L.seq2seq_loss_with_attention(pred, tg2, att, 0.5)
    assert torch.allclose(withreg - base, 0.5 * (1 - att.sum(1)).pow(2).sum(-1).mean(), atol=1e-6)
    (L.cross_entropy(logits, tgt) + withreg).backward()
    assert torch.isfinite(logits.grad).all() and torch.isfinite(pred.grad).all()


def test_spectral_family():
    import math
    from torsh_b200 import signal as S
    torch.manual_seed(0)
    x = torch.randn(3, 256)
    assert torch.allclose(S.ifft(S.fft(x)).real, x, atol=1e-5) and torch.allclose(S.irfft(S.rfft(x), 256), x, atol=1e-5)
    img = torch.randn(2, 16, 16)
    assert torch.allclose(S.ifftn(S.fftn(img)).real, img, atol=1e-5) and S.rfft2(img).shape == (2, 16, 9) and S.rfftn(img).shape[-1] == 9
    assert torch.allclose(S.fft2(img), S.fftn(img, dim=(-2, -1)), atol=1e-5)
    assert torch.allclose(S.ihfft(x[0]), S.rfft(x[0]).conj() / 256, atol=1e-6) and S.hfft(S.ihfft(x[0]), 256).shape == (256,)
    for htk in (True, False):
        f = torch.tensor([0.0, 440.0, 1000.0, 4000.0, 8000.0], dtype=torch.float64)
        assert torch.allclose(S.mel_to_hz(S.hz_to_mel(f, htk), htk), f, atol=1e-6)
    assert abs(float(S.hz_to_mel(1000.0)) - 999.99) < 0.1
    sr, t = 16000, torch.arange(16000) / 16000
    tone = torch.sin(2 * math.pi * 1000 * t)
    spec = S.spectrogram(tone, 512, 128)
    cen = S.spectral_centroid(spec, sr)
    assert abs(float(cen[5:-5].mean()) - 1000) < 40 and abs(float(S.spectral_rolloff(spec, sr, 0.85)[5:-5].mean()) - 1000) < 80
    mel = S.mel_spectrogram(tone, sr, 512, 128, n_mels=40, log=True)
    assert mel.shape[0] == 40 and torch.isfinite(mel).all()
    band = int(mel[:, 10].argmax())
    centre = float(S.mel_to_hz(torch.linspace(float(S.hz_to_mel(0.0)), float(S.hz_to_mel(8000.0)), 42)[band + 1]))
    assert abs(centre - 1000) < 150
    assert torch.allclose(S.create_mel_filterbank(40, 512, sr), S.mel_filterbank(40, 512, sr))
    X = S.stft_complete(x[0], 64, 16)
    assert torch.allclose(S.istft_complete(X, 64, 16, length=256), x[0], atol=1e-4)
    # cepstrum of an impulse train with period 32 has its first rahmonic at quefrency 32
    e = torch.zeros(256); e[::32] = 1.0
    c = S.cepstrum(e + 1e-3 * torch.randn(256))
    assert int(c[8:128].argmax()) + 8 == 32
    assert torch.equal(S.generate_window("hann", 16), S.window("hann", 16))


def test_text_generation_metrics_datasets_embeddings(tmp_path):
    import json
    import math
    from torsh_b200.text import Vocab, WhitespaceTokenizer
    from torsh_b200.text import datasets as D, embeddings as E, generation as G, metrics as M
    V = 10

    def step(ids):                                   # toy LM: strongly prefers last + 1, weakly last + 2
        l = torch.full((ids.shape[0], V), -6.0)
        r = torch.arange(ids.shape[0])
        l[r, (ids[:, -1] + 1) % V] = 4.0
        l[r, (ids[:, -1] + 2) % V] = 3.0
        return l
    assert G.TextGenerator(G.GenerationConfig(max_length=8, eos_token_id=7)).generate(step, [2, 3]) == [2, 3, 4, 5, 6, 7]
    beams = G.BeamSearchDecoder(3, 7, 1.0, eos_token_id=None).search(step, torch.tensor([0]))
    assert beams[0].tokens == [0, 1, 2, 3, 4, 5, 6] and beams[0].score > beams[1].score and len(beams) == 3
    s = G.TextSampler(seed=0)
    logits = torch.tensor([0.0, 5.0, 4.0, -3.0])
    assert s.greedy_sample(logits) == 1 and s.top_k_sample(logits, 1) == 1 and s.top_p_sample(logits, 0.5) == 1
    draws = {s.top_k_top_p_sample(logits, 2, 1.0, 1.0) for _ in range(40)}
    assert draws == {1, 2}
    pen = G.RepetitionPenalty.apply(torch.tensor([2.0, -2.0, 1.0]), [0, 1], 2.0)
    assert pen.tolist() == [1.0, -4.0, 1.0]
    f = G.NGramRepetitionFilter(2)
    assert f.banned([1, 2, 3, 1]) == {2} and f.filter_logits(torch.zeros(5), [1, 2, 3, 1])[2] == float("-inf")
    sampled = G.TextGenerator(G.GenerationConfig(max_length=12, do_sample=True, top_k=2, temperature=0.7, seed=3, no_repeat_ngram_size=2)).generate(step, [0])
    grams = list(zip(sampled, sampled[1:]))
    assert len(sampled) == 12 and len(set(grams[1:])) == len(grams[1:])
    # metrics
    ref, cand = "the cat sat on the mat".split(), "the cat sat on a mat".split()
    assert M.bleu([ref], [[ref]]) == 1.0 and 0.5 < M.sentence_bleu(cand, [ref]) < 1.0 and M.bleu([["x"]], [[ref]]) == 0.0
    assert M.rouge_n(cand, ref, 1)["f1"] == pytest.approx(5 / 6) and M.rouge_l(cand, ref)["recall"] == pytest.approx(5 / 6)
    assert M.edit_distance("kitten", "sitting") == 3 and M.word_error_rate("a b c", "a x c d") == pytest.approx(0.5)
    lg = torch.zeros(4, 8)
    assert M.perplexity(lg, torch.tensor([1, 2, 3, 4])) == pytest.approx(8.0, rel=1e-5)
    assert M.token_overlap_f1(cand, ref)["precision"] == pytest.approx(5 / 6)
    table = torch.eye(12)
    emb = lambda toks: table[[hash(t) % 12 for t in toks]]
    assert M.embedding_match_score(ref, ref, emb)["f1"] == pytest.approx(1.0)
    # datasets
    (tmp_path / "c.csv").write_text("text,label\nGood film,pos\nBad film,neg\nGreat   FUN movie,pos\n")
    tok = WhitespaceTokenizer()
    vocab = Vocab.build(["good film bad great fun movie"])
    pipe = D.PreprocessingPipeline(D.PreprocessingConfig(max_length=3), tok, vocab)
    ds = D.ClassificationDataset(tmp_path / "c.csv", pipeline=pipe)
    assert len(ds) == 3 and ds.num_classes == 2 and ds.label_names == ["neg", "pos"] and ds[2] == (vocab.encode(["great", "fun", "movie"]), 1)
    (tmp_path / "c.jsonl").write_text("\n".join(json.dumps({"text": t, "label": l}) for t, l in [("a b", 1), ("c", 0)]))
    assert D.ClassificationDataset(tmp_path / "c.jsonl")[0] == ("a b", 1)
    batches = list(D.BatchIterator(D.CachedDataset(ds), 2, pad_id=0, bucket=True))
    assert batches[0]["input_ids"].shape == (2, 2) and batches[0]["labels"].tolist() == [1, 0] and batches[1]["lengths"].tolist() == [3]
    lm = D.LanguageModelingDataset(list(range(20)), block_size=4, stride=4)
    x, y = lm[1]
    assert len(lm) == 4 and x.tolist() == [4, 5, 6, 7] and y.tolist() == [5, 6, 7, 8]
    (tmp_path / "train.de").write_text("ein hund\n\nzwei katzen\n")
    (tmp_path / "train.en").write_text("a dog\n\ntwo cats\n")
    tr = D.multi30k(tmp_path, "train")
    assert len(tr) == 2 and tr[1] == ("zwei katzen", "two cats")
    (tmp_path / "ner.conll").write_text("-DOCSTART- O\n\nJohn B-PER\nsmiles O\n\nParis B-LOC\n")
    ner = D.SequenceLabelingDataset(tmp_path / "ner.conll")
    assert len(ner) == 2 and ner[0] == (["John", "smiles"], ["B-PER", "O"]) and ner.tag_names == ["B-LOC", "B-PER", "O"]
    (tmp_path / "train.csv").write_text('"3","Title","Stocks rise"\n"1","T2","Match won"\n')
    ag = D.ag_news(tmp_path, "train")
    assert len(ag) == 2 and ag[0] == ("Stocks rise", 1)
    (tmp_path / "wiki.train.tokens").write_text(" = Title = \n the quick brown fox jumps over the lazy dog again and again \n")
    wt = D.wikitext(tmp_path, "train", block_size=4)
    assert len(wt) >= 2 and wt[0][0].shape == (4,)
    with pytest.raises(FileNotFoundError):
        D.ag_news(tmp_path / "nope")
    ids, mask, lens = D.pad_sequences([[1, 2, 3], [4]], pad_id=9)
    assert ids.tolist() == [[1, 2, 3], [4, 9, 9]] and mask.tolist() == [[True, True, True], [True, False, False]] and lens.tolist() == [3, 1]
    # embeddings
    (tmp_path / "glove.txt").write_text("3 4\ngood 1 0 0 0\nfilm 0 1 0 0\nzzz 0 0 1 0\n")
    w = E.EmbeddingUtils.load_pretrained_embeddings(tmp_path / "glove.txt", vocab)
    assert w.shape == (len(vocab), 4) and w[vocab["good"]].tolist() == [1, 0, 0, 0] and w.found == 2
    toks, mat = E.EmbeddingUtils.load_pretrained_embeddings(tmp_path / "glove.txt")
    assert toks == ["good", "film", "zzz"] and mat.shape == (3, 4)
    we = E.WordEmbedding.from_pretrained(w)
    assert not we.emb.weight.requires_grad and torch.equal(we(torch.tensor([vocab["film"]]))[0], w[vocab["film"]])
    pe = E.PositionalEncoding(8, 32)
    z = torch.zeros(2, 5, 8)
    assert torch.allclose(pe(z)[0, 0], torch.tensor([0., 1.] * 4)) and torch.allclose(pe(z, offset=3)[0, 0], pe.pe[3])
    ce = E.CombinedEmbeddings(len(vocab), 8, max_len=16, dropout=0.0)
    out = ce(torch.tensor([[1, 2, 3]]), torch.tensor([[0, 0, 1]]))
    assert out.shape == (1, 3, 8) and abs(float(out.mean())) < 1e-5
    ee = torch.tensor([[1., 0.], [0.9, 0.1], [0., 1.]])
    assert E.EmbeddingUtils.most_similar(ee, 0, 1)[0][0] == 1 and E.EmbeddingUtils.cosine_similarity(ee, 0, 2) == 0.0
    assert E.EmbeddingUtils.xavier_uniform_embeddings(10, 4).abs().max() <= math.sqrt(6 / 14) + 1e-6


def test_vision_detection_and_image_io(tmp_path):
    from torsh_b200.vision import box_iou, detection as Det, io as VIO
    torch.manual_seed(0)
    # anchors, coding, matching
    ag = Det.AnchorGenerator(sizes=(32, 64), ratios=(0.5, 1.0, 2.0), scales=(1.0,))
    anchors = ag([(4, 4), (2, 2)], [8, 16])
    assert anchors.shape == (4 * 4 * 3 + 2 * 2 * 3, 4) and ag.num_anchors == 3
    a0 = anchors[1]                                       # ratio 1 at the first cell: a 32 x 32 box centred at (4, 4)
    assert torch.allclose(a0, torch.tensor([-12., -12., 20., 20.]))
    coder = Det.BoxCoder()
    gt = torch.tensor([[2., 3., 30., 40.], [10., 10., 20., 28.]])
    sel = anchors[:2]
    assert torch.allclose(coder.decode(coder.encode(gt, sel), sel), gt, atol=1e-4)
    m = Det.match_anchors(anchors, gt)
    assert set(m.tolist()) <= {-2, -1, 0, 1} and (m == 0).any() and (m == 1).any()
    assert (Det.match_anchors(anchors, torch.zeros(0, 4)) == -1).all()
    # post-processing
    boxes = torch.tensor([[0., 0., 10., 10.], [1., 1., 11., 11.], [50., 50., 60., 60.]])
    scores = torch.tensor([[0.9, 0.0], [0.8, 0.0], [0.1, 0.7]])
    dets = Det.postprocess(boxes, scores, 0.05, 0.5, 10, (64, 64))
    assert [(d.label, round(d.score, 2)) for d in dets] == [(0, 0.9), (1, 0.7), (0, 0.1)]
    assert dets[0].box.area() == 100.0 and dets[0].box.center() == (5.0, 5.0)
    # detectors: shapes, losses decrease under a few steps, detections decode
    net = Det.retinanet_tiny(3)
    img = torch.randn(2, 3, 64, 64)
    cls, reg, anc = net(img)
    assert cls.shape == (2, anc.shape[0], 3) and reg.shape == (2, anc.shape[0], 4)
    assert torch.sigmoid(cls).mean() < 0.05                  # focal-loss prior: everything starts as background
    targets = [{"boxes": torch.tensor([[8., 8., 40., 40.]]), "labels": torch.tensor([1])},
               {"boxes": torch.tensor([[20., 16., 60., 50.], [4., 30., 30., 62.]]), "labels": torch.tensor([0, 2])}]
    opt = torch.optim.Adam(net.parameters(), 1e-3)
    first = last = None
    for _ in range(12):
        l = net.loss(img, targets)
        tot = l["classification"] + l["regression"]
        opt.zero_grad(); tot.backward(); opt.step()
        first = float(tot) if first is None else first
        last = float(tot)
    assert last < first
    net.eval()
    assert all(isinstance(d, Det.Detection) for d in net.detect(img, score_thresh=0.0, top_k=5)[0])
    ssd = Det.ssd_tiny(4).eval()
    c2, r2, a2 = ssd(img)
    assert c2.shape == (2, a2.shape[0], 5) and len(ssd.detect(img, score_thresh=0.0, top_k=7)[1]) == 7
    pred = torch.zeros(1, 2, 4, 4, 5 + 3)
    yb, ys = Det.decode_yolo_grid(pred, [(10., 20.), (30., 30.)], stride=8)
    assert yb.shape == (1, 32, 4) and ys.shape == (1, 32, 3) and torch.allclose(ys, torch.full_like(ys, 0.25))
    assert torch.allclose(yb[0, 0], torch.tensor([4 - 5., 4 - 10., 4 + 5., 4 + 10.]))     # sigmoid(0): centre of cell 0, anchor size
    # image IO round trips in every format
    io = VIO.VisionIO().with_caching(True, 4)
    rgb = (torch.rand(3, 13, 17) * 255).to(torch.uint8)
    for ext in ("png", "ppm", "bmp", "npy"):
        io.save_image(rgb, tmp_path / f"a.{ext}")
        assert torch.equal(io.load_image(tmp_path / f"a.{ext}"), rgb), ext
    grey = (torch.rand(1, 9, 5) * 255).to(torch.uint8)
    io.save_image(grey, tmp_path / "g.pgm"); io.save_image(grey, tmp_path / "g.png")
    assert torch.equal(io.load_image(tmp_path / "g.pgm"), grey) and torch.equal(io.load_image(tmp_path / "g.png"), grey)
    rgba = (torch.rand(4, 6, 6) * 255).to(torch.uint8)
    io.save_image(rgba, tmp_path / "t.png")
    assert torch.equal(io.load_image(tmp_path / "t.png"), rgba)
    io.save_image(torch.full((3, 4, 4), 0.5), tmp_path / "f.png")
    assert int(io.load_image(tmp_path / "f.png")[0, 0, 0]) == 128
    # a PNG whose scan lines use the Sub / Up / Average / Paeth filters decodes to the same pixels
    import struct, zlib
    arr = rgb.permute(1, 2, 0).numpy().astype(int)
    h, w, c = arr.shape
    flat = arr.reshape(h, w * c)
    raw = bytearray()
    for y in range(h):
        f = [1, 2, 3, 4][y % 4]
        raw.append(f)
        for i in range(w * c):
            a = flat[y, i - c] if i >= c else 0
            b = flat[y - 1, i] if y else 0
            cc = flat[y - 1, i - c] if (y and i >= c) else 0
            p = a + b - cc
            paeth = a if (abs(p - a) <= abs(p - b) and abs(p - a) <= abs(p - cc)) else (b if abs(p - b) <= abs(p - cc) else cc)
            pred = {1: a, 2: b, 3: (a + b) // 2, 4: paeth}[f]
            raw.append((flat[y, i] - pred) & 255)
    png = (b"\\x89PNG\\r\\n\\x1a\\n".decode("unicode_escape").encode("latin1") + VIO._png_chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
           + VIO._png_chunk(b"IDAT", zlib.compress(bytes(raw))) + VIO._png_chunk(b"IEND", b""))
    assert torch.equal(VIO.decode_png(png), rgb)
    (tmp_path / "bad.png").write_bytes(b"not an image")
    res = io.load_images_from_dir(tmp_path)
    assert not res.all_successful() and len(res.failed) == 1 and "bad.png" in res.failed[0][0] and 0.8 < res.success_rate() < 1.0
    assert len(io.load_images_with_pattern(tmp_path, "a.*").ok) == 4
    conv = io.batch_convert_format([tmp_path / "a.png", tmp_path / "g.pgm"], tmp_path / "out", "bmp")
    assert conv.all_successful() and torch.equal(io.load_image(tmp_path / "out" / "a.bmp"), rgb)
    saved = io.batch_save_images([rgb, grey], tmp_path / "batch", fmt="png")
    assert saved.all_successful() and (tmp_path / "batch" / "img_00001.png").exists()
    info = io.get_image_info(tmp_path / "a.png")
    assert (info.width, info.height, info.channels, info.format) == (17, 13, 3, "png") and info.file_size > 0
    assert io.is_supported_image("x.PNG") and not io.is_supported_image("x.gif") and "png" in io.supported_formats()
    VIO.configure_global_io(io)
    assert VIO.global_io() is io


def test_rl_models_learn_a_two_armed_bandit_chain():
    """DQN with replay and a target net, PPO with GAE and A3C n-step loss each improve on a tiny deterministic task:
    state = one-hot position on a 4-cell line, action 1 moves right (+1 reward at the end), action 0 ends the episode."""
    import random
    from torsh_b200.models import create_model, rl
    torch.manual_seed(0)
    rng = random.Random(0)

    def env_step(pos, a):
        if a == 0:
            return pos, 0.0, True
        return pos + 1, (1.0 if pos + 1 == 3 else 0.0), pos + 1 == 3
    onehot = lambda p: torch.eye(4)[p]
    q, tgt = rl.DQN(rl.DQNConfig(4, 2, (32,), dueling=True)), rl.DQN(rl.DQNConfig(4, 2, (32,), dueling=True))
    tgt.load_state_dict(q.state_dict())
    buf, opt = rl.ReplayBuffer(500, 4), torch.optim.Adam(q.parameters(), 5e-3)
    for ep in range(150):
        pos, done = 0, False
        while not done:
            a = q.act(onehot(pos), epsilon=0.3, rng=rng)
            npos, r, done = env_step(pos, a)
            buf.push(onehot(pos), a, r, onehot(min(npos, 3)), done)
            pos = npos
        if len(buf) >= 32:
            for _ in range(2):
                loss = q.td_loss(tgt, buf.sample(32))
                opt.zero_grad(); loss.backward(); opt.step()
        if ep % 10 == 0:
            tgt.load_state_dict(q.state_dict())
    assert all(q.act(onehot(p), epsilon=0.0) == 1 for p in range(3))               # learned to walk right
    # GAE on a known trajectory
    adv, ret = rl.gae(torch.tensor([0., 0., 1.]), torch.zeros(3), torch.tensor([0., 0., 1.]), 5.0, gamma=0.5, lam=1.0)
    assert torch.allclose(ret, torch.tensor([0.25, 0.5, 1.0])) and torch.allclose(adv, ret)
    ppo = create_model("ppo", state_dim=4, action_dim=2, hidden=(32,))
    popt = torch.optim.Adam(ppo.parameters(), 1e-2)
    def rollout():
        S, A, LP, R, V, D = [], [], [], [], [], []
        for _ in range(16):
            pos, done = 0, False
            while not done:
                a, lp, v = ppo.act(onehot(pos)[None])
                npos, r, done = env_step(pos, int(a))
                S.append(onehot(pos)); A.append(int(a)); LP.append(float(lp)); R.append(r); V.append(float(v)); D.append(done)
                pos = npos
        return torch.stack(S), torch.tensor(A), torch.tensor(LP), torch.tensor(R), torch.tensor(V), torch.tensor(D)
    first = None
    for it in range(30):
        S, A, LP, R, V, D = rollout()
        first = float(R.sum()) if first is None else first
        adv, ret = rl.gae(R, V, D, 0.0, ppo.cfg.gamma, ppo.cfg.lam)
        for _ in range(4):
            l = ppo.loss(S, A, LP, adv, ret)
            popt.zero_grad(); l["total"].backward(); popt.step()
    assert float(rollout()[3].sum()) > max(first, 8.0)                             # most of 16 episodes reach the goal
    a3c = create_model("a3c", state_dim=4, action_dim=2, hidden=32)
    l0 = a3c.loss(torch.eye(4)[:3], torch.tensor([1, 1, 1]), torch.tensor([0., 0., 1.]))
    l0.backward()
    assert torch.isfinite(l0) and all(p.grad is not None for p in a3c.parameters())
    cont = rl.PPO(rl.PPOConfig(3, 2, (16,), continuous=True))
    a, lp, v = cont.act(torch.randn(5, 3))
    assert a.shape == (5, 2) and lp.shape == (5,) and v.shape == (5,)


def test_video_generative_few_shot_and_3d_models():
    from torsh_b200.models import create_model, few_shot as FS, generative as G, list_models, video as VD, vision_3d as V3
    torch.manual_seed(0)
    assert {"dqn", "slowfast", "vae", "diffusion_unet", "pointnet2", "video_transformer"} <= set(list_models())
    clip = torch.randn(2, 3, 8, 64, 64)
    for m in (VD.ResNet3D(VD.ResNet3DConfig(num_classes=5, widths=(8, 16), depths=(1, 1))),
              VD.SlowFast(VD.SlowFastConfig(num_classes=5, widths=(16, 32))),
              VD.VideoTransformer(VD.VideoTransformerConfig(num_classes=5, dim=32, depth=1))):
        out = m(clip)
        out.sum().backward()
        assert out.shape == (2, 5) and all(p.grad is not None for p in m.parameters() if p.requires_grad)
    # VAE: the ELBO falls; eval mode is deterministic
    x = torch.rand(8, 3, 32, 32)
    vae = create_model("vae", latent_dim=8, widths=(8, 16))
    opt = torch.optim.Adam(vae.parameters(), 2e-3)
    losses = []
    for _ in range(15):
        l = vae.loss(x)["total"]
        opt.zero_grad(); l.backward(); opt.step(); losses.append(float(l))
    assert losses[-1] < losses[0]
    vae.eval()
    assert torch.equal(vae(x)[0], vae(x)[0]) and vae.sample(3).shape == (3, 3, 32, 32)
    # GAN: shapes, both objectives, gradient penalty is differentiable w.r.t. the discriminator
    gan = G.GAN(G.GANConfig(latent_dim=16, width=8))
    fake = gan.generate(4)
    assert fake.shape == (4, 3, 32, 32) and fake.abs().max() <= 1
    assert gan.discriminator_loss(x[:4] * 2 - 1, fake) > 0 and torch.isfinite(gan.generator_loss(fake, wasserstein=True))
    gan.gradient_penalty(x[:4] * 2 - 1, fake).backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in gan.discriminator.parameters())
    # diffusion: schedules, q_sample limits, loss falls, both samplers return finite images
    cfg = G.DiffusionConfig(width=8, timesteps=50)
    diff = G.GaussianDiffusion(cfg)
    assert (diff.alphas_bar[1:] < diff.alphas_bar[:-1]).all() and G.GaussianDiffusion(G.DiffusionConfig(schedule="cosine")).alphas_bar[-1] < 1e-3
    x0, noise = x * 2 - 1, torch.randn_like(x)
    assert torch.allclose(diff.q_sample(x0, torch.zeros(8, dtype=torch.long), noise), x0, atol=0.05)
    unet = G.DiffusionUNet(cfg)
    dopt = torch.optim.Adam(unet.parameters(), 2e-3)
    gen = torch.Generator().manual_seed(0)
    hist = []
    for _ in range(25):
        l = diff.loss(unet, x0, gen)
        dopt.zero_grad(); l.backward(); dopt.step(); hist.append(float(l))
    assert sum(hist[-5:]) < sum(hist[:5])
    assert torch.isfinite(diff.sample(unet, (2, 3, 32, 32), steps=5, eta=0.0)).all() and diff.sample(unet, (1, 3, 32, 32)).shape == (1, 3, 32, 32)
    # few-shot: clusters in 2-D; prototypes classify them, MAML / Reptile adapt a linear model
    centers = torch.tensor([[4., 0.], [-4., 0.], [0., 4.], [0., -4.], [4., 4.], [-4., -4.]])
    y = torch.arange(6).repeat_interleave(12)
    xs = centers[y] + 0.3 * torch.randn(72, 2)
    fcfg = FS.FewShotConfig(n_way=3, k_shot=2, n_query=4, inner_lr=0.5, inner_steps=3)
    ds = FS.FewShotDataset(xs, y, fcfg)
    ep = ds.sample_episode()
    assert ep.support_x.shape == (6, 2) and ep.query_y.tolist() == [0] * 4 + [1] * 4 + [2] * 4
    proto = FS.PrototypicalNetwork(torch.nn.Identity(), fcfg)
    assert FS.FewShotEvaluator(ds, 20).evaluate(proto).mean_accuracy > 0.95
    for metric in ("cosine", "manhattan"):
        assert FS.pairwise_distance(xs[:3], xs[:3], metric).diagonal().abs().max() < 1e-5
    lin = torch.nn.Linear(2, 3)
    maml = FS.MAML(lin, fcfg)
    mopt = torch.optim.Adam(lin.parameters(), 1e-2)
    for _ in range(30):
        l, _ = maml.meta_loss(ds.sample_episode())
        mopt.zero_grad(); l.backward(); mopt.step()
    ev = FS.FewShotEvaluator(ds, 20).evaluate(lambda e: torch.func.functional_call(lin, maml.adapt(e, create_graph=False), (e.query_x,)))
    assert ev.mean_accuracy > 0.8 and ev.episodes == 20 and ev.ci95 >= 0
    rep = FS.Reptile(torch.nn.Linear(2, 3), fcfg, meta_lr=0.3)
    accs = [rep.meta_step(ds.sample_episode()) for _ in range(20)]
    assert sum(accs[-5:]) / 5 > 0.7
    with pytest.raises(ValueError):
        FS.FewShotDataset(xs, y, FS.FewShotConfig(n_way=7))
    # 3-D: PointNet is invariant to point order, transforms start at the identity, FPS / ball query do what they say
    pts = torch.randn(2, 64, 3)
    pn = V3.PointNet().eval()
    perm = torch.randperm(64)
    assert torch.allclose(pn(pts)[0], pn(pts[:, perm])[0], atol=1e-5)
    assert torch.allclose(V3.TransformNet(3).eval()(pts.transpose(1, 2)), torch.eye(3).expand(2, 3, 3))
    assert V3.orthogonality_regularizer(torch.eye(4)[None]) == 0
    line = torch.stack([torch.arange(10.), torch.zeros(10), torch.zeros(10)], -1)[None]
    assert V3.farthest_point_sampling(line, 3)[0].tolist() == [0, 9, 4] or V3.farthest_point_sampling(line, 3)[0].tolist() == [0, 9, 5]
    bq = V3.ball_query(line, line[:, [0, 9]], radius=1.5, k=3)
    assert bq[0, 0].tolist() == [0, 1, 0] and sorted(bq[0, 1].tolist()) == [8, 9, 9]
    p2 = V3.PointNetPlusPlus(V3.PointNetPlusPlusConfig(num_classes=4, centers=(16, 4), k=8))
    out = p2(pts)
    out.sum().backward()
    assert out.shape == (2, 4) and V3.CNN3D()(torch.randn(2, 1, 16, 16, 16)).shape == (2, 10)
    assert torch.isfinite(V3.PointNet().loss(pts, torch.tensor([1, 2])))


def test_data_formats_tfrecord_idx_cifar_image_folder(tmp_path):
    import pickle
    import numpy as np
    from torsh_b200.data import formats as F
    from torsh_b200.vision.io import VisionIO
    # CRC-32C test vector (RFC 3720) and record round trip with corruption detection
    assert F.crc32c(b"123456789") == 0xE3069283 and F.crc32c(b"\x00" * 32) == 0x8A9136AA
    exs = [{"image": b"\x01\x02\x03", "label": [7], "weights": [0.5, -1.25], "name": "a"},
           {"image": b"", "label": [-3, 1 << 40], "weights": [1e-3], "name": "bb"}]
    with F.TFRecordWriter(tmp_path / "d.tfrecord") as w:
        for e in exs:
            w.write(F.encode_example(e))
    got = list(F.TFRecordDataset(tmp_path / "d.tfrecord"))
    assert got[0]["image"] == [b"\x01\x02\x03"] and got[0]["label"] == [7] and got[0]["weights"] == [0.5, -1.25] and got[0]["name"] == [b"a"]
    assert got[1]["label"] == [-3, 1 << 40] and abs(got[1]["weights"][0] - 1e-3) < 1e-9
    ds = F.TFRecordDataset([tmp_path / "d.tfrecord"], transform=lambda e: (torch.tensor(e["weights"]), e["label"][0]))
    assert [y for _, y in ds] == [7, -3]
    raw = bytearray((tmp_path / "d.tfrecord").read_bytes())
    raw[14] ^= 0xFF
    (tmp_path / "bad.tfrecord").write_bytes(bytes(raw))
    with pytest.raises(ValueError):
        list(F.read_tfrecords(tmp_path / "bad.tfrecord"))
    assert len(list(F.read_tfrecords(tmp_path / "bad.tfrecord", verify=False))) == 2
    # IDX / MNIST layout
    imgs = (torch.rand(10, 28, 28) * 255).to(torch.uint8)
    labs = torch.arange(10, dtype=torch.uint8)
    F.write_idx(tmp_path / "train-images-idx3-ubyte", imgs)
    F.write_idx(tmp_path / "train-labels-idx1-ubyte", labs)
    assert torch.equal(F.read_idx(tmp_path / "train-images-idx3-ubyte"), imgs)
    f32 = torch.randn(3, 4)
    F.write_idx(tmp_path / "f.idx", f32)
    assert torch.equal(F.read_idx(tmp_path / "f.idx"), f32)
    mn = F.MNIST(tmp_path, train=True)
    x, y = mn[3]
    assert len(mn) == 10 and x.shape == (1, 28, 28) and y == 3 and torch.allclose(x[0], imgs[3].float() / 255)
    with pytest.raises(FileNotFoundError):
        F.MNIST(tmp_path, train=False)
    # CIFAR python batches
    for name, n in (("data_batch_1", 6), ("data_batch_2", 4), ("test_batch", 5)):
        with open(tmp_path / name, "wb") as f:
            pickle.dump({b"data": np.random.randint(0, 255, (n, 3072), dtype=np.uint8), b"labels": list(range(n))}, f)
    c10 = F.CIFAR(tmp_path, train=True)
    assert len(c10) == 10 and c10[7][1] == 1 and c10[0][0].shape == (3, 32, 32) and len(F.CIFAR(tmp_path, train=False)) == 5
    # image folder
    io = VisionIO()
    for c in ("cat", "dog"):
        (tmp_path / "imgs" / c).mkdir(parents=True)
        for i in range(2):
            io.save_image((torch.rand(3, 8, 8) * 255).to(torch.uint8), tmp_path / "imgs" / c / f"{i}.png")
    (tmp_path / "imgs" / "cat" / "notes.txt").write_text("x")
    fol = F.ImageFolder(tmp_path / "imgs")
    assert fol.classes == ["cat", "dog"] and len(fol) == 4 and fol[3][1] == 1 and fol[0][0].shape == (3, 8, 8) and fol[0][0].max() <= 1


def test_linalg_equations_matrices_solvers_and_special_functions_against_scipy():
    import math
    import numpy as np
    sp = pytest.importorskip("scipy.special")
    sl = pytest.importorskip("scipy.linalg")
    st = pytest.importorskip("scipy.stats")
    from torsh_b200 import linalg as LA, special_functions as SF
    torch.manual_seed(0)
    f64 = torch.float64
    a, b, c = torch.randn(4, 4, dtype=f64), torch.randn(3, 3, dtype=f64), torch.randn(4, 3, dtype=f64)
    x = LA.solve_sylvester(a, b, c)
    assert torch.allclose(a @ x + x @ b, c, atol=1e-8)
    stable = -torch.eye(4, dtype=f64) * 2 + 0.3 * a
    q = torch.eye(4, dtype=f64)
    xl = LA.solve_lyapunov(stable, -q)
    assert torch.allclose(stable @ xl + xl @ stable.mT, -q, atol=1e-8)
    ad = 0.4 * a / a.norm()
    xd = LA.solve_discrete_lyapunov(ad, q)
    assert torch.allclose(ad @ xd @ ad.mT - xd + q, torch.zeros(4, 4, dtype=f64), atol=1e-9)
    bb, r = torch.randn(4, 2, dtype=f64), torch.eye(2, dtype=f64)
    xa = LA.solve_continuous_are(a, bb, q, r)
    assert np.allclose(xa.numpy(), sl.solve_continuous_are(a.numpy(), bb.numpy(), q.numpy(), r.numpy()), atol=1e-6)
    spd = a @ a.mT + 4 * torch.eye(4, dtype=f64)
    assert torch.allclose(LA.sqrtm(spd) @ LA.sqrtm(spd), spd, atol=1e-8) and torch.allclose(torch.linalg.matrix_exp(LA.logm(spd)), spd, atol=1e-8)
    assert torch.allclose(LA.cosm(spd) @ LA.cosm(spd) + LA.sinm(spd) @ LA.sinm(spd), torch.eye(4, dtype=f64), atol=1e-8)
    assert torch.allclose(LA.signm(spd), torch.eye(4, dtype=f64), atol=1e-8)
    u, p = LA.polar(a)
    assert torch.allclose(u @ p, a, atol=1e-10) and torch.allclose(u @ u.mT, torch.eye(4, dtype=f64), atol=1e-10)
    assert np.allclose(LA.hilbert(5).numpy(), sl.hilbert(5)) and np.allclose(LA.circulant(torch.arange(4.)).numpy(), sl.circulant(np.arange(4.)))
    cc, rr = torch.tensor([1., 2., 3.]), torch.tensor([1., 5., 6., 7.])
    assert np.allclose(LA.toeplitz(cc, rr).numpy(), sl.toeplitz(cc.numpy(), rr.numpy())) and np.allclose(LA.hankel(cc, torch.tensor([3., 8., 9.])).numpy(), sl.hankel(cc.numpy(), [3., 8., 9.]))
    assert np.allclose(LA.vandermonde(cc).numpy(), np.vander(cc.numpy()))
    coeffs = torch.tensor([6., -5.], dtype=f64)               # x^2 - 5x + 6 = (x - 2)(x - 3)
    assert sorted(torch.linalg.eigvals(LA.companion(coeffs)).real.tolist()) == pytest.approx([2.0, 3.0])
    m = torch.randn(30, 30, dtype=f64) + 8 * torch.eye(30, dtype=f64)
    rhs = torch.randn(30, dtype=f64)
    ref = torch.linalg.solve(m, rhs)
    assert torch.allclose(LA.gmres(m, rhs, restart=15), ref, atol=1e-6) and torch.allclose(LA.bicgstab(lambda v: m @ v, rhs), ref, atol=1e-6)
    fx = lambda v: (v ** 3).sum()
    v3 = torch.tensor([1., 2., 3.], dtype=f64)
    assert torch.allclose(LA.jacobian(fx, v3), 3 * v3 ** 2) and torch.allclose(LA.hessian(fx, v3), torch.diag(6 * v3))
    rep = LA.condition_report(LA.hilbert(8))
    assert rep["cond"] > 1e9 and rep["rank"] == 8 and rep["forward_error_bound"] > 1e-7
    # special functions against scipy
    mm = torch.tensor([0.0, 0.3, 0.7, 0.95], dtype=f64)
    assert np.allclose(SF.ellipk(mm).numpy(), sp.ellipk(mm.numpy()), rtol=1e-10) and np.allclose(SF.ellipe(mm).numpy(), sp.ellipe(mm.numpy()), rtol=1e-10)
    ph = torch.tensor([0.2, 0.9, 1.4], dtype=f64)
    assert np.allclose(SF.ellipkinc(ph, 0.6).numpy(), sp.ellipkinc(ph.numpy(), 0.6), rtol=1e-9) and np.allclose(SF.ellipeinc(ph, 0.6).numpy(), sp.ellipeinc(ph.numpy(), 0.6), rtol=1e-9)
    xw = torch.tensor([-0.36, -0.2, 0.0, 0.5, 3.0, 100.0], dtype=f64)
    assert np.allclose(SF.lambertw(xw).numpy(), sp.lambertw(xw.numpy()).real, rtol=1e-9, atol=1e-12)
    xm = torch.tensor([-0.36, -0.2, -0.01], dtype=f64)
    assert np.allclose(SF.lambertw(xm, -1).numpy(), sp.lambertw(xm.numpy(), -1).real, rtol=1e-9)
    assert torch.isnan(SF.lambertw(torch.tensor(-1.0)))
    xe = torch.tensor([0.05, 0.7, 1.0, 2.5, 12.0], dtype=f64)
    assert np.allclose(SF.exp1(xe).numpy(), sp.exp1(xe.numpy()), rtol=1e-9) and np.allclose(SF.expi(xe).numpy(), sp.expi(xe.numpy()), rtol=1e-9)
    assert np.allclose(SF.expn(3, xe).numpy(), sp.expn(3, xe.numpy()), rtol=1e-8)
    xo = torch.linspace(-0.95, 0.95, 7, dtype=f64)
    assert np.allclose(SF.legendre(5, xo).numpy(), sp.eval_legendre(5, xo.numpy())) and np.allclose(SF.chebyshev_t(6, xo).numpy(), sp.eval_chebyt(6, xo.numpy()))
    assert np.allclose(SF.chebyshev_u(4, xo).numpy(), sp.eval_chebyu(4, xo.numpy())) and np.allclose(SF.hermite(5, xo).numpy(), sp.eval_hermite(5, xo.numpy()))
    assert np.allclose(SF.laguerre(4, xo + 2, 0.5).numpy(), sp.eval_genlaguerre(4, 0.5, xo.numpy() + 2)) and np.allclose(SF.gegenbauer(3, 1.5, xo).numpy(), sp.eval_gegenbauer(3, 1.5, xo.numpy()))
    assert np.allclose(SF.hyp1f1(1.5, 2.5, xo * 3).numpy(), sp.hyp1f1(1.5, 2.5, xo.numpy() * 3), rtol=1e-10)
    assert np.allclose(SF.hyp2f1(0.5, 1.0, 1.5, xo * 0.9).numpy(), sp.hyp2f1(0.5, 1.0, 1.5, xo.numpy() * 0.9), rtol=1e-9)
    xa_ = torch.tensor([-4.0, -1.0, 0.0, 0.5, 2.0, 4.5], dtype=f64)
    ai, bi = SF.airy(xa_)
    ref_ai, _, ref_bi, _ = sp.airy(xa_.numpy())
    assert np.allclose(ai.numpy(), ref_ai, rtol=1e-7, atol=1e-10) and np.allclose(bi.numpy(), ref_bi, rtol=1e-7)
    far = torch.tensor([8.0, -9.0], dtype=f64)
    assert np.allclose(SF.airy(far)[0].numpy(), sp.airy(far.numpy())[0], rtol=2e-3, atol=1e-4)
    xb = torch.tensor([0.0, 0.1, 0.5, 0.9, 1.0], dtype=f64)
    assert np.allclose(SF.betainc(2.5, 1.5, xb).numpy(), sp.betainc(2.5, 1.5, xb.numpy()), atol=1e-10)
    tt = torch.tensor([-2.0, 0.0, 0.7, 3.0], dtype=f64)
    assert np.allclose(SF.student_t_cdf(tt, 5.0).numpy(), st.t.cdf(tt.numpy(), 5), atol=1e-9) and np.allclose(SF.norm_cdf(tt).numpy(), st.norm.cdf(tt.numpy()))
    assert np.allclose(SF.norm_ppf(torch.tensor([0.025, 0.5, 0.9])).numpy(), st.norm.ppf([0.025, 0.5, 0.9]), atol=1e-9)
    assert np.allclose(SF.chi2_cdf(torch.tensor([1.0, 4.0]), 3.0).numpy(), st.chi2.cdf([1.0, 4.0], 3), atol=1e-9)
    assert np.allclose(SF.f_cdf(torch.tensor([0.5, 2.0]), 4.0, 7.0).numpy(), st.f.cdf([0.5, 2.0], 4, 7), atol=1e-9)
    assert np.allclose(SF.binom_cdf(torch.tensor([2.0, 5.0, 10.0]), 10.0, 0.3).numpy(), st.binom.cdf([2, 5, 10], 10, 0.3), atol=1e-9)
    xf = torch.linspace(-6, 6, 101)
    assert (SF.fast_tanh(xf) - torch.tanh(xf)).abs().max() < 1e-3 and ((SF.fast_exp(xf) - torch.exp(xf)).abs() / torch.exp(xf)).max() < 5e-3


def test_onnx_export_import_round_trip(tmp_path):
    """Export by hand-written protobuf, parse back, evaluate: same outputs as the PyTorch module (MLP on 3-D input,
    CNN with BatchNorm / pooling, embedding classifier with functional ops)."""
    from torsh_b200 import onnx_io as O
    torch.manual_seed(0)

    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ln, self.fc1, self.act, self.fc2 = torch.nn.LayerNorm(16), torch.nn.Linear(16, 32), torch.nn.GELU(approximate="tanh"), torch.nn.Linear(32, 8, bias=False)

        def forward(self, x):
            h = self.fc2(self.act(self.fc1(self.ln(x))))
            return torch.softmax(h + h.transpose(1, 2).contiguous().transpose(1, 2) * 0.5, dim=-1)
    m = MLP()
    x = torch.randn(3, 5, 16)
    data = O.export_onnx(m, x, tmp_path / "mlp.onnx")
    back = O.load_onnx(tmp_path / "mlp.onnx")
    assert back.opset == 20 and back.producer == "torsh_b200" and back.input_names == ["x"]
    assert {"LayerNormalization", "MatMul", "Gelu", "Transpose", "Softmax"} <= set(back.op_types())
    assert torch.allclose(back(x), m.eval()(x), atol=1e-6)
    assert torch.allclose(back(torch.randn(7, 5, 16)).sum(-1), torch.ones(7, 5), atol=1e-5)        # the batch dimension is dynamic
    cnn = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, stride=2, padding=1), torch.nn.BatchNorm2d(8), torch.nn.ReLU(), torch.nn.MaxPool2d(2),
                              torch.nn.Conv2d(8, 8, 3, padding=1, groups=2, bias=False), torch.nn.SiLU(), torch.nn.AdaptiveAvgPool2d(1),
                              torch.nn.Flatten(), torch.nn.Dropout(0.5), torch.nn.Linear(8, 4))
    cnn[1].running_mean.normal_(); cnn[1].running_var.uniform_(0.5, 2.0)
    img = torch.randn(2, 3, 16, 16)
    back2 = O.load_onnx(O.export_onnx(cnn, img))
    assert torch.allclose(back2(img), cnn.eval()(img), atol=1e-5) and "Gemm" in back2.op_types() and "BatchNormalization" in back2.op_types()

    class Emb(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb, self.out = torch.nn.Embedding(50, 12), torch.nn.Linear(48, 3)

        def forward(self, ids):
            return self.out(torch.tanh(self.emb(ids)).reshape(-1, 48))
    e = Emb()
    ids = torch.randint(0, 50, (6, 4))
    back4 = O.load_onnx(O.export_onnx(e, ids))
    assert "Gather" in back4.op_types() and torch.allclose(back4(ids), e(ids), atol=1e-6)
    with pytest.raises(NotImplementedError):
        O.export_onnx(torch.nn.Sequential(torch.nn.LSTM(4, 4)), torch.randn(2, 3, 4))


def test_series_utilities_changepoints_frequency_and_forecasts():
    import math
    from torsh_b200 import series as S
    torch.manual_seed(0)
    f64 = torch.float64
    x = torch.arange(30, dtype=f64) ** 2
    assert torch.allclose(S.difference(x, 2), torch.full((28,), 2.0, dtype=f64)) and torch.allclose(S.undifference(S.difference(x), x[:1]), x)
    sx = torch.arange(24, dtype=f64) % 4 + torch.arange(24, dtype=f64)
    assert torch.allclose(S.undifference(S.difference(sx, 1, 4), sx[:4], 4), sx)
    # AR(1) with phi = 0.7: acf decays geometrically, pacf cuts off after lag 1
    e = torch.randn(4000, dtype=f64)
    ar = torch.zeros(4000, dtype=f64)
    for t in range(1, 4000):
        ar[t] = 0.7 * ar[t - 1] + e[t]
    a, pa = S.acf(ar, 3), S.pacf(ar, 3)
    assert a[0] == 1 and abs(a[1] - 0.7) < 0.05 and abs(a[2] - 0.49) < 0.07 and abs(pa[1] - 0.7) < 0.05 and abs(pa[2]) < 0.06 and abs(pa[3]) < 0.06
    t = torch.arange(512, dtype=f64)
    wave = torch.sin(2 * math.pi * t / 16) + 0.1 * torch.randn(512, dtype=f64)
    assert S.dominant_period(wave) == pytest.approx(16.0, rel=0.02) and S.spectral_entropy(wave) < 0.5 < S.spectral_entropy(torch.randn(512, dtype=f64))
    freqs, p = S.periodogram(wave, fs=1.0)
    assert float(p.sum() * (freqs[1] - freqs[0])) == pytest.approx(float(wave.var(unbiased=False)), rel=0.05)       # Parseval
    steps = torch.cat([torch.zeros(60), torch.full((50,), 4.0), torch.full((70,), -2.0)]).double() + 0.3 * torch.randn(180, dtype=f64)
    cps = S.binary_segmentation(steps, max_changes=4)
    assert len(cps) == 2 and abs(cps[0] - 60) <= 2 and abs(cps[1] - 110) <= 2 and S.binary_segmentation(0.3 * torch.randn(150, dtype=f64)) == []
    drift = torch.cat([torch.zeros(100), torch.full((100,), 2.0)]).double() + 0.5 * torch.randn(200, dtype=f64)
    alarms = S.cusum(drift, threshold=6.0, drift=0.5)
    assert alarms and S.cusum(0.5 * torch.randn(200, dtype=f64), threshold=8.0, drift=0.5) == []
    seas = torch.tensor([1., 5., 2., 8.] * 5)
    assert S.seasonal_naive(seas, 6, 4).tolist() == [1., 5., 2., 8., 1., 5.]
    assert float(S.simple_exp_smoothing(torch.full((10,), 3.0), 0.3)[0]) == pytest.approx(3.0)
    line = 2.0 * torch.arange(40, dtype=f64) + 5
    th = S.theta_forecast(line, 3)
    assert abs(float(th[0]) - 85.0) < 3.0 and torch.allclose(th[1:] - th[:-1], torch.ones(2, dtype=f64))   # half the slope: the other half sits in the flat SES line
    m = S.fit_arima(ar, (1, 0, 0))
    assert abs(float(m.ar[0]) - 0.7) < 0.05 and abs(m.sigma2 - 1.0) < 0.1
    fc = S.forecast_arima(m, 5)
    assert float(fc[0]) == pytest.approx(m.const + float(m.ar[0]) * float(ar[-1]), rel=1e-9) and abs(float(fc[-1])) < abs(float(ar[-1])) + 1
    ma = e[1:] + 0.6 * e[:-1]
    m2 = S.fit_arima(ma, (0, 0, 1))
    assert abs(float(m2.ma[0]) - 0.6) < 0.08
    rw = (0.5 + torch.randn(600, dtype=f64) * 0.1).cumsum(0)
    m3 = S.fit_arima(rw, (0, 1, 0))
    f3 = S.forecast_arima(m3, 4)
    assert m3.const == pytest.approx(0.5, abs=0.02) and torch.allclose(f3, rw[-1] + m3.const * torch.arange(1, 5, dtype=f64), atol=1e-9)
    spiky = wave.clone(); spiky[100] += 6; spiky[300] -= 6
    flags = S.anomaly_seasonal_residual(spiky, 16, z=5.0)
    assert flags[100] and flags[300] and int(flags.sum()) <= 6
    assert S.anomaly_iqr(torch.cat([torch.randn(200), torch.tensor([15.0])]))[-1]


def _softclip_for_jit_test(t):
    return 3.0 * torch.tanh(t / 3.0)


torch.fx.wrap("_softclip_for_jit_test")       # traced as one call node, which the custom-op rule below picks up


def test_jit_compiler_lowering_fusion_specialisation_debugger_and_custom_ops():
    from torsh_b200 import jit_compiler as J
    torch.manual_seed(0)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = torch.nn.Linear(16, 16)
            self.act = torch.nn.SiLU()
            self.two = torch.nn.Parameter(torch.tensor(2.0), requires_grad=False)     # a parameter stays a graph node (buffers are folded by the tracer)

        def forward(self, x, y):
            h = self.fc(x)
            z = torch.tanh(h) * y + self.act(h) - 0.5            # one element-wise region of five ops
            dead = torch.exp(z)                                   # noqa: F841  unused: removed
            scale = torch.sqrt(self.two * 8.0)                    # constant: folded to 4
            return torch.relu(z / scale).sum(-1)
    net = Net()
    x, y = torch.randn(4, 16), torch.randn(4, 16)
    gm = J.trace_with_source(net)
    g = J.lower_fx(gm, (x, y))
    assert any(n.op == "ew:tanh" for n in g.nodes) and any(n.op == "call" for n in g.nodes)
    tanh = next(n for n in g.nodes if n.op == "ew:tanh")
    assert tanh.shape == (4, 16) and tanh.dtype == torch.float32 and "test_breadth_cpu.py" in tanh.source
    assert J.constant_evaluation(g) == 2 and J.dead_code_elimination(g) >= 1 and not any(n.op == "ew:exp" for n in g.nodes)
    assert J.fuse_elementwise(g) == 1
    fused = [n for n in g.nodes if n.op == "fused"]
    assert len(fused) == 1 and fused[0].fused_ops >= 6 and len(fused[0].inputs) == 2 and "fused" in g.to_text() and "lightblue" in g.to_dot()
    exe = J.Executable(g)
    assert torch.allclose(exe(x, y), net(x, y), atol=1e-6)
    # tiered + specialised
    jf = J.jit(net, hot_threshold=2)
    for _ in range(4):
        out = jf(x, y)
    assert torch.allclose(out, net(x, y), atol=1e-6) and jf.stats.interpreted == 2 and jf.stats.compiled_calls == 2 and jf.stats.specializations == 1
    x8, y8 = torch.randn(8, 16), torch.randn(8, 16)
    for _ in range(3):
        out8 = jf(x8, y8)
    assert jf.stats.specializations == 2 and torch.allclose(out8, net(x8, y8), atol=1e-6) and jf.graph_for(x8, y8).nodes[0].shape == (8, 16)
    assert jf.stats.fused_regions == 2 and jf.stats.ops_fused >= 12

    def branchy(a):
        return a * 2 if a.sum() > 0 else a - 1                     # data-dependent control flow cannot be traced
    jb = J.jit(branchy, hot_threshold=0)
    v = torch.ones(3)
    assert torch.equal(jb(v), v * 2) and torch.equal(jb(-v), -v - 1) and jb.stats.specializations == 0 and jb.errors
    # debugger: breakpoints, watch statistics, first NaN with its source line
    def bad(a):
        b = torch.log(a - 1.0)
        return torch.relu(b) + 1.0
    gb = J.lower_fx(J.trace_with_source(bad), (torch.ones(3),))
    dbg = J.Debugger(J.Executable(gb))
    dbg.add_breakpoint("ew:log")
    dbg.run(torch.tensor([3.0, 0.5, 2.0]))
    assert len(dbg.hits) == 1 and dbg.hits[0][1] == "ew:log" and torch.isnan(dbg.hits[0][2][1])
    fb = dbg.first_bad_node()
    assert fb["op"] == "ew:log" and fb["nan"] == 1 and "test_breadth_cpu.py" in fb["source"]
    # diagnostics point at the node
    def mism(a, b):
        return torch.matmul(a, b)
    gm2 = J.lower_fx(J.trace_with_source(mism), (torch.ones(2, 3), torch.ones(3, 2)))
    with pytest.raises(J.CompileError) as ei:
        J.Executable(gm2)(torch.ones(2, 3), torch.ones(4, 2))
    assert "matmul" in str(ei.value) and "node %" in str(ei.value)
    # custom operator joining a fused region, plus a plugin pass
    import torsh_b200.jit_compiler as jc

    softclip = _softclip_for_jit_test
    jc.registry.register_op(jc.CustomOp("softclip", evaluate=softclip, match=lambda n: n.op == "call_function" and getattr(n.target, "__name__", "") == "_softclip_for_jit_test",
                                        elementwise_expr=lambda t: 3.0 * jc.kg.tanh(t / 3.0)))
    seen = []
    jc.registry.register_pass(lambda graph: seen.append([n.op for n in graph.nodes]) or 0)

    class M2(torch.nn.Module):
        def forward(self, a, b):
            return _softclip_for_jit_test(torch.sigmoid(a) * b) + b
    try:
        j2 = jc.jit(M2(), hot_threshold=0)
        a, b = torch.randn(5, 7), torch.randn(5, 7)
        assert torch.allclose(j2(a, b), softclip(torch.sigmoid(a) * b) + b, atol=1e-6) and seen
        assert j2.stats.specializations == 1
        ops = seen[-1]
        assert "fused" in ops and not any(o.startswith("custom:") for o in ops)            # the custom op was fused with its neighbours
    finally:
        jc.registry.passes.clear()
        jc.registry.ops.clear()


def test_autograd_transforms_implicit_ode_discrete_symbolic_and_analysis():
    import math
    from torsh_b200.autograd import transforms as T
    torch.manual_seed(0)
    f64 = torch.float64
    f = lambda x: (x ** 3).sum()
    x = torch.tensor([1.0, 2.0], dtype=f64)
    v, g = T.value_and_grad(f)(x)
    assert float(v) == 9.0 and torch.allclose(g, 3 * x ** 2) and torch.allclose(T.hessian(f)(x), torch.diag(6 * x))
    assert float(T.nth_derivative(lambda t: t ** 4, 3)(torch.tensor(2.0, dtype=f64))) == pytest.approx(48.0)
    assert torch.allclose(T.hessian_vector_product(f, x, torch.tensor([1.0, 1.0], dtype=f64)), 6 * x)
    assert torch.allclose(T.vmap(T.grad(lambda t: torch.sin(t)))(x), torch.cos(x))
    # meta-gradient of the post-update loss w.r.t. the inner learning-rate-like meta parameter (closed form for a quadratic)
    w0, a = torch.tensor(2.0, dtype=f64, requires_grad=True), torch.tensor(0.5, dtype=f64, requires_grad=True)
    inner = lambda th, meta: meta["a"] * th["w"] ** 2
    outer = lambda th, meta: th["w"] ** 2
    out, (ga,) = T.unrolled_meta_gradient(inner, outer, {"w": w0}, {"a": a}, inner_lr=0.1, steps=1)
    w1 = 2.0 * (1 - 0.2 * 0.5)                                   # w - lr * 2 a w
    assert float(out) == pytest.approx(w1 ** 2) and float(ga) == pytest.approx(2 * w1 * (-0.2 * 2.0))
    # fixed point z = tanh(W z + b): implicit gradients equal the gradients through 300 unrolled iterations
    W = (0.3 * torch.randn(4, 4, dtype=f64)).requires_grad_(True)
    b = torch.randn(4, dtype=f64, requires_grad=True)
    step = lambda z, W_, b_: torch.tanh(W_ @ z + b_)
    z = T.fixed_point(step, torch.zeros(4, dtype=f64), W, b, tol=1e-12, max_iter=500)
    gW, gb = torch.autograd.grad(z.sum(), (W, b))
    zu = torch.zeros(4, dtype=f64)
    for _ in range(300):
        zu = step(zu, W, b)
    rW, rb = torch.autograd.grad(zu.sum(), (W, b))
    assert torch.allclose(z, zu, atol=1e-10) and torch.allclose(gW, rW, atol=1e-8) and torch.allclose(gb, rb, atol=1e-8)
    # argmin_x 0.5 |x - theta|^2 + 0.5 |x|^2  =>  x* = theta / 2, dL/dtheta = 0.5 dL/dx
    th = torch.tensor([1.0, -2.0], dtype=f64)
    inner2 = lambda x_, t_: 0.5 * ((x_ - t_) ** 2).sum() + 0.5 * (x_ ** 2).sum()
    gth = T.argmin_implicit_gradient(inner2, th / 2, th, torch.tensor([1.0, 3.0], dtype=f64))
    assert torch.allclose(gth, torch.tensor([0.5, 1.5], dtype=f64))
    # ODE: dy/dt = -k y, exact solution and gradient w.r.t. k through both solvers
    for method in ("rk4", "dopri5"):
        k = torch.tensor(0.7, dtype=f64, requires_grad=True)
        ts = torch.linspace(0, 2, 5, dtype=f64)
        ys = T.odeint(lambda t, y: -k * y, torch.tensor([1.5], dtype=f64), ts, method=method)
        assert torch.allclose(ys[:, 0], 1.5 * torch.exp(-0.7 * ts), atol=1e-5)
        gk, = torch.autograd.grad(ys[-1, 0], k)
        assert float(gk) == pytest.approx(-2 * 1.5 * math.exp(-1.4), rel=1e-4)
    rot = T.odeint(lambda t, y: torch.stack([y[1], -y[0]]), torch.tensor([1.0, 0.0], dtype=f64), torch.tensor([0.0, math.pi], dtype=f64), method="dopri5", rtol=1e-8, atol=1e-10)
    assert torch.allclose(rot[-1], torch.tensor([-1.0, 0.0], dtype=f64), atol=1e-5)
    # discrete ops
    xr = torch.tensor([0.2, 1.7, -0.6], requires_grad=True)
    yr = T.straight_through(xr, torch.round)
    yr.sum().backward()
    assert yr.tolist() == [0.0, 2.0, -1.0] and xr.grad.tolist() == [1.0, 1.0, 1.0]
    logits = torch.tensor([[2.0, 0.5, -1.0]], requires_grad=True)
    gen = torch.Generator().manual_seed(0)
    hard = T.gumbel_softmax(logits, tau=0.5, hard=True, generator=gen)
    (hard * torch.tensor([1.0, 2.0, 3.0])).sum().backward()
    assert hard.sum() == 1 and set(hard.flatten().tolist()) <= {0.0, 1.0} and logits.grad.abs().sum() > 0
    counts = torch.stack([T.gumbel_softmax(logits.detach(), 1.0, True, gen)[0] for _ in range(400)]).mean(0)
    assert torch.allclose(counts, torch.softmax(logits.detach()[0], -1), atol=0.08)
    # score function: gradient of E_{b ~ Bernoulli(p)}[b] w.r.t. the logit is p (1 - p)
    lg = torch.tensor(0.3, requires_grad=True)
    d = torch.distributions.Bernoulli(logits=lg)
    s = d.sample((20000,))
    T.score_function_surrogate(d.log_prob(s), s, baseline=s.mean()).backward()
    p = torch.sigmoid(torch.tensor(0.3))
    assert float(lg.grad) == pytest.approx(float(p * (1 - p)), abs=0.02)
    # symbolic
    X = T.Sym.var("x")
    e = T.sym_sin(X * X) + 3 * X ** 3 - T.sym_exp(2 * X) / X
    d1 = e.diff("x").simplify()
    xv = torch.tensor(0.8, dtype=f64, requires_grad=True)
    val = e.evaluate({"x": xv})
    ref, = torch.autograd.grad(val, xv)
    assert float(d1.evaluate({"x": xv.detach()})) == pytest.approx(float(ref), rel=1e-10)
    assert str((X * 1 + 0).simplify()) == "x" and str((X ** 2).diff("x").simplify()) == "(2 * x)" and str((T.Sym.const(2) * 3).simplify()) == "6"
    # analysis tools
    deep = torch.nn.Sequential(*[m for _ in range(12) for m in (torch.nn.Linear(8, 8), torch.nn.Sigmoid())])
    deep(torch.randn(4, 8)).sum().backward()
    rep = T.gradient_flow_report(deep, vanish=1e-6)
    assert rep["max_over_min"] > 100 and "0.weight" in rep["vanishing"] and len(rep["layers"]) == 24
    ema = T.GradientFilter("ema", beta=0.5)
    assert ema(torch.ones(2)).tolist() == [1, 1] and ema(torch.full((2,), 3.0)).tolist() == [2, 2]
    med = T.GradientFilter("median", window=3)
    for gvals in (1.0, 100.0, 2.0):
        mo = med(torch.full((2,), gvals))
    assert mo.tolist() == [2.0, 2.0]
    out_f = T.GradientFilter("outlier", k=4.0)
    for i in range(10):
        out_f(torch.full((4,), 1.0 + 0.01 * i))
    assert out_f(torch.full((4,), 500.0)).max() < 2 and out_f.rejected == 1
    gcomp = T.staleness_compensated_gradient(torch.tensor([2.0]), torch.tensor([1.5]), torch.tensor([1.0]), lam=0.1)
    assert gcomp.item() == pytest.approx(2 + 0.1 * 4 * 0.5)
    pq = torch.nn.Parameter(torch.tensor([5.0]))
    hg = T.HypergradientLR([pq], lr=0.01, hyper_lr=0.001)
    for _ in range(30):
        pq.grad = 2 * pq.detach()
        hg.step()
    assert hg.lr > 0.01 and abs(float(pq)) < 5 * (1 - 0.02) ** 30               # the rate grew while successive gradients agreed
    mixed = T.MixedOp({"id": torch.nn.Identity(), "zero": torch.nn.Dropout(1.0), "double": torch.nn.Sequential()})
    opt = torch.optim.SGD([mixed.alpha], 0.5)
    xin = torch.randn(64, 4)
    mixed.train()
    for _ in range(40):
        loss = ((mixed(xin) - xin) ** 2).mean()
        opt.zero_grad(); loss.backward(); opt.step()
    assert mixed.derive() in ("id", "double") and float(torch.softmax(mixed.alpha, 0)[1]) < 0.2
    dot = T.autograd_graph_dot(deep(torch.randn(2, 8)).sum())
    assert dot.startswith("digraph autograd") and "AddmmBackward0" in dot and "->" in dot


def test_blackwell_low_precision_formats_and_structured_sparsity():
    from torsh_b200 import quantization_fp as Q
    torch.manual_seed(0)
    x = torch.randn(64, 128) * 3
    q, s = Q.fp8_quantize(x, "e4m3")
    assert q.dtype == torch.float8_e4m3fn and float(q.float().abs().max()) == 448.0 and Q.quantization_error(x, Q.fp8_dequantize(q, s))["sqnr_db"] > 25
    big, _ = Q.fp8_quantize(torch.tensor([1e9, -1e9]), "e4m3", scale=1.0)
    assert big.float().tolist() == [448.0, -448.0]                              # saturation, not NaN
    q5, s5 = Q.fp8_quantize(x, "e5m2")
    assert Q.quantization_error(x, Q.fp8_dequantize(q5, s5))["sqnr_db"] < Q.quantization_error(x, Q.fp8_dequantize(q, s))["sqnr_db"]
    ds = Q.DelayedScaling("e4m3", history=4)
    for k in range(6):
        qd, sc = ds.quantize(x * (1 + k))
    assert float(sc) == pytest.approx(float((x * 6).abs().max()) / 448.0, rel=1e-6) and len(ds.hist) == 4
    # FP4 grid: exact values survive, ties go to the even code, packing round-trips
    assert torch.equal(Q.fp4_decode(Q.fp4_encode(torch.tensor([0.0, 0.5, -1.5, 6.0, -6.0, 9.0]))), torch.tensor([0.0, 0.5, -1.5, 6.0, -6.0, 6.0]))
    assert Q.fp4_decode(Q.fp4_encode(torch.tensor([0.25, 0.75, 2.5, 5.0]))).tolist() == [0.0, 1.0, 2.0, 4.0]
    codes = torch.randint(0, 16, (5, 32), dtype=torch.uint8)
    assert torch.equal(Q.unpack_fp4(Q.pack_fp4(codes)), codes) and Q.pack_fp4(codes).shape == (5, 16)
    # MX formats: power-of-two block scales, error ordered by mantissa bits, exactness on representable data
    for fmt in ("mxfp8_e4m3", "mxfp8_e5m2", "mxfp6_e2m3", "mxfp6_e3m2", "mxfp4"):
        t = Q.mx_quantize(x, fmt)
        assert t.scale_exp.shape == (64, 4) and t.scale_exp.dtype == torch.int8 and Q.mx_dequantize(t).shape == x.shape
    e8 = Q.quantization_error(x, Q.mx_dequantize(Q.mx_quantize(x, "mxfp8_e4m3")))["sqnr_db"]
    e6 = Q.quantization_error(x, Q.mx_dequantize(Q.mx_quantize(x, "mxfp6_e2m3")))["sqnr_db"]
    e4 = Q.quantization_error(x, Q.mx_dequantize(Q.mx_quantize(x, "mxfp4")))["sqnr_db"]
    e6b = Q.quantization_error(x, Q.mx_dequantize(Q.mx_quantize(x, "mxfp6_e3m2")))["sqnr_db"]
    # E4M3 and E2M3 both carry three mantissa bits, so inside a scaled block they are equally precise; E3M2 has two, FP4 one
    assert abs(e8 - e6) < 2 and e6 > e6b > e4 > 8 and e8 > 28
    exact = torch.tensor([0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -6.0] * 4)[None] * 2.0 ** -5
    assert torch.equal(Q.mx_dequantize(Q.mx_quantize(exact, "mxfp4")), exact)
    # one outlier only hurts its own block
    xo = torch.randn(1, 64) * 0.1
    xo[0, 3] = 50.0
    d = Q.mx_dequantize(Q.mx_quantize(xo, "mxfp4"))
    assert (d[0, 32:] - xo[0, 32:]).abs().max() < 0.05 and (d[0, :32] - xo[0, :32]).abs().max() > 0.05
    # NVFP4: finer blocks and E4M3 scales beat MXFP4 at half a bit more
    nv = Q.nvfp4_quantize(x)
    assert nv.packed.shape == (64, 64) and nv.block_scale.dtype == torch.float8_e4m3fn and nv.block_scale.shape == (64, 8)
    env = Q.quantization_error(x, Q.nvfp4_dequantize(nv))["sqnr_db"]
    assert env > e4 and Q.bits_per_element("nvfp4") == 4.5 and Q.bits_per_element("mxfp4") == 4.25
    rep = Q.compare_formats(x)
    assert set(rep) == {"fp8", "mxfp8_e4m3", "mxfp6_e2m3", "mxfp6_e3m2", "mxfp4", "nvfp4"} and rep["mxfp4"]["cosine"] > 0.95
    with pytest.raises(ValueError):
        Q.mx_quantize(torch.randn(4, 30))
    # 2:4 sparsity
    w = torch.randn(8, 32)
    p = Q.prune_2_4(w)
    g = p.reshape(8, 8, 4)
    assert ((g != 0).sum(-1) == 2).all() and torch.equal(g.abs().sum(-1), w.reshape(8, 8, 4).abs().topk(2, -1).values.sum(-1))
    vals, meta = Q.compress_2_4(p)
    assert vals.shape == (8, 16) and meta.shape == (8, 8) and meta.dtype == torch.uint8 and torch.equal(Q.expand_2_4(vals, meta), p)
    sparse_group = torch.tensor([[0.0, 0.0, 0.0, 5.0, 1.0, 0.0, 0.0, 0.0]])
    v2, m2 = Q.compress_2_4(sparse_group)
    assert torch.equal(Q.expand_2_4(v2, m2), sparse_group)
    with pytest.raises(ValueError):
        Q.compress_2_4(w)
    xin = torch.randn(5, 32)
    assert torch.allclose(xin @ Q.expand_2_4(vals, meta).t(), xin @ p.t())


def test_graph_layers_sampling_generators_metrics_and_link_prediction(tmp_path):
    nx = pytest.importorskip("scipy.sparse.csgraph")
    import numpy as np
    import scipy.sparse as sps
    from torsh_b200 import graph as G
    torch.manual_seed(0)
    e = G.erdos_renyi(30, 0.15, seed=1)
    assert (e[0] != e[1]).all() and torch.equal(torch.sort(e[0] * 30 + e[1]).values, torch.sort(e.flip(0)[0] * 30 + e.flip(0)[1]).values)
    x = torch.randn(30, 8)
    # ChebConv with K = 1 is a linear layer; higher orders see neighbours up to K - 1 hops
    c1 = G.ChebConv(8, 4, K=1)
    assert torch.allclose(c1(x, e), c1.lins[0](x) + c1.bias)
    line = torch.tensor([[0, 1, 1, 2, 2, 3], [1, 0, 2, 1, 3, 2]])
    c3 = G.ChebConv(1, 1, K=3)
    xi = torch.zeros(4, 1); xi[0] = 1.0
    base = c3(torch.zeros(4, 1), line)
    resp = (c3(xi, line) - base).abs().flatten()
    assert resp[2] > 0 and resp[3] == 0                                      # two hops reached, three not
    gt = G.GraphTransformerLayer(8, heads=2)
    out = gt(x, e)
    out.sum().backward()
    assert out.shape == (30, 8) and all(p.grad is not None for p in gt.parameters())
    iso = torch.tensor([[0], [1]])                                          # node 1 attends to node 0 only: attention weight 1
    h = gt.n1(x[:2])
    want = x[:2].clone(); want[1] = want[1] + gt.o(gt.v(h)[0])
    want = want + gt.mlp(gt.n2(want))
    assert torch.allclose(gt(x[:2], iso)[1], want[1], atol=1e-5)
    # neighbour sampling: fan-out respected, edges relabelled into the returned node list, seeds first
    ba = G.barabasi_albert(200, 3, seed=0)
    deg = torch.bincount(ba[0], minlength=200)
    assert deg.max() > 4 * deg.float().median() and ba.shape[1] >= 2 * 3 * 190
    ns = G.NeighborSampler(ba, 200, fanouts=[5, 3])
    seeds = torch.tensor([10, 20, 30])
    nodes, layers = ns.sample(seeds)
    assert nodes[:3].tolist() == [10, 20, 30] and len(layers) == 2
    inner = layers[1]
    assert set(inner[1].tolist()) <= {0, 1, 2} and torch.bincount(inner[1]).max() <= 3 and torch.bincount(layers[0][1]).max() <= 5
    have = set((ba[0] * 200 + ba[1]).tolist())
    assert all(int(nodes[u]) * 200 + int(nodes[v]) in have for u, v in layers[0].t().tolist())
    # metrics against scipy / closed forms
    two = torch.cat([G.grid_graph(3, 3), G.grid_graph(2, 2) + 9], 1)
    comp = G.connected_components(two, 13)
    ncomp, ref = nx.connected_components(sps.coo_matrix((np.ones(two.shape[1]), (two[0].numpy(), two[1].numpy())), shape=(13, 13)), directed=False)
    assert int(comp.max()) + 1 == ncomp == 2 and len(set(zip(comp.tolist(), ref.tolist()))) == 2
    assert G.modularity(two, comp) == pytest.approx(1 - ((24 / 32) ** 2 + (8 / 32) ** 2))
    tri = torch.tensor([[0, 1, 1, 2, 2, 0, 2, 3], [1, 0, 2, 1, 0, 2, 3, 2]])
    assert G.clustering_coefficient(tri, 4).tolist() == pytest.approx([1.0, 1.0, 1 / 3, 0.0])
    pr = G.pagerank(ba, 200)
    assert float(pr.sum()) == pytest.approx(1.0) and int(pr.argmax()) == int(deg.argmax())
    star = torch.tensor([[1, 2, 3], [0, 0, 0]])
    ps = G.pagerank(star, 4)
    assert ps[0] > 3 * ps[1] and ps[1] == pytest.approx(float(ps[2]))
    # link prediction on two cliques: embeddings trained with negative sampling separate inside / outside pairs
    k = 6
    a = torch.combinations(torch.arange(k)).t()
    pos = torch.cat([a, a + k], 1)
    pos = torch.cat([pos, pos.flip(0)], 1)
    neg = G.negative_sampling(pos, 2 * k, pos.shape[1], seed=0)
    assert not set((neg[0] * 12 + neg[1]).tolist()) & set((pos[0] * 12 + pos[1]).tolist()) and (neg[0] != neg[1]).all()
    z = torch.nn.Parameter(0.1 * torch.randn(2 * k, 4))
    opt = torch.optim.Adam([z], 0.05)
    for _ in range(200):
        l = G.link_prediction_loss(z, pos, neg)
        opt.zero_grad(); l.backward(); opt.step()
    s_in = (z[0] * z[1]).sum().item(); s_out = (z[0] * z[k]).sum().item()
    assert l < 0.2 and s_in > 1 > s_out
    (tmp_path / "c.content").write_text("p1 1 0 1 ml\np2 0 1 1 db\np3 1 1 0 ml\n")
    (tmp_path / "c.cites").write_text("p1 p2\np3 p1\np9 p1\n")
    gd = G.load_planetoid_like(tmp_path / "c.content", tmp_path / "c.cites")
    assert gd.x.shape == (3, 3) and gd.y.tolist() == [1, 0, 1] and gd.num_edges == 4


def test_cluster_hierarchy_optics_streaming_drift_and_evaluation():
    sk = pytest.importorskip("sklearn")
    import numpy as np
    from scipy.cluster import hierarchy as sch
    from sklearn import metrics as skm
    from sklearn.cluster import OPTICS as SkOptics
    from torsh_b200 import cluster as C
    torch.manual_seed(0)
    cen = torch.tensor([[0.0, 0.0], [6.0, 0.0], [0.0, 6.0]])
    x = torch.cat([c + 0.5 * torch.randn(40, 2) for c in cen])
    truth = torch.arange(3).repeat_interleave(40)
    # merge distances equal scipy's for each linkage; flat cuts recover the blobs
    for m in ("single", "complete", "average", "ward"):
        r = C.linkage(x, m)
        ref = sch.linkage(x.double().numpy(), m)
        assert np.allclose(sorted(s[2] for s in r.steps), np.sort(ref[:, 2]), rtol=1e-6), m
        assert C.adjusted_rand_index(r.flat_clusters(3), truth) == pytest.approx(1.0)
    assert int(r.clusters_by_distance(15.0).max()) + 1 == 3 and int(r.flat_clusters(1).max()) == 0
    assert C.AgglomerativeClustering(3).fit(x).labels.unique().numel() == 3
    with pytest.raises(ValueError):
        C.linkage(x, "centroidal")
    # OPTICS: core distances and the multiset of reachabilities match scikit-learn; eps cut finds the blobs
    o = C.OPTICS(min_samples=5).fit(x)
    so = SkOptics(min_samples=5, metric="euclidean").fit(x.double().numpy())
    assert np.allclose(o.core_distances.numpy(), so.core_distances_, rtol=1e-6)
    fin = torch.isfinite(o.reachability)
    assert fin.sum() == len(x) - 1
    same = np.isclose(o.reachability.numpy(), so.reachability_, rtol=1e-6)        # ties in the queue may resolve differently
    assert same.mean() > 0.97 and o.ordering[:6].tolist() == so.ordering_[:6].tolist()
    assert C.adjusted_rand_index(o.extract_dbscan(1.0), truth) > 0.95
    # streaming k-means follows the data; window k-means re-fits on schedule
    perm = torch.randperm(len(x))
    ok = C.OnlineKMeans(3)
    ok.centers, ok.counts = cen + 1.0, torch.ones(3)
    ok.partial_fit(x[perm])
    assert torch.cdist(ok.centers, cen).min(1).values.max() < 0.4 and C.adjusted_rand_index(ok.predict(x), truth) == pytest.approx(1.0)
    sw = C.SlidingWindowKMeans(3, window_size=60, recompute_frequency=30)
    for i in range(0, 120, 15):
        sw.partial_fit(x[perm][i:i + 15])
    assert sw.n_refits == 4 and len(sw.window) == 60 and sw.centers.shape == (3, 2)
    # drift detectors: quiet on a stationary stream, fire after a mean shift
    g = torch.Generator().manual_seed(1)
    stream = torch.cat([torch.randn(300, generator=g) * 0.1, 2 + torch.randn(100, generator=g) * 0.1]).tolist()
    for det in (C.PageHinkley(lam=5.0), C.ADWIN(delta=0.002, max_window_size=400)):
        st = [det.update(v) for v in stream]
        assert C.DRIFT not in st[:300] and C.DRIFT in st[300:], type(det).__name__
    ddm = C.DDM()
    errs = (torch.rand(400, generator=g) < torch.cat([torch.full((250,), 0.1), torch.full((150,), 0.6)])).float().tolist()
    st = [ddm.update(e) for e in errs]
    assert C.DRIFT not in st[:250] and C.DRIFT in st[250:]
    comp = C.CompositeDriftDetector()
    assert C.DRIFT in [comp.update(v) for v in stream]
    # initialisation, scaling and parameter suggestion
    for init in (C.init_forgy, C.init_random_partition, C.init_kmeans_plus_plus):
        assert init(x, 3, seed=0).shape == (3, 2)
    assert torch.cdist(C.init_kmeans_plus_plus(x, 3), cen).min(0).values.max() < 2.0
    s = C.standardize_features(x)
    assert torch.allclose(s.mean(0), torch.zeros(2), atol=1e-5) and torch.allclose(s.std(0, unbiased=False), torch.ones(2), atol=1e-5)
    assert C.normalize_features(x).min() == 0 and C.normalize_features(x).max() == 1
    assert torch.allclose(C.unit_normalize(x).norm(dim=1), torch.ones(len(x)))
    assert torch.allclose(C.robust_scale(x).median(0).values, torch.zeros(2), atol=0.05)
    eps, ms = C.suggest_dbscan_params(x)
    assert 0.1 < eps < 2.0 and C.adjusted_rand_index(C.dbscan(x, eps, ms).clamp(min=0), truth) > 0.9
    assert torch.allclose(C.pairwise_distance(x[:3], x[:3], "cosine").diagonal(), torch.zeros(3), atol=1e-6)
    with pytest.raises(ValueError):
        C.validate_cluster_input(torch.tensor([[float("nan"), 1.0]]))
    # evaluation against scikit-learn
    pred = truth.clone(); pred[::7] = (pred[::7] + 1) % 3; pred[5:20] = 3
    t, p = truth.numpy(), pred.numpy()
    assert C.normalized_mutual_info(truth, pred) == pytest.approx(skm.normalized_mutual_info_score(t, p))
    assert C.adjusted_mutual_info(truth, pred) == pytest.approx(skm.adjusted_mutual_info_score(t, p), abs=1e-9)
    assert C.homogeneity_completeness_v_measure(truth, pred) == pytest.approx(skm.homogeneity_completeness_v_measure(t, p))
    assert C.fowlkes_mallows(truth, pred) == pytest.approx(skm.fowlkes_mallows_score(t, p))
    assert C.rand_index(truth, pred) == pytest.approx(skm.rand_score(t, p))
    assert C.mutual_information(truth, pred) == pytest.approx(skm.mutual_info_score(t, p))
    assert C.calinski_harabasz(x, pred) == pytest.approx(skm.calinski_harabasz_score(x.numpy(), p), rel=1e-4)
    assert C.purity(truth, truth) == 1.0 and 0 < C.jaccard_index(truth, pred) < 1 and C.dunn_index(x, truth) > C.dunn_index(x, pred)
    assert C.gap_statistic(x, k_max=5, n_refs=5)[0] == 3


def test_fx_tools_codegen_analysis_rewrite_shapes_editor_memory_placement_quant_nas(tmp_path):
    import ctypes
    import subprocess
    import numpy as np
    from torsh_b200 import fx as tfx_, fx_tools as T
    torch.manual_seed(0)

    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.act, self.b = torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4)
            self.register_buffer("shift", torch.randn(4))

        def forward(self, x):
            h = self.act(self.a(x))
            return torch.tanh(self.b(h)) + self.shift

    m = MLP().eval()
    gm = tfx_.symbolic_trace(m)
    x = torch.randn(5, 8)
    want = m(x)
    # generated Python and NumPy source reproduce the module; C++ (plain loops) compiles and does too
    py = T.PythonCodeGen(True).generate(gm)
    assert "def forward(consts, x)" in py.source and torch.allclose(py.load()(x), want, atol=1e-6)
    npc = T.PythonCodeGen(False).generate(gm)
    assert "import numpy as np" in npc.source and np.allclose(npc.load()(x.numpy()), want.detach().numpy(), atol=1e-5)
    assert "torch::linear" in T.CppCodeGen(True).generate(gm).source
    tfx_.ShapeProp(gm).run(x)
    cpp = T.CppCodeGen(False).generate(gm)
    (tmp_path / "g.cpp").write_text(cpp.source)
    subprocess.run(["g++", "-O1", "-shared", "-fPIC", str(tmp_path / "g.cpp"), "-o", str(tmp_path / "g.so")], check=True)
    lib = ctypes.CDLL(str(tmp_path / "g.so"))
    cs = [c.numpy() for c in cpp.constants.values()]
    arr = (ctypes.c_void_p * len(cs))(*[c.ctypes.data for c in cs])
    out = np.zeros((5, 4), np.float32)
    xin = x.numpy().copy()
    lib.forward(arr, ctypes.c_void_p(xin.ctypes.data), ctypes.c_void_p(out.ctypes.data))
    assert np.allclose(out, want.detach().numpy(), atol=1e-5)
    lc = T.LazyCompiler()
    assert lc.compile(gm) is lc.compile(gm) and lc.cache_stats() == {"entries": 1, "hits": 1, "misses": 1}
    # metrics, lint, patterns, diff
    def messy(x, y):
        a = x + 0
        b = torch.relu(x * y)
        c = torch.relu(x * y)
        unused = x - y
        return (a + b + c).reshape(-1).reshape(2, -1)
    g2 = tfx_.symbolic_trace(messy)
    rules = {i.rule for i in T.GraphLinter().lint_graph(g2)}
    assert {"unused-value", "noop-arithmetic", "duplicate-computation", "reshape-chain"} <= rules
    assert {i.rule for i in T.GraphLinter("error").lint_graph(g2)} == set()
    mt = T.calculate_graph_metrics(gm)
    assert mt["compute_nodes"] == 5 and mt["depth"] == 7 and mt["max_width"] == 1

    class Res(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.n, self.l = torch.nn.LayerNorm(8), torch.nn.Linear(8, 8)

        def forward(self, x, k):
            h = x + torch.relu(self.l(self.n(x)))
            return torch.matmul(torch.softmax(torch.matmul(h, k.transpose(0, 1)) / 2.0, -1), k)
    pats = {p["pattern"] for p in T.detect_patterns(tfx_.symbolic_trace(Res()))}
    assert {"residual", "norm+linear", "linear+activation", "attention"} <= pats
    import copy
    ed = T.GraphEditor(copy.deepcopy(gm))
    before = copy.deepcopy(ed.gm)
    ed.insert_after("a", torch.neg)
    assert torch.allclose(ed.gm(x), torch.tanh(m.b(torch.relu(-m.a(x)))) + m.shift, atol=1e-6)
    d = T.graph_diff(before, ed.gm)
    assert d["added"] == ["neg"] and d["changed"] == ["act"] and not d["identical"]
    ed.remove("neg")
    assert torch.allclose(ed.gm(x), want)
    assert ed.undo() and "neg" in {n.name for n in ed.gm.graph.nodes} and ed.undo() and torch.allclose(ed.gm(x), want)
    assert ed.redo() and "neg" in ed.export_graph("json") and not T.GraphEditor(gm).undo()
    # rewriting: conv+bn fold is exact in eval mode, conv+relu becomes one node, user pattern replaced
    net = torch.nn.Sequential(torch.nn.Conv2d(3, 6, 3, padding=1, bias=False), torch.nn.BatchNorm2d(6), torch.nn.ReLU(), torch.nn.Conv2d(6, 2, 1)).eval()
    net[1].running_mean.normal_(); net[1].running_var.uniform_(0.5, 2.0); net[1].weight.data.normal_(); net[1].bias.data.normal_()
    img = torch.randn(2, 3, 8, 8)
    ref = net(img)
    gn = tfx_.symbolic_trace(net)
    rw = T.SubgraphRewriter().with_common_fusions().add_pattern(lambda v: torch.neg(torch.neg(v)), lambda v: v)
    rep = rw.apply(gn)
    assert rep["fold_conv_bn"] == 1 and rep["fuse_module_activation"] == 1 and torch.allclose(gn(img), ref, atol=1e-5)
    assert sum(n.op == "call_module" for n in gn.graph.nodes) == 2
    gdn = tfx_.symbolic_trace(lambda v: torch.neg(torch.neg(v)) * 2)
    assert rw.find_matches(gdn, lambda v: torch.neg(torch.neg(v))) == 1 and T.SubgraphRewriter().add_pattern(lambda v: torch.neg(torch.neg(v)), lambda v: v).apply(gdn)["<lambda>"] == 1
    assert torch.equal(gdn(x), x * 2)
    # dynamic shapes
    B, S = T.DynamicDim.symbolic("B"), T.DynamicDim.symbolic("S")
    assert repr(T.broadcast_dynamic_shapes(T.DynamicShape([B, 1, 8]), T.DynamicShape([S, 8]))) == "[B, S, 8]"
    assert repr(T.matmul_dynamic_shape(T.DynamicShape(["B", "S", 8]), T.DynamicShape([8, 32]))) == "[B, S, 32]"
    with pytest.raises(ValueError):
        T.matmul_dynamic_shape(T.DynamicShape(["B", 8]), T.DynamicShape([9, 2]))
    ctx = T.DynamicShapeContext()
    ctx.register_symbol("B", min=1, max=64)
    ctx.register_symbol("S", multiple_of=8)
    ctx.infer(gm, {"x": T.DynamicShape(["B", "S", 8])})
    assert repr(ctx.get_shape("add")) == "[B, S, 4]" and ctx.get_unresolved_symbols({"B": 2}) == ["S"]
    assert ctx.resolve_symbols({"B": 2, "S": 16})["add"] == (2, 16, 4)
    assert len(ctx.validate_constraints({"B": 128, "S": 12})) == 2
    with pytest.raises(ValueError):
        T.DynamicShape(["B", 3]).to_static_shape()
    # checkpoints and resumable execution
    digest = T.save_graph_checkpoint(gm, tmp_path / "g.pt", {"note": "mlp"})
    g3, meta = T.load_graph_checkpoint(tmp_path / "g.pt")
    assert len(digest) == 64 and meta == {"note": "mlp"} and torch.equal(g3(x), want)
    ri = T.ResumableInterpreter(gm)
    assert ri.run(x, stop_after="act") is None and ri.saved["at"] == "act"
    saved = ri.saved
    assert torch.equal(ri.run(x, resume=saved), want) and "a" not in ri.executed and ri.executed[0] == "b"
    # memory: peak from liveness, reuse plan smaller than the sum of intermediates
    chain = tfx_.symbolic_trace(torch.nn.Sequential(*[torch.nn.Linear(32, 32) for _ in range(6)]))
    rep = T.MemoryAnalyzer(chain).analyze(torch.randn(64, 32))
    one = 64 * 32 * 4
    assert rep["peak_bytes"] == 2 * one and rep["total_intermediate_bytes"] == 6 * one and rep["planned_bytes"] == 2 * one and rep["buffers"] == 2
    # placement: big matmuls go to the fast device, tiny graphs stay where the input is
    devs = [T.DeviceCapability("cpu", 1e11, 5e10, 64e9), T.DeviceCapability("b200", 1e15, 6e12, 180e9)]
    big = tfx_.symbolic_trace(torch.nn.Sequential(torch.nn.Linear(512, 512), torch.nn.ReLU(), torch.nn.Linear(512, 512)))
    plan = T.HeterogeneousPlanner(devs).plan_execution(big, torch.randn(256, 512))
    assert set(plan["placement"].values()) == {"b200"} and len(plan["transfers"]) == 1
    tiny = tfx_.symbolic_trace(lambda v: torch.relu(v) + 1)
    assert set(T.HeterogeneousPlanner(devs).plan_execution(tiny, torch.randn(4))["placement"].values()) == {"cpu"}
    reg = T.BackendRegistry()
    name, out = reg.execute_with_auto_backend(gm, x, require={"source"})
    assert name == "generated-python" and torch.allclose(out, want, atol=1e-6) and "interpreter" in reg.find_backends_with_capability("debug")
    reg.register("broken", lambda gm, *a: 1 / 0, {"special", "debug"})
    with pytest.raises(RuntimeError):
        reg.execute_with_auto_backend(gm, x, require={"special"})
    gc = T.GraphCache()
    assert gc.run(gm, x) is gc.run(gm, x) and gc.statistics()["hits"] == 1 and gc.run(gm, x + 1) is not None and gc.statistics()["misses"] == 2
    # quantisation passes: PTQ error is small but non-zero; QAT ranges receive gradients
    prep = T.prepare_ptq(gm)
    with pytest.raises(RuntimeError):
        T.convert_ptq(prep)
    for _ in range(4):
        prep(torch.randn(32, 8))
    q8, q4 = T.convert_ptq(prep, 8), T.convert_ptq(prep, 4)
    e8, e4 = T.quantization_error(gm, q8, x), T.quantization_error(gm, q4, x)
    assert 0 < e8["mse"] < e4["mse"] and e8["sqnr_db"] > 25 > e4["sqnr_db"]
    qat = T.prepare_qat(gm, torch.randn(32, 8))
    qat(x).sum().backward()
    ranges = [p for n, p in qat.named_parameters() if n.endswith("range")]
    assert len(ranges) == 6 and all(p.grad is not None for p in ranges) and qat.a.weight.grad.abs().sum() > 0
    # architecture search improves on the initial population and avoids the "zero" op on a learnable target
    xs = torch.randn(128, 4)
    ys = torch.tanh(xs @ torch.randn(4, 2))
    nas = T.ArchitectureSearch(4, 2, dim=8, depth=2, seed=0)
    best, fit = nas.search((xs[:96], ys[:96]), (xs[96:], ys[96:]), population=6, generations=2, steps=40)
    assert nas.history[-1] <= nas.history[0] and fit < 0.1 and not all(g["op"] == "zero" and not g["skip"] for g in best)


def test_package_operations_delta_backup_mirrors_replication_security_governance(tmp_path):
    import json
    import os
    from torsh_b200 import package_ops as P
    from torsh_b200.hub import Package
    rng = __import__("random").Random(0)
    blob = bytes(rng.randrange(256) for _ in range(20000))
    v1 = Package("demo", "1.0.0", {"numlib": "1.2.0"})
    v1.add_bytes("weights.bin", blob)
    v1.add_bytes("notes.txt", b"first release\n" * 50)
    v1.add_source("model", "def f(x):\n    return x + 1\n")
    v1.add_model(torch.nn.Linear(3, 2))
    v2 = Package("demo", "1.1.0", {"numlib": "1.3.0"})
    v2.files = dict(v1.files)
    v2.files["weights.bin"] = blob[:7000] + b"PATCHED" + blob[7100:] + b"tail"
    v2.files["new.txt"] = b"added"
    del v2.files["notes.txt"]
    patch = P.create_patch(v1, v2)
    kinds = {op[1]: op[0] for op in patch.operations}
    assert kinds == {"notes.txt": "delete", "new.txt": "add", "weights.bin": "modify"} and patch.size() < 1500
    patch.save(tmp_path / "p.delta")
    back = P.apply_patch(v1, P.DeltaPatch.load(tmp_path / "p.delta"))
    assert back.files == v2.files and back.version == "1.1.0" and back.dependencies == {"numlib": "1.3.0"}
    with pytest.raises(ValueError):
        P.apply_patch(v2, patch)
    patch.operations = [op for op in patch.operations if op[0] != "add"]
    with pytest.raises(IOError):
        P.apply_patch(v1, patch)
    v3 = Package("demo", "1.2.0"); v3.files = dict(v2.files); v3.files["weights.bin"] = bytes(rng.randrange(256) for _ in range(20000))
    assert {op[1]: op[0] for op in P.create_patch(v2, v3).operations}["weights.bin"] == "replace"
    # compression, optimisation, diagnostics
    comp = P.AdvancedCompressor()
    assert comp.algorithm_for_resource("weights.bin", blob) == "none" and comp.algorithm_for_resource("a.txt", b"abc" * 5000) != "none"
    algo, out = comp.compress_resource("a.txt", b"abc" * 5000)
    assert P.decompress_data(out, algo) == b"abc" * 5000 and comp.overall_ratio() < 0.05 and comp.space_saved() > 14000
    assert set(P.AdvancedCompressor.benchmark_algorithms(b"hello world " * 400)) == {"zlib", "bz2", "lzma"}
    v1.add_bytes("copy_of_weights.bin", blob)
    rep = P.PackageOptimizer().analyze(v1)
    assert rep["duplicate_groups"] == [["copy_of_weights.bin", "weights.bin"]] or rep["duplicate_groups"] == [["weights.bin", "copy_of_weights.bin"]]
    assert rep["duplicate_bytes"] == 20000 and "notes.txt" in rep["compressible"]
    slim, aliases = P.PackageOptimizer().optimize(v1)
    assert aliases == {"weights.bin": "copy_of_weights.bin"} and P.resolve_alias(slim, "weights.bin") == blob
    assert P.diagnose(v1)["health"] == "healthy"
    bad = Package("bad name!", "one"); bad.add_source("m", "def (:"); bad.add_bytes("../evil", b"x")
    d = P.diagnose(bad)
    assert d["health"] == "broken" and {i["category"] for i in d["issues"]} >= {"manifest", "code", "security"}
    # lazy resources under a memory budget
    v1.save(tmp_path / "demo.zip")
    lz = P.LazyResourceManager(tmp_path / "demo.zip", memory_limit=25000)
    assert lz.get_resource("weights.bin") == blob and lz.get_resource("weights.bin") is lz.get_resource("weights.bin") and lz.loads == 1
    lz.get_resource("copy_of_weights.bin")
    assert not lz.is_loaded("weights.bin") and lz.memory_usage() <= 25000
    assert b"".join(lz.stream("notes.txt", 64)) == v1.files["notes.txt"]
    # audit chain and metrics
    log = P.AuditLogger(tmp_path / "audit.jsonl")
    seen = []
    log.add_listener(seen.append)
    log.log_upload("demo-1.0.0", "ann"); log.log_download("demo-1.0.0", "bob"); log.log_access_denied("demo-1.0.0", "eve")
    log.log_security_violation("demo-1.0.0", "bad signature")
    assert log.validate() == [] and len(seen) == 4 and len(log.query(user="eve")) == 1 and log.get_statistics()["denied"] == 1
    again = P.AuditLogger(tmp_path / "audit.jsonl")
    assert again.validate() == [] and len(again.events) == 4
    again.events[1]["user"] = "mallory"
    assert again.validate() == [1]
    del again.events[1]
    assert again.validate()[0] == 1
    mc = P.MetricsCollector()
    mc.set_alert_threshold("error_rate", 0.3)
    for _ in range(3):
        mc.record_download("demo", "bob", 100)
    mc.record_error("demo"); mc.record_error("demo")
    assert mc.get_package_stats("demo")["downloads"] == 3 and mc.get_active_alerts()[0]["metric"] == "error_rate"
    assert mc.get_time_series("downloads")["count"] == 3 and mc.generate_report()["top_packages"] == ["demo"]
    # storage, backups with an incremental chain and retention
    st = P.LocalStorage(tmp_path / "store")
    st.put("a/b.bin", b"123")
    assert st.get("a/b.bin") == b"123" and st.list("a/") == ["a/b.bin"] and st.get_metadata("a/b.bin")["size"] == 3
    with pytest.raises(PermissionError):
        st.put("../out.bin", b"x")
    bm = P.BackupManager(st, "incremental")
    b1 = bm.create_backup(v1, now=0.0)
    b2 = bm.create_backup(v2, now=86400.0 * 10)
    assert b2["parent"] == b1["id"] and b2["stored_files"] == ["new.txt", "weights.bin"]
    assert bm.restore_backup(b2["id"]).files == v2.files and bm.restore_backup(b1["id"]).files == v1.files
    assert bm.apply_retention_policy(keep_last=1, now=86400.0 * 10) == [] and len(bm.list_backups("demo")) == 2    # parent is still needed
    assert P.BackupManager(st).list_backups()[1]["id"] == b2["id"]
    st.put(f"backups/{b1['id']}.bin", b"garbage")
    assert not bm.verify_backup(b1["id"])["valid"]
    with pytest.raises(IOError):
        bm.restore_backup(b2["id"])
    full = P.BackupManager(P.MemoryStorage(), "full")
    ids = [full.create_backup(v1, now=86400.0 * i)["id"] for i in range(4)]
    assert full.apply_retention_policy(keep_days=1.5, now=86400.0 * 3) == ids[:2] and len(full.list_backups()) == 2
    # mirrors: fail-over and health
    class Flaky(P.MemoryStorage):
        def get(self, key): raise IOError("down")
    good, flaky = P.MemoryStorage(), Flaky()
    good.put("demo.zip", b"pkg")
    mm = P.MirrorManager("priority", max_failures=2)
    mm.add_mirror(P.Mirror("flaky", flaky, priority=10)); mm.add_mirror(P.Mirror("good", good, priority=1))
    assert mm.select_mirror().name == "flaky" and mm.fetch("demo.zip") == ("good", b"pkg") and mm.fetch("demo.zip")[0] == "good"
    assert mm.mirrors["flaky"].health == "unhealthy" and mm.failovers == 1 and mm.select_mirror().name == "good"
    good.delete("demo.zip")
    with pytest.raises(IOError):
        mm.fetch("demo.zip")                                                   # good fails, flaky is the last resort and fails again
    assert mm.mirrors["flaky"].health == "offline" and mm.mirrors["flaky"].requests == 2
    good.put("demo.zip", b"pkg")
    third = P.MemoryStorage()
    mm.add_mirror(P.Mirror("third", third))
    assert mm.sync(good) == {"flaky": 1, "third": 1} and third.get("demo.zip") == b"pkg"
    # replication: quorum commit, stale replica repaired, conflict settled
    rm = P.ReplicationManager("quorum")
    for n in "abc":
        rm.add_node(n, P.MemoryStorage())
    assert rm.replicate_package("demo", b"v1", now=1.0)["status"] == "committed"
    rm.set_online("c", False)
    r2 = rm.replicate_package("demo", b"v2", now=2.0)
    assert r2["status"] == "committed" and r2["acks"] == ["a", "b"] and r2["version"] == 2
    rm.set_online("b", False)
    assert rm.replicate_package("demo", b"v3", now=3.0)["status"] == "failed"
    rm.set_online("b", True); rm.set_online("c", True)
    assert rm.get_package("demo") == b"v3"
    assert sorted(rm.synchronize("demo")["repaired"]) == ["b", "c"] and rm.synchronize("demo") == {"repaired": [], "conflicts": 0}
    rec = json.loads(rm.nodes["a"]["storage"].get("demo")); rec.update(data=b"fork".hex(), sha256=P._sha(b"fork"), time=9.0)
    rm.nodes["a"]["storage"].put("demo", json.dumps(rec).encode())
    assert rm.synchronize("demo")["conflicts"] == 1 and rm.get_package("demo") == b"fork" and len(rm.conflicts) == 1
    # vulnerability scan and sandbox
    risky = Package("risky", "0.1.0", {"numlib": "1.2.0", "safe": "2.0.0"})
    risky.add_source("m", "import os, pickle\napi_key = 'sk-1234567890'\ndef run(c):\n    os.system(c)\n    return eval(c)\n")
    risky.add_bytes("state.pkl", b"\x80\x04N.")
    adv = [{"package": "numlib", "affected": ">=1.0.0,<1.2.5", "id": "ADV-1", "severity": "critical"}, {"package": "safe", "affected": "<1.0.0", "id": "ADV-2"}]
    rep = P.VulnerabilityScanner("standard", adv).scan(risky)
    assert {i["type"] for i in rep["issues"]} == {"risky_call", "embedded_secret", "pickled_payload", "vulnerable_dependency"}
    assert rep["critical"] == 2 and not rep["passed"] and rep["risk_score"] > 40 and P.VulnerabilityScanner().scan(v2)["passed"]
    assert len(P.VulnerabilityScanner("lenient", adv).scan(risky)["issues"]) <= len(P.VulnerabilityScanner("strict", adv).scan(risky)["issues"])
    (tmp_path / "ok").mkdir(); (tmp_path / "ok" / "in.txt").write_text("41")
    sb = P.Sandbox(read_paths=[tmp_path / "ok"])
    src = "import math\ndef go(p):\n    return int(open(p).read()) + int(math.sqrt(1))\n"
    assert sb.execute(src, "go", str(tmp_path / "ok" / "in.txt"))["value"] == 42
    for bad_src, kind in (("import os\n", "import"), ("open('/etc/hostname').read()\n", "file_read"), (f"open({str(tmp_path / 'ok' / 'x')!r}, 'w')\n", "file_write"),
                          ("while True:\n    pass\n", "cpu_budget")):
        box = P.Sandbox(read_paths=[tmp_path / "ok"], max_lines=10000)
        with pytest.raises(P.SandboxViolation):
            box.execute(bad_src)
        assert box.violations[0]["type"] == kind
    with pytest.raises(NameError):
        P.Sandbox().execute("eval('1')\n")
    assert P.Sandbox().execute_package_module(v1, "model", "f", 2)["value"] == 3
    # lineage and compliance
    lt = P.LineageTracker()
    lt.add_lineage("ft-1", "base-1", "fine_tuned_from", dataset="d1")
    lt.add_lineage("q-1", "ft-1", "quantized_from")
    with pytest.raises(ValueError):
        lt.add_lineage("base-1", "q-1")
    assert lt.get_ancestors("q-1") == ["ft-1", "base-1"] and lt.get_descendants("base-1") == ["ft-1", "q-1"]
    lt.set_compliance("base-1", "Apache-2.0", pii=True); lt.set_compliance("ft-1", "MIT"); lt.set_compliance("q-1", "proprietary")
    lt.record_provenance("q-1", "ci", "ann"); lt.record_transformation("q-1", "int8", bits=8)
    cr = lt.generate_compliance_report("q-1")
    assert not cr["compliant"] and sum(i["severity"] == "error" for i in cr["issues"]) == 2
    lt.set_compliance("q-1", "MIT", pii=True)
    assert lt.generate_compliance_report("q-1")["compliant"] and '"base-1" -> "ft-1"' in lt.export_to_dot() and lt.get_statistics()["roots"] == ["base-1"]
    # other layouts round-trip the tensors
    fm = P.FormatCompatibilityManager()
    from torsh_b200.serialize import model_state as ms
    want = ms.decode_binary(v1.files["model.trsm"])["parameters"]
    for fmt in fm.supported_formats:
        out = fm.export_package(v1, fmt, tmp_path / f"exp_{fmt}")
        got = ms.decode_binary(fm.import_package(out, fmt).files["model.trsm"])["parameters"]
        assert {k: (v["shape"], v["data"]) for k, v in got.items()} == {k: (v["shape"], v["data"]) for k, v in want.items()}, fmt
    assert "numlib==1.2.0" in (tmp_path / "exp_mlflow" / "requirements.txt").read_text()


def test_advanced_optimizers_continual_dp_online_composition_and_analysis():
    import math
    import numpy as np
    from torsh_b200.optim import advanced as A
    torch.manual_seed(0)
    # continual learning: task B pulls the weights task A needs toward zero; a penalty on what mattered for A resists it
    xa, xb = torch.randn(64, 4), torch.randn(64, 4)
    xa[:, 2:] = 0
    xb[:, :2] *= 0.3
    ya, yb = xa @ torch.tensor([[1.0], [-1.0], [0.0], [0.0]]), xb[:, 2:] @ torch.tensor([[2.0], [1.0]])
    mse = torch.nn.functional.mse_loss
    def train(m, opt, x, y, n=150):
        for _ in range(n):
            opt.zero_grad(); mse(m(x), y).backward(); opt.step()
    forgetting = {}
    for kind in ("none", "ewc", "mas", "si"):
        torch.manual_seed(1)
        m = torch.nn.Linear(4, 1, bias=False)
        base = torch.optim.SGD(m.parameters(), 0.1)
        opt = {"none": base, "ewc": A.EWCOptimizer(base, 5.0), "mas": A.MASOptimizer(base, 2.0), "si": A.SIOptimizer(base, 5.0)}[kind]
        train(m, opt, xa, ya)
        if kind == "ewc":                                                    # per-sample gradients of noisy labels: the empirical Fisher
            opt.consolidate(m, [(xa[i:i + 1], ya[i:i + 1] + 0.5 * torch.randn(1, 1)) for i in range(64)], mse)
            assert opt.importance[0][0, :2].min() > 0.3 and opt.importance[0][0, 2:].abs().max() == 0
        elif kind == "mas":
            opt.consolidate(m, [xa])
        elif kind == "si":
            opt.consolidate()
        train(m, opt, xb, yb)
        forgetting[kind] = float(mse(m(xa), ya).detach())
        assert float(mse(m(xb), yb).detach()) < 0.2, kind                            # task B is still learned
    assert forgetting["none"] > 0.5 and all(forgetting[k] < 0.3 * forgetting["none"] for k in ("ewc", "mas", "si")), forgetting
    assert float(opt.penalty().detach()) > 0
    # differential privacy: clipping bounds each sample, accountant grows with steps and shrinks with noise
    m = torch.nn.Linear(4, 1)
    x, y = torch.randn(16, 4), torch.randn(16, 1)
    psg = A.per_sample_gradients(m, mse, x, y)
    mse(m(x), y).backward()
    assert torch.allclose(psg[0].mean(0), m.weight.grad, atol=1e-5) and psg[0].shape == (16, 1, 4)
    dp = A.DPOptimizer(torch.optim.SGD(m.parameters(), 0.1), noise_multiplier=0.0, max_grad_norm=0.01, sample_rate=0.1, seed=0)
    w0 = m.weight.detach().clone(); b0 = m.bias.detach().clone()
    dp.step(psg)
    moved = math.sqrt(float((m.weight.detach() - w0).pow(2).sum() + (m.bias.detach() - b0).pow(2).sum()))
    assert moved <= 0.1 * 0.01 + 1e-7 and dp.clipped_fraction == 1.0
    acc1, acc2 = A.RDPAccountant(), A.RDPAccountant()
    acc1.step(0.01, 1.1, 1000); acc2.step(0.01, 2.0, 1000)
    e1, e2 = acc1.get_epsilon(1e-5), acc2.get_epsilon(1e-5)
    assert 0.5 < e1 < 3.0 and e2 < e1 and A.RDPAccountant().get_epsilon(1e-5) > 0
    full = A.RDPAccountant(); full.step(1.0, 1.0, 1)
    assert full.rdp[0] == pytest.approx(2 / 2.0)                             # alpha / (2 sigma^2) at alpha = 2 without sampling
    # online and proximal methods
    w = torch.nn.Parameter(torch.tensor([3.0, -3.0]))
    ogd = A.OnlineGradientDescent([w], lr=1.0, radius=1.0)
    for _ in range(50):
        loss = ((w - torch.tensor([0.5, 0.2])) ** 2).sum()
        ogd.zero_grad(); loss.backward(); ogd.step(loss.item())
    assert float(w.detach().norm()) <= 1.0 + 1e-6 and torch.allclose(w.detach(), torch.tensor([0.5, 0.2]), atol=0.05) and ogd.regret(0.0) > 0
    xs = torch.randn(100, 10)
    true = torch.zeros(10); true[[1, 4]] = torch.tensor([2.0, -3.0])
    ys = xs @ true
    for accel in (False, True):
        w = torch.nn.Parameter(torch.zeros(10))
        pg = A.ProximalGradient([w], lr=0.05, prox=A.prox_l1, reg=0.1, accelerated=accel)
        for _ in range(200):
            pg.zero_grad(); (0.5 * ((xs @ w - ys) ** 2).mean()).backward(); pg.step()
        assert int((w.detach().abs() > 1e-6).sum()) == 2 and torch.allclose(w.detach()[[1, 4]], torch.tensor([2.0, -3.0]), atol=0.25)
    assert torch.equal(A.prox_box(-1, 1)(torch.tensor([-3.0, 0.5]), 0.1), torch.tensor([-1.0, 0.5]))
    assert A.prox_group_lasso(torch.tensor([[0.1, 0.1], [3.0, 4.0]]), 1.0)[0].abs().sum() == 0
    # SVRG and SAGA reach the least-squares solution with a constant step where plain SGD keeps jittering
    sol = torch.linalg.lstsq(xs, (ys + 0.5 * torch.randn(100))[:, None]).solution.squeeze()
    yn = None
    torch.manual_seed(2)
    yn = xs @ true + 0.5 * torch.randn(100)
    sol = torch.linalg.lstsq(xs, yn[:, None]).solution.squeeze()
    gfn = lambda ps, idx: [(xs[idx] * (xs[idx] @ ps[0] - yn[idx])[:, None]).mean(0)]
    w = torch.zeros(10)
    sv = A.SVRG([w], gfn, 100, lr=0.05)
    for ep in range(30):
        sv.snapshot()
        for i in torch.randperm(100).tolist():
            sv.step(torch.tensor([i]))
    assert float((w - sol).norm()) < 1e-3
    w2 = torch.zeros(10)
    sg = A.SAGA([w2], gfn, 100, lr=0.03)
    for ep in range(60):
        for i in torch.randperm(100).tolist():
            sg.step(i)
    assert float((w2 - sol).norm()) < 1e-2
    # composition
    def quad_run(make, steps=60):
        p = torch.nn.Parameter(torch.tensor([2.0, -1.5]))
        o = make([p])
        for _ in range(steps):
            l = (p ** 2).sum()
            o.zero_grad(); l.backward(); o.step(l.item()) if isinstance(o, A.ComposedOptimizer) else o.step()
        return p, o
    p, o = quad_run(lambda ps: A.ComposedOptimizer([torch.optim.Adam(ps, 0.1), torch.optim.SGD(ps, 0.1)], "sequential", phases=[20, 40]))
    assert o.active == 1 and float(p.detach().norm()) < 0.05
    p, o = quad_run(lambda ps: A.ComposedOptimizer([torch.optim.SGD(ps, 1e-4), torch.optim.SGD(ps, 0.2)], "switch", criterion=lambda h: len(h) >= 5))
    assert o.switches == [5] and float(p.detach().norm()) < 1e-3
    p, o = quad_run(lambda ps: A.ComposedOptimizer([torch.optim.SGD(ps, 0.1), torch.optim.SGD(ps, 0.3)], "average"), steps=1)
    assert torch.allclose(p.detach(), torch.tensor([2.0, -1.5]) * (1 - 2 * 0.2))
    p, o = quad_run(lambda ps: A.ComposedOptimizer([torch.optim.SGD(ps, 0.1), torch.optim.SGD(ps, 0.2), torch.optim.SGD(ps, 0.1, maximize=True)], "vote"), steps=1)
    assert torch.allclose(p.detach(), torch.tensor([2.0, -1.5]) * (1 - 2 * 0.1))
    assert A.plateau_criterion(3, 0.0)([5, 4, 3, 3, 3, 3]) and not A.plateau_criterion(3, 0.0)([5, 4, 3, 2, 1, 0.5])
    # analysis
    def analyse(lr):
        p = torch.nn.Parameter(torch.tensor([2.0, -1.5]))
        o = torch.optim.SGD([p], lr)
        an = A.OptimizerAnalyzer(o)
        for _ in range(30):
            l = (p ** 2).sum()
            o.zero_grad(); l.backward(); an.before_step(); o.step(); an.after_step(l.item())
        return an.report()
    good, bad, tiny = analyse(0.1), analyse(1.05), analyse(1e-9)
    assert good["improved"] and good["convergence_rate"] < -0.1 and not good["recommendations"]
    assert bad["recommendations"][0]["severity"] == "critical" and "raise" in tiny["recommendations"][0]["message"]
    def run(cfg):
        p = torch.nn.Parameter(torch.tensor([2.0, -1.5]))
        o = torch.optim.SGD([p], cfg["lr"], momentum=cfg["momentum"])
        for _ in range(20):
            o.zero_grad(); (p ** 2).sum().backward(); o.step()
        return float((p.detach() ** 2).sum())
    sens = A.hyperparameter_sensitivity(run, {"lr": 0.05, "momentum": 0.1})
    assert sens["ranking"][0] == "lr" and sens["parameters"]["lr"]["sensitivity"] > sens["parameters"]["momentum"]["sensitivity"]


def test_advanced_optimizers_storage_skipping_search_and_special_methods(tmp_path):
    import math
    import numpy as np
    from torsh_b200.optim import advanced as A
    torch.manual_seed(0)
    # 8-bit / bf16 state tracks fp32 Adam closely at a fraction of the state size
    x = torch.randn(1000) * torch.logspace(-3, 1, 1000)
    q = A.quantize_blockwise(x, 64)
    assert (A.dequantize_blockwise(*q) - x).abs().max() <= x.abs().reshape(-1, 8).amax() and q[0].dtype == torch.int8
    rel = ((A.dequantize_blockwise(*q) - x).abs() / x.abs().clamp(min=1e-6))
    assert rel.median() < 0.05
    xs, ys = torch.randn(256, 32), torch.randn(256, 8)
    finals = {}
    for kind in ("fp32", "int8", "bf16"):
        torch.manual_seed(1)
        m = torch.nn.Linear(32, 8)
        o = torch.optim.Adam(m.parameters(), 1e-2) if kind == "fp32" else A.LowPrecisionAdam(m.parameters(), 1e-2, state_dtype=kind, block=64)
        for _ in range(100):
            o.zero_grad(); torch.nn.functional.mse_loss(m(xs), ys).backward(); o.step()
        finals[kind] = torch.nn.functional.mse_loss(m(xs), ys).item()
        if kind != "fp32":
            assert o.state_bytes() < (0.3 if kind == "int8" else 0.55) * 2 * 4 * sum(p.numel() for p in m.parameters()) + 64
    assert abs(finals["int8"] - finals["fp32"]) < 0.02 and abs(finals["bf16"] - finals["fp32"]) < 0.02
    m = torch.nn.Linear(32, 8)
    fa = A.MemoryEfficientAdam(m.parameters(), lr=0.02)
    l0 = torch.nn.functional.mse_loss(m(xs), ys).item()
    for _ in range(150):
        fa.zero_grad(); torch.nn.functional.mse_loss(m(xs), ys).backward(); fa.step()
    assert torch.nn.functional.mse_loss(m(xs), ys).item() < 0.8 * l0
    fa2 = A.MemoryEfficientAdam(m.parameters(), lr=0.02, beta1=None)
    torch.nn.functional.mse_loss(m(xs), ys).backward(); fa2.step()
    assert fa2.state_numel() == 32 + 8 + 8                                  # row + column statistics for the matrix, full for the bias
    cb = A.CircularBuffer(3)
    for i in range(5):
        cb.push(i)
    assert list(cb) == [2, 3, 4] and len(cb) == 3
    p = torch.nn.Parameter(torch.tensor([-1.2, 1.0]))
    lb = A.MemoryEfficientLBFGS([p], history=5)
    def rosen():
        p.grad = None
        l = (1 - p[0]) ** 2 + 100 * (p[1] - p[0] ** 2) ** 2
        l.backward()
        return l
    for _ in range(60):
        lb.step(rosen)
    assert torch.allclose(p.detach(), torch.ones(2), atol=1e-3) and len(lb.pairs) == 5
    # memory-mapped state equals in-memory Adam and survives re-opening
    torch.manual_seed(3)
    a = torch.nn.Parameter(torch.randn(5, 3)); b = torch.nn.Parameter(a.detach().clone())
    oa, ob = A.MemoryMappedAdam([a], tmp_path / "adam.state", lr=0.01), torch.optim.Adam([b], 0.01)
    for i in range(5):
        g = torch.randn(5, 3)
        a.grad, b.grad = g.clone(), g.clone()
        oa.step(); ob.step()
        if i == 2:
            oa = A.MemoryMappedAdam([a], tmp_path / "adam.state", lr=0.01)                 # a new process would do the same
    assert torch.allclose(a, b, atol=1e-6) and (tmp_path / "adam.state").stat().st_size == (2 * 15 + 1) * 4
    # lazy and sparse updates
    big, small = torch.nn.Parameter(torch.ones(4) * 100), torch.nn.Parameter(torch.ones(4) * 0.01)
    lz = A.LazyUpdateOptimizer(torch.optim.SGD([big, small], 0.1), threshold=0.05, max_delay=4)
    for _ in range(4):
        big.grad, small.grad = torch.ones(4), torch.ones(4)
        lz.step()
    assert lz.statistics() == {"applied": 5, "skipped": 3, "skip_rate": 3 / 8} and torch.allclose(big.detach(), torch.full((4,), 99.9))
    w = torch.nn.Parameter(torch.zeros(100))
    target = torch.randn(100)
    sp = A.SparseUpdateOptimizer(torch.optim.SGD([w], 0.08), density=0.1)     # residuals apply ~10 steps at once: lr * delay < 1
    for _ in range(400):
        w.grad = (w.detach() - target)
        sp.step()
    st = sp.statistics()
    assert float((w.detach() - target).norm()) < 0.05 * float(target.norm()) and 0.09 < st["density"] < 0.12 and st["coverage"] == 1.0
    # state-dict tools
    m = torch.nn.Linear(16, 16)
    o = torch.optim.SGD(m.parameters(), 0.1, momentum=0.9)
    m(torch.randn(2, 16)).sum().backward(); o.step()
    sd = o.state_dict()
    blob = A.StateDictManager.compress(sd)
    assert torch.equal(A.StateDictManager.decompress(blob)["state"][0]["momentum_buffer"], sd["state"][0]["momentum_buffer"])
    assert A.StateDictManager.memory_estimate(sd) == {"total_bytes": (256 + 16) * 4, "by_key": {"momentum_buffer": (256 + 16) * 4}}
    conv = A.StateDictManager.convert(sd, {"momentum_buffer": "exp_avg"}, {"exp_avg_sq": lambda st: torch.zeros_like(st["exp_avg"]), "step": lambda st: torch.tensor(1.0)})
    adam = torch.optim.Adam(m.parameters(), 1e-3)
    conv["param_groups"] = adam.state_dict()["param_groups"]
    adam.load_state_dict(conv)
    assert torch.equal(adam.state[m.weight]["exp_avg"], sd["state"][0]["momentum_buffer"])
    sd2 = A.StateDictManager.decompress(blob); sd2["state"][0]["momentum_buffer"] = sd2["state"][0]["momentum_buffer"] * 3
    assert torch.allclose(A.StateDictManager.merge([sd, sd2])["state"][0]["momentum_buffer"], sd["state"][0]["momentum_buffer"] * 2)
    # hyper-parameter tuner: halving finds a good lr with less budget than random search at full budget
    def objective(cfg, budget):
        p = torch.nn.Parameter(torch.tensor([2.0, -1.5]))
        o = torch.optim.SGD([p], cfg["lr"], momentum=cfg["momentum"])
        for _ in range(budget):
            o.zero_grad(); (p ** 2).sum().backward(); o.step()
        v = float((p.detach() ** 2).sum())
        return v if math.isfinite(v) else 1e30
    space = {"lr": ("log", 1e-4, 0.9), "momentum": ("choice", [0.0, 0.5, 0.9])}
    rnd = A.HyperparameterTuner(space, "random", seed=0).tune(objective, n_trials=9, budget=27)
    hal = A.HyperparameterTuner(space, "halving", seed=0).tune(objective, n_trials=9, budget=27, min_budget=3, eta=3)
    assert hal["budget_spent"] == 3 * 9 + 9 * 3 + 27 * 1 < rnd["budget_spent"] == 243 and hal["best_loss"] < 1e-3 and rnd["best_loss"] < 1e-3
    grid = A.HyperparameterTuner(space, "grid").grid(3)
    assert len(grid) == 9 and grid[0]["lr"] == pytest.approx(1e-4)
    assert A.HyperparameterTuner(space, "random", seed=0).tune(objective, n_trials=9, budget=5, early_stopping_patience=2)["trials"] <= 9
    # learned optimizer: meta-training lowers the unrolled loss, and the trained rule optimises an unseen quadratic
    no = A.NeuralOptimizer()
    hist = no.meta_train(iters=120)
    assert np.mean(hist[-10:]) < 0.7 * np.mean(hist[:10])
    p = torch.nn.Parameter(torch.tensor([1.5, -2.0, 0.7]))
    scale, state = torch.tensor([0.5, 1.0, 2.0]), {}
    start = float((0.5 * scale * p.detach() ** 2).sum())
    for _ in range(40):
        p.grad = None
        (0.5 * scale * p ** 2).sum().backward()
        no.apply([p], state)
    assert float((0.5 * scale * p.detach() ** 2).sum()) < 0.5 * start
    mo = A.MetaOptimizer()
    assert mo.recommend({"a": 1.0})["optimizer"] == "adam"
    noisy, clean = torch.randn(8, 50) + 0.1, torch.ones(8, 50) + 0.001 * torch.randn(8, 50)
    fn, fc = A.MetaOptimizer.characterize(noisy), A.MetaOptimizer.characterize(clean)
    assert fn["noise"] > 10 * fc["noise"]
    mo.record(fn, {"optimizer": "adam", "lr": 1e-3}, 0.1); mo.record(fc, {"optimizer": "sgd", "lr": 0.1}, 0.1)
    assert mo.recommend(A.MetaOptimizer.characterize(torch.randn(8, 50) + 0.1))["optimizer"] == "adam"
    assert mo.recommend(A.MetaOptimizer.characterize(torch.ones(8, 50)))["optimizer"] == "sgd"
    # robustness: NaN gradients are skipped, spikes roll back and halve the learning rate
    p = torch.nn.Parameter(torch.tensor([1.0, 1.0]))
    rb = A.RobustnessManager(torch.optim.SGD([p], 0.1), max_grad_norm=0.5, snapshot_every=2)
    p.grad = torch.tensor([float("nan"), 1.0])
    assert rb.step(1.0) == "skipped" and torch.equal(p.detach(), torch.ones(2))
    for _ in range(6):
        p.grad = torch.tensor([3.0, 4.0])
        assert rb.step(1.0) == "ok"
    assert rb.stats["clipped"] == 6 and torch.allclose(p.detach(), torch.ones(2) - 6 * 0.1 * torch.tensor([0.3, 0.4]), atol=1e-5)
    keep = p.detach().clone()
    p.grad = torch.tensor([1.0, 1.0])
    assert rb.step(100.0) == "rolled_back" and rb.get_lr() == [0.05] and torch.allclose(p.detach(), keep)
    # energy accounting with a fake meter and clock
    clock = iter(np.arange(0, 100, 1.0))
    watts = iter([500, 1200, 1200, 1200, 1200, 500, 500, 500])
    p = torch.nn.Parameter(torch.zeros(1)); p.grad = torch.ones(1)
    ea = A.EnergyAwareOptimizer(torch.optim.SGD([p], 0.1), lambda: next(watts), carbon_intensity=360.0, power_cap=1000.0, clock=lambda: float(next(clock)))
    did = [ea.step() for _ in range(6)]
    assert did == [True, False, False, False, True, True] and ea.metrics()["steps"] == 3
    assert ea.energy_j == pytest.approx(500 + 4 * 1200 + 500) and ea.carbon_g == pytest.approx(5800 / 3.6e6 * 360)
    ea.budget = 0.0001
    with pytest.raises(RuntimeError):
        ea.step()
    # STDP: pre-before-post potentiates, post-before-pre depresses; event-driven SGD fires only on large accumulations
    w = torch.full((1, 1), 0.5)
    st = A.STDPOptimizer(w)
    st.step(torch.tensor([1]), torch.tensor([0])); st.step(torch.tensor([0]), torch.tensor([1]))
    assert float(w) > 0.5
    w2 = torch.full((1, 1), 0.5)
    st = A.STDPOptimizer(w2)
    st.step(torch.tensor([0]), torch.tensor([1])); st.step(torch.tensor([1]), torch.tensor([0]))
    assert float(w2) < 0.5
    p = torch.nn.Parameter(torch.zeros(2))
    ev = A.EventDrivenOptimizer([p], lr=1.0, threshold=0.25)
    for _ in range(3):
        p.grad = torch.tensor([0.1, 0.3])
        ev.step()
    assert torch.allclose(p.detach(), torch.tensor([-0.3, -0.9])) and ev.events == 4 and ev.event_rate() == pytest.approx(4 / 6)
    # quantum-inspired searches on a multimodal function and a bit-counting problem
    rast = lambda v: float(10 * len(v) + (v ** 2 - 10 * np.cos(2 * np.pi * v)).sum())
    for algo in (A.QuantumAnnealing(2, seed=0), A.QuantumPSO(2, seed=0)):
        r = algo.minimize(rast)
        assert r["fun"] < 1.1 and np.abs(r["x"]).max() < 1.1, type(algo).__name__
    pattern = np.array([1, 0, 1, 1, 0, 0, 1, 0, 1, 1, 1, 0])
    r = A.QuantumGeneticAlgorithm(12, seed=0).maximize(lambda b: float((b == pattern).sum()))
    assert r["fitness"] >= 11
    # step-for-step agreement of this package's optimizers with torch.optim
    from torsh_b200.optim import extra
    v = A.CrossFrameworkValidator()
    assert v.validate(lambda ps: extra.RAdam(ps, 1e-2), lambda ps: torch.optim.RAdam(ps, 1e-2))["passed"]
    assert v.validate(lambda ps: A.LowPrecisionAdam(ps, 1e-2, state_dtype="bf16"), lambda ps: torch.optim.Adam(ps, 1e-2))["max_abs_diff"] < 5e-3
    assert not v.validate(lambda ps: torch.optim.SGD(ps, 0.1), lambda ps: torch.optim.SGD(ps, 0.2))["passed"]


def test_vision_ops_color_filters_geometry_roi_and_metrics():
    import colorsys
    import numpy as np
    from scipy import ndimage
    import torchvision
    from torsh_b200.vision import ops as V
    torch.manual_seed(0)
    img = torch.rand(2, 3, 24, 32)
    # colour spaces against colorsys / round trips
    hsv = V.rgb_to_hsv(img)
    px = img[0, :, 5, 7].tolist()
    assert hsv[0, :, 5, 7].tolist() == pytest.approx(colorsys.rgb_to_hsv(*px), abs=1e-5)
    assert torch.allclose(V.hsv_to_rgb(hsv), img, atol=1e-5) and torch.allclose(V.yuv_to_rgb(V.rgb_to_yuv(img)), img, atol=1e-5)
    lab = V.rgb_to_lab(torch.tensor([1.0, 1.0, 1.0]).reshape(3, 1, 1))
    assert lab.flatten().tolist() == pytest.approx([100.0, 0.0, 0.0], abs=0.01)
    assert V.rgb_to_lab(torch.tensor([1.0, 0.0, 0.0]).reshape(3, 1, 1)).flatten().tolist() == pytest.approx([53.24, 80.09, 67.20], abs=0.05)
    assert torch.allclose(V.adjust_hue(img, 1.0), img, atol=1e-5) and torch.allclose(V.adjust_saturation(img, 0.0)[:, 0], V.rgb_to_grayscale(img)[:, 0], atol=1e-6)
    assert torch.allclose(V.adjust_contrast(img, 1.0), img) and V.adjust_brightness(img, 2.0).max() <= 1.0
    assert torch.allclose(V.gamma_correction(img, 1.0), img) and V.normalize_imagenet(img).shape == img.shape
    z = V.zscore(img)
    assert torch.allclose(z.mean((-2, -1)), torch.zeros(2, 3), atol=1e-5) and torch.allclose(z.std((-2, -1)), torch.ones(2, 3), atol=1e-4)
    h = V.compute_histogram(img, 16)
    assert h.shape == (2, 3, 16) and torch.all(h.sum(-1) == 24 * 32)
    assert np.allclose(h[0, 0].numpy(), np.histogram(img[0, 0].numpy(), 16, (0, 1))[0])
    dark = img ** 3
    eq = V.histogram_equalization(dark)
    assert abs(float(eq.mean()) - 0.5) < 0.1 and float(dark.mean()) < 0.3 and eq.min() >= 0 and eq.max() <= 1
    assert (eq[0, 0].flatten()[dark[0, 0].flatten().argsort()].diff() >= -1e-6).all()                   # monotone mapping
    cl = V.clahe(dark, tiles=(2, 2), clip_limit=2.0)
    assert cl.shape == dark.shape and float(cl.std()) > float(dark.std()) and float(cl.mean()) < float(eq.mean()) + 0.2
    # filters against scipy.ndimage
    g = img[0, 0]
    npg = g.numpy()
    assert np.allclose(V.gaussian_blur(g[None], 1.5)[0].numpy(), ndimage.gaussian_filter(npg, 1.5, mode="mirror", truncate=3.0 + 1e-6), atol=2e-3)
    gx, gy = V.sobel(g[None])
    assert np.allclose(gx[0].numpy(), ndimage.sobel(npg, axis=1, mode="mirror"), atol=1e-5) and np.allclose(gy[0].numpy(), ndimage.sobel(npg, axis=0, mode="mirror"), atol=1e-5)
    assert np.allclose(V.prewitt(g[None])[0][0].numpy(), ndimage.prewitt(npg, axis=1, mode="mirror"), atol=1e-5)
    assert np.allclose(V.laplacian(g[None])[0].numpy(), ndimage.laplace(npg, mode="mirror"), atol=1e-5)
    assert np.allclose(V.median_filter(g[None], 3)[0].numpy(), ndimage.median_filter(npg, 3, mode="mirror"))
    assert np.allclose(V.erosion(g[None], 3)[0].numpy(), ndimage.grey_erosion(npg, 3, mode="nearest")) and np.allclose(V.dilation(g[None], 5)[0].numpy(), ndimage.grey_dilation(npg, 5, mode="nearest"))
    assert np.allclose(V.opening(g[None])[0].numpy(), ndimage.grey_opening(npg, 3, mode="nearest")) and np.allclose(V.closing(g[None])[0].numpy(), ndimage.grey_closing(npg, 3, mode="nearest"))
    assert (V.morphological_gradient(g[None]) >= 0).all() and (V.top_hat(g[None]) >= -1e-7).all() and V.box_blur(img, 3).shape == img.shape
    step = torch.zeros(1, 20, 20); step[:, :, 10:] = 1.0
    noisy = (step + 0.05 * torch.randn(1, 20, 20)).clamp(0, 1)
    bl = V.bilateral_filter(noisy, 5, 2.0, 0.2)
    assert float(bl[:, :, :8].std()) < 0.6 * float(noisy[:, :, :8].std()) and float(bl[0, 10, 10] - bl[0, 10, 9]) > 0.8     # smooths, keeps the edge
    assert float((V.unsharp_mask(V.gaussian_blur(step, 1.0), 1.0, 1.0) - step).abs().mean()) < float((V.gaussian_blur(step, 1.0) - step).abs().mean())
    sq = torch.zeros(1, 32, 32); sq[:, 8:24, 8:24] = 1.0
    edges = V.canny(sq, 0.1, 0.3, 1.0)
    ring = (V.dilation(sq, 5) - V.erosion(sq, 5)) > 0
    assert edges.dtype == torch.bool and 40 <= int(edges.sum()) <= 80 and not (edges & ~ring).any() and not edges[0, 14:18, 14:18].any()
    assert float(V.sobel_edge_detection(sq)[0, 16, 16]) == 0 and float(V.sobel_edge_detection(sq)[0, 16, 8]) > 1
    # geometry
    assert torch.equal(V.horizontal_flip(V.horizontal_flip(img)), img) and V.center_crop(img, (10, 12)).shape == (2, 3, 10, 12)
    assert torch.equal(V.crop_region(img, 2, 3, 4, 5), img[..., 2:6, 3:8]) and V.pad(img, (1, 2, 3, 4)).shape == (2, 3, 31, 35)
    assert V.resize(img, (12, 16)).shape == (2, 3, 12, 16) and torch.allclose(V.resize(img, (24, 32)), img, atol=1e-6)
    sqi = torch.rand(1, 16, 16)
    assert torch.allclose(V.rotate(sqi, 90.0), torch.rot90(sqi, 1, (-2, -1)), atol=1e-5) and torch.allclose(V.rotate(sqi, 0.0), sqi, atol=1e-6)
    r180 = V.rotate(img, 180.0)
    assert torch.allclose(r180, img.flip(-1).flip(-2), atol=1e-5)
    tr = V.translate(sqi, 3, -2)
    assert torch.allclose(tr[:, :14, 3:], sqi[:, 2:, :13], atol=1e-5) and float(tr[:, :, :3].abs().sum()) == 0
    hm = torch.tensor([[1.0, 0, 2.0], [0, 1.0, 1.0], [0, 0, 1.0]])
    wp = V.warp_perspective(sqi, hm)
    assert torch.allclose(wp[:, :15, :14], sqi[:, 1:, 2:], atol=1e-5)
    sc = V.warp_affine(sqi, V.affine_grid_matrix(scale=2.0))
    assert torch.allclose(sc[:, ::2, ::2][:, 1:-1, 1:-1], F.interpolate(sqi[None], scale_factor=2.0, mode="bilinear", align_corners=False)[0][:, 8:24:2, 8:24:2][:, 1:-1, 1:-1], atol=1e-5) if (F := torch.nn.functional) else True
    # boxes and RoI ops against torchvision
    b = torch.tensor([[2.0, 3.0, 10.0, 9.0], [0.0, 0.0, 4.0, 4.0]])
    for fmt in ("xywh", "cxcywh"):
        assert torch.allclose(V.convert_bbox_format(V.convert_bbox_format(b, "xyxy", fmt), fmt, "xyxy"), b)
    assert V.convert_bbox_format(b, "xyxy", "cxcywh")[0].tolist() == [6.0, 6.0, 8.0, 6.0]
    assert V.clip_bbox(torch.tensor([[-5.0, 2.0, 50.0, 60.0]]), 24, 32).tolist() == [[0.0, 2.0, 32.0, 24.0]] and V.filter_boxes_by_size(b, 5).tolist() == [0]
    b2 = torch.tensor([[4.0, 4.0, 12.0, 12.0], [20.0, 20.0, 22.0, 25.0]])
    assert torch.allclose(V.generalized_iou(b, b2), torchvision.ops.generalized_box_iou(b, b2), atol=1e-6)
    feat = torch.randn(2, 4, 16, 16)
    rois = torch.tensor([[0, 1.0, 2.0, 9.0, 11.0], [1, 0.0, 0.0, 15.0, 15.0], [0, 3.5, 4.25, 7.75, 12.0]])
    assert torch.allclose(V.roi_align(feat, rois, (3, 3), 1.0, 2), torchvision.ops.roi_align(feat, rois, (3, 3), 1.0, 2, aligned=True), atol=1e-5)
    assert torch.allclose(V.roi_align(feat, rois, (2, 4), 0.5, 3), torchvision.ops.roi_align(feat, rois, (2, 4), 0.5, 3, aligned=True), atol=1e-5)
    irois = torch.tensor([[0, 1.0, 2.0, 9.0, 11.0], [1, 0.0, 0.0, 15.0, 15.0]])
    assert torch.allclose(V.roi_pool(feat, irois, (3, 3)), torchvision.ops.roi_pool(feat, irois, (3, 3)), atol=1e-6)
    # losses and metrics
    logits = torch.randn(2, 3, 8, 8, requires_grad=True)
    tgt = torch.randint(0, 3, (2, 8, 8))
    perfect = torch.nn.functional.one_hot(tgt, 3).permute(0, 3, 1, 2).float() * 50
    assert float(V.dice_loss(perfect, tgt)) < 1e-3 and 0.3 < float(V.dice_loss(logits, tgt).detach()) < 1.0
    V.dice_loss(logits, tgt).backward()
    assert logits.grad.abs().sum() > 0
    assert float(V.focal_loss(logits.detach(), tgt, gamma=0.0)) == pytest.approx(float(torch.nn.functional.cross_entropy(logits.detach(), tgt)), rel=1e-5)
    assert float(V.focal_loss(logits.detach(), tgt, gamma=2.0)) < float(V.focal_loss(logits.detach(), tgt, gamma=0.0))
    assert float(V.iou_loss(b, b)) == 0 and float(V.iou_loss(b, b2, "giou")) > float(V.iou_loss(b, b2))
    pred = tgt.clone(); pred[0, :2] = (pred[0, :2] + 1) % 3
    sm = V.compute_segmentation_metrics(pred, tgt, 3)
    assert sm["pixel_accuracy"] == pytest.approx(1 - 16 / 128) and 0.6 < sm["mean_iou"] < sm["mean_dice"] < 1
    from sklearn.metrics import jaccard_score
    assert sm["per_class_iou"] == pytest.approx(jaccard_score(tgt.flatten().numpy(), pred.flatten().numpy(), average=None).tolist())
    gt_b, gt_l = torch.tensor([[0.0, 0, 10, 10], [20.0, 20, 30, 30]]), torch.tensor([1, 1])
    pb = torch.tensor([[0.0, 0, 10, 9], [50.0, 50, 60, 60], [20.0, 21, 30, 30]])
    dm = V.compute_detection_metrics(pb, torch.tensor([0.9, 0.8, 0.7]), torch.tensor([1, 1, 1]), gt_b, gt_l)
    assert dm["precision"] == pytest.approx(2 / 3) and dm["recall"] == 1.0 and dm["map"] == pytest.approx(0.5 * 1.0 + 0.5 * 2 / 3)
    cmx = V.compute_classification_metrics(torch.tensor([[2.0, 1.0, 0.0], [0.0, 1.0, 2.0], [0.1, 0.3, 0.2]]), torch.tensor([0, 1, 1]), topk=(1, 2))
    assert cmx["top1"] == pytest.approx(2 / 3) and cmx["top2"] == 1.0 and 0 < cmx["macro_f1"] < 1


def test_vision_augmentation_policies_and_self_supervised_views():
    from torsh_b200.vision import augment as A, ops as V
    torch.manual_seed(0)
    img = torch.rand(3, 32, 32)
    for name in A.OPS:
        out = A._Random(0).apply_op(img, name, 0.5)
        assert out.shape == img.shape and torch.isfinite(out).all(), name
    assert torch.equal(A._Random(0).apply_op(img, "identity", 1.0), img) and torch.allclose(A._Random(0).apply_op(img, "invert", 0.3), 1 - img)
    assert A._posterize(img, 4).unique().numel() <= 16 and torch.allclose(A._solarize(torch.tensor([0.2, 0.8]), 0.5), torch.tensor([0.2, 0.2]))
    ac = A._autocontrast(0.25 + 0.5 * img)
    assert ac.amin((-2, -1)).abs().max() < 1e-6 and (ac.amax((-2, -1)) - 1).abs().max() < 1e-6
    ra = A.RandAugment(n=3, m=9, seed=1)
    a, b = ra(img), A.RandAugment(n=3, m=9, seed=1)(img)
    assert torch.equal(a, b) and len(ra.last) == 3 and not torch.equal(a, A.RandAugment(n=3, m=9, seed=2)(img))
    weak, strong = A.RandAugment(2, 1, ops=["rotate"], seed=0)(img), A.RandAugment(2, 30, ops=["rotate"], seed=0)(img)
    assert float((weak - img).abs().mean()) < float((strong - img).abs().mean())
    for pol in ("imagenet", "cifar10"):
        aa = A.AutoAugment(pol, seed=0)
        outs = [aa(img) for _ in range(6)]
        assert all(o.shape == img.shape and o.min() >= 0 and o.max() <= 1 for o in outs) and any(not torch.equal(o, img) for o in outs)
    assert torch.equal(A.AutoAugment([[("invert", 1.0, 0)]], seed=0)(img), 1 - img) and torch.equal(A.AutoAugment([[("invert", 0.0, 0)]], seed=0)(img), img)
    am = A.AugMix(seed=0)(img)
    assert am.shape == img.shape and 0 < float((am - img).abs().mean()) < float((A.RandAugment(3, 20, seed=0)(img) - img).abs().mean()) + 0.2
    gm = A.GridMask((8, 8), 0.5, seed=0)
    mk = gm.mask(32, 32)
    assert mk.float().mean() == pytest.approx(0.75) and torch.equal(mk[:24, :24], mk[8:, 8:]) and (A.GridMask(seed=0)(img) == 0).any()
    imgs = [torch.full((3, 20, 30), v) for v in (0.1, 0.4, 0.7, 1.0)]
    boxes = [torch.tensor([[0.0, 0.0, 30.0, 20.0]])] * 3 + [torch.zeros(0, 4)]
    canvas, mb, src = A.Mosaic(64, seed=3)(imgs, boxes)
    assert canvas.shape == (3, 64, 64) and sorted(canvas.mul(100).round().unique().tolist()) == [10, 40, 70, 100] and src.tolist() == [0, 1, 2]
    area = ((mb[:, 2] - mb[:, 0]) * (mb[:, 3] - mb[:, 1]))
    for i, v in enumerate((0.1, 0.4, 0.7)):
        assert float(((canvas[0] - v).abs() < 1e-4).sum()) == pytest.approx(float(area[i]))        # the box still covers its whole image
    g = torch.Generator().manual_seed(0)
    flat = torch.full((1, 64, 64), 0.5)
    assert float(A.add_noise(flat, "gaussian", 0.1, g).std()) == pytest.approx(0.1, rel=0.1)
    sp = A.add_noise(flat, "salt_pepper", 0.2, g)
    assert float(((sp == 0) | (sp == 1)).float().mean()) == pytest.approx(0.2, abs=0.03)
    assert float(A.add_noise(flat, "speckle", 0.1, g).std()) == pytest.approx(0.05, rel=0.15) and float(A.add_noise(flat, "poisson", 0.01, g).mean()) == pytest.approx(0.5, abs=0.01)
    co = A.cutout(torch.ones(1, 32, 32), 8, g)
    assert 16 <= int((co == 0).sum()) <= 64
    assert A.RandomAffine(seed=0)(img).shape == img.shape and A.RandomResizedCrop(16, seed=0)(img).shape == (3, 16, 16)
    # self-supervised views: shapes, determinism per seed, two views differ, positives score above negatives after a few steps
    v1, v2 = A.SimCLRAugmentation(16, seed=0).generate_pair(img)
    assert v1.shape == v2.shape == (3, 16, 16) and not torch.equal(v1, v2) and torch.equal(v1, A.SimCLRAugmentation(16, seed=0).generate_pair(img)[0])
    assert [tuple(v.shape[-2:]) for v in A.SwAVAugmentation(32, 16, 2, 4).generate_views(img)] == [(32, 32)] * 2 + [(16, 16)] * 4
    assert len(A.DINOAugmentation(32, 16, 6).generate_views(img)) == 8 and A.BYOLAugmentation(16).generate_pair(img)[0].shape == (3, 16, 16)
    assert A.MoCoAugmentation(16).generate_pair(img)[1].shape == (3, 16, 16)
    z = torch.nn.functional.normalize(torch.randn(8, 16), dim=1)
    assert float(A.nt_xent_loss(z, z, 0.1)) < float(A.nt_xent_loss(z, z.roll(1, 0), 0.1)) and float(A.byol_loss(z, z)) == pytest.approx(0.0, abs=1e-6)
    assert float(A.byol_loss(z, -z)) == pytest.approx(4.0, abs=1e-5)
    data = torch.rand(8, 3, 16, 16)
    enc = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(768, 32))
    opt = torch.optim.Adam(enc.parameters(), 1e-2)
    aug = A.SimCLRAugmentation(16, strength=0.3, seed=0)
    first = None
    for _ in range(30):
        pairs = [aug.generate_pair(d) for d in data]
        loss = A.nt_xent_loss(enc(torch.stack([p[0] for p in pairs])), enc(torch.stack([p[1] for p in pairs])))
        opt.zero_grad(); loss.backward(); opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < first


def test_vision_analysis_segmentation_features_spatial_streaming_and_3d(tmp_path):
    import numpy as np
    from scipy import ndimage
    from scipy.spatial import cKDTree
    from torsh_b200.vision import analysis as N, ops as V
    torch.manual_seed(0)
    # connected components against scipy
    mask = torch.rand(24, 24) > 0.55
    for conn, st in ((4, None), (8, np.ones((3, 3)))):
        lab, n = N.connected_components(mask, conn)
        ref, nref = ndimage.label(mask.numpy(), structure=st)
        assert n == nref and len(set(zip(lab.flatten().tolist(), ref.flatten().tolist()))) == n + 1
    # two flat regions with a ramp: region growing with a fixed reference stops at the step
    img = torch.zeros(1, 20, 20); img[:, :, 10:] = 1.0
    img = img + 0.02 * torch.randn(1, 20, 20)
    rg = N.region_growing(img, [(5, 3), (5, 15)], threshold=0.2)
    assert (rg[:, :10] == 1).all() and (rg[:, 10:] == 2).all()
    # watershed splits two touching discs along the neck
    yy, xx = torch.meshgrid(torch.arange(40.0), torch.arange(60.0), indexing="ij")
    d1, d2 = ((yy - 20) ** 2 + (xx - 20) ** 2).sqrt(), ((yy - 20) ** 2 + (xx - 40) ** 2).sqrt()
    blobs = (d1 < 13) | (d2 < 13)
    height = -torch.from_numpy(ndimage.distance_transform_edt(blobs.numpy())).float()
    markers = torch.zeros(40, 60, dtype=torch.long); markers[20, 20], markers[20, 40], markers[0, 0] = 1, 2, 3
    ws = N.watershed(height, markers)
    left, right = ws[20, 5:29], ws[20, 32:55]
    assert (left == 1).all() and (right == 2).all() and set(ws[blobs].unique().tolist()) >= {1, 2}
    auto = N.watershed(height)
    assert auto[20, 20] != auto[20, 40] and (auto > 0).all()
    # graph cut recovers a noisy square from a few seeds
    truth = torch.zeros(24, 24, dtype=torch.bool); truth[6:18, 6:18] = True
    noisy = (truth.float() * 0.6 + 0.2 + 0.15 * torch.randn(24, 24)).clamp(0, 1)
    fg = torch.zeros_like(truth); fg[10:14, 10:14] = True
    bg = torch.zeros_like(truth); bg[:2] = True; bg[:, :2] = True
    seg = N.graph_cuts(noisy, fg, bg, lam=5.0, sigma=0.2)
    naive = noisy > 0.5
    assert float((seg == truth).float().mean()) > 0.97 and float((seg == truth).float().mean()) >= float((naive == truth).float().mean())
    # corners of a square, descriptors and matching under a known homography
    sq = torch.zeros(1, 48, 48); sq[:, 12:36, 14:34] = 1.0
    kp = N.detect_corners(V.gaussian_blur(sq, 1.0), max_points=4, min_distance=5)
    found = sorted((round(x), round(y)) for x, y in kp.xy.tolist())
    want = sorted([(14, 12), (33, 12), (14, 35), (33, 35)])
    assert all(abs(a[0] - b[0]) <= 2 and abs(a[1] - b[1]) <= 2 for a, b in zip(found, want))
    assert len(N.detect_corners(V.gaussian_blur(sq, 1.0), kind="shi_tomasi", max_points=4, min_distance=5).xy) == 4
    tex = V.gaussian_blur(torch.rand(1, 96, 96), 1.5)
    tex = (tex - tex.min()) / (tex.max() - tex.min())
    hm_true = torch.tensor([[1.0, 0.03, 4.0], [-0.02, 1.0, -3.0], [0.0, 0.0, 1.0]])
    warped = V.warp_perspective(tex, torch.linalg.inv(hm_true))                                # warped(p') = tex(H^-1 p'), so p' = H p
    k1, k2 = N.detect_corners(tex, max_points=150, border=12), N.detect_corners(warped, max_points=150, border=12)
    d1, d2 = N.describe(tex, k1), N.describe(warped, k2)
    assert d1.shape == (len(k1.xy), 128) and torch.allclose(d1.norm(dim=1), torch.ones(len(d1)), atol=1e-4)
    m = N.match_features(d1, d2, ratio=0.85)
    assert len(m) >= 20
    hm, inl = N.ransac_homography(k1.xy[m[:, 0]], k2.xy[m[:, 1]], threshold=2.0, iters=300)
    assert inl.float().mean() > 0.6
    probe = torch.tensor([[20.0, 20.0], [70.0, 30.0], [40.0, 80.0]])
    assert (N.apply_homography(hm, probe) - N.apply_homography(hm_true, probe)).norm(dim=1).max() < 1.5
    pts = torch.rand(12, 2) * 50
    assert torch.allclose(N.fit_homography(pts, N.apply_homography(hm_true, pts)), hm_true, atol=1e-3)
    ms = N.detect_multiscale(tex, levels=2, max_points=50)
    assert set(ms.scale.unique().tolist()) == {1.0, 1.5} and ms.xy.max() < 96
    # template matching: exact location with score 1, matcher keeps peaks above threshold
    tmpl = tex[0, 30:42, 50:66]
    ncc = N.match_template(tex, tmpl)
    assert divmod(int(ncc.argmax()), ncc.shape[1]) == (30, 50) and float(ncc.max()) == pytest.approx(1.0, abs=1e-4) and float(ncc.min()) >= -1.0001
    tm = N.TemplateMatcher(0.95); tm.add_template("t", tmpl)
    hits = tm.match_templates(tex)
    assert hits[0]["x"] == 50 and hits[0]["y"] == 30 and len(hits) == 1
    assert N.find_similar_patches(tex, tmpl, 1)[0] == [(50, 30)]
    # k-d tree against scipy
    cloud = torch.rand(300, 3)
    tree, ref = N.KDTree(cloud), cKDTree(cloud.numpy())
    for q in torch.rand(5, 3):
        idx, dist = tree.find_neighbors(q.numpy(), 5)
        rd, ri = ref.query(q.numpy(), 5)
        assert idx == ri.tolist() and dist == pytest.approx(rd.tolist(), abs=1e-6)
        assert tree.query_region(q.numpy(), 0.2) == sorted(ref.query_ball_point(q.numpy().astype(float), 0.2))
    # tracker keeps identities through motion, opens and closes tracks
    tr = N.SpatialObjectTracker(0.3, max_age=1)
    a, b = torch.tensor([0.0, 0, 10, 10]), torch.tensor([50.0, 50, 60, 60])
    ids0 = tr.track_objects(torch.stack([a, b]))
    ids1 = tr.track_objects(torch.stack([b + 2, a + 2]))
    assert ids0 == [0, 1] and ids1 == [1, 0]
    ids2 = tr.track_objects(torch.stack([a + 4, torch.tensor([100.0, 100, 110, 110])]))
    assert ids2 == [0, 2] and tr.get_trajectory(0) == [(5.0, 5.0), (7.0, 7.0), (9.0, 9.0)]
    tr.track_objects(a[None] + 6); tr.track_objects(a[None] + 8)
    assert 1 in tr.finished and 0 in tr.tracks and len(tr.get_trajectory(1)) == 2
    # distortion: correcting with k = 0 is the identity; barrel then its inverse roughly restores the centre
    assert torch.allclose(N.correct_radial_distortion(tex, 0.0), tex, atol=1e-5)
    bar = N.correct_radial_distortion(tex, -0.2)
    assert not torch.allclose(bar, tex, atol=1e-2) and torch.allclose(bar[:, 44:52, 44:52], tex[:, 44:52, 44:52], atol=0.05)
    flow = torch.zeros(2, 96, 96); flow[0] = 3.0
    assert torch.allclose(N.warp_by_flow(tex, flow)[:, :, :90], tex[:, :, 3:93], atol=1e-5)
    shifted = N.warp_by_flow(tex, -flow)                                                          # content moved 3 px to the right
    mid = N.interpolate_frames(tex, shifted, flow, 0.5)
    assert float((mid[:, :, 8:88] - N.warp_by_flow(tex, -flow / 2)[:, :, 8:88]).abs().max()) < 1e-4
    assert N.smooth_flow_field(torch.randn(2, 16, 16)).std() < 0.5
    pts2 = torch.tensor([[0.0, 0.0], [9.0, 0.0], [0.0, 9.0], [9.0, 9.0]])
    grid = N.interpolate_to_grid(pts2, torch.tensor([0.0, 1.0, 1.0, 2.0]), 10, 10)
    assert grid[0, 0] == 0 and grid[9, 9] == 2 and abs(float(grid[4, 5]) - 1.0) < 0.1 and N.interpolate_to_grid(pts2, torch.tensor([0.0, 1.0, 1.0, 2.0]), 10, 10, "nearest")[1, 8] == 1
    ramp = torch.linspace(0, 1, 20).expand(1, 20, 20).clone()
    valid = torch.ones(1, 20, 20, dtype=torch.bool); valid[:, 8:12, 8:12] = False
    filled = N.interpolate_image_gaps(ramp, valid)
    assert torch.equal(filled[valid], ramp[valid]) and (filled - ramp).abs().max() < 0.03
    assert N.compute_image_similarity(tex, tex) == pytest.approx(1.0, abs=1e-4) and N.compute_image_similarity(tex, tex.flip(-1)) < 0.5
    assert N.compute_image_similarity(tex, tex, "psnr") > 100 and N.compute_image_similarity(tex, 1 - tex, "ncc") == pytest.approx(-1.0, abs=1e-4)
    gal = torch.rand(6, 3, 32, 32)
    assert N.find_similar_images((gal[4] * 0.9 + 0.05), gal, 2)[0][0] == 4
    # streaming: drops when full, batches, adapts resolution to a slow consumer with a fake clock
    now = [0.0]
    def slow(batch):
        now[0] += 0.05 * batch.shape[0] * batch.shape[-1] / 64                                   # cost grows with resolution
        return batch.mean().item()
    sp = N.StreamProcessor(slow, target_fps=30.0, buffer_size=4, batch_size=2, clock=lambda: now[0])
    for i in range(6):
        sp.push_frame(torch.full((3, 80, 80), float(i)))
    assert sp.dropped == 2 and len(sp) == 4 and [f.index for f in sp.queue] == [2, 3, 4, 5] and sp.is_full()
    res = sp.process_available()
    assert [r["indices"] for r in res] == [[2, 3], [4, 5]] and res[0]["resolution"] == (64, 64) and sp.is_empty()
    for i in range(20):
        sp.push_frame(torch.rand(3, 80, 80)); sp.push_frame(torch.rand(3, 80, 80)); sp.process_available()
    st = sp.stats()
    assert st["resolution"] == (32, 32) and st["processed"] == 44 and st["mean_latency"] < 1 / 30 and sp.is_realtime()
    keep = N.StreamProcessor(lambda b: 0, buffer_size=2, drop_policy="drop_newest")
    assert [keep.push_frame(torch.zeros(3, 8, 8)) for _ in range(3)] == [True, True, False] and len(keep.flush()) == 2
    assert N.FramePreprocessor((8, 8), True, ((0.5,), (0.5,))).preprocess(torch.ones(3, 16, 16)).shape == (1, 8, 8)
    # 3-D: sphere mesh geometry, sampled cloud, normals, voxel grid, boxes, scene export
    sph = N.Mesh3D.create_sphere(2.0, 24, 48)
    assert sph.surface_area() == pytest.approx(4 * np.pi * 4, rel=0.01) and sph.volume() == pytest.approx(4 / 3 * np.pi * 8, rel=0.02)
    assert (sph.compute_vertex_normals() * torch.nn.functional.normalize(sph.vertices, dim=1)).sum(1).min() > 0.99
    cube = N.Mesh3D.create_cube(2.0)
    assert cube.volume() == pytest.approx(8.0) and cube.surface_area() == pytest.approx(24.0) and (cube.compute_face_normals().abs().max(1).values == 1).all()
    pc = sph.sample_points(2000)
    assert (pc.points.norm(dim=1) - 2.0).abs().max() < 0.02
    nrm = pc.estimate_normals(10)
    assert (nrm * torch.nn.functional.normalize(pc.points, dim=1)).sum(1).mean() > 0.97
    ds = pc.voxel_downsample(0.5)
    assert 50 < len(ds) < 400 and ds.points.norm(dim=1).max() <= 2.0 + 1e-5
    assert len(pc.filter_by_distance((0, 0, 2.0), 1.0)) < 400 and pc.to_tensor().shape == (2000, 6)
    noisy_pc = N.PointCloud(torch.cat([pc.points, torch.tensor([[30.0, 30.0, 30.0]])]))
    assert len(noisy_pc.remove_statistical_outliers()) == 2000
    moved = pc.transform(torch.tensor([[1.0, 0, 0, 5], [0, 1.0, 0, 0], [0, 0, 1.0, 0], [0, 0, 0, 1.0]]))
    assert moved.centroid()[0] == pytest.approx(5.0, abs=0.1)
    bb = N.BoundingBox3D.from_points(cube.vertices)
    assert bb.volume() == 8.0 and bb.contains_point((0.5, 0, 0)) and not bb.contains_point((2, 0, 0)) and bb.corners().shape == (8, 3)
    assert bb.iou(N.BoundingBox3D(torch.zeros(3), torch.full((3,), 2.0))) == pytest.approx(1 / 15)
    sc = N.Scene3D(); sc.add_mesh(cube, "cube"); sc.add_point_cloud(ds, "cloud"); sc.add_bounding_box(bb, "box")
    summ = sc.export_summary()
    assert summ["faces"] == 12 and summ["points"] == len(ds) and sc.num_objects() == 3
    sc.export_ply(tmp_path / "s.ply")
    head = (tmp_path / "s.ply").read_text().splitlines()
    assert head[2] == f"element vertex {8 + len(ds)}" and head[6] == "element face 12" and len(head) == 9 + 8 + len(ds) + 12


def test_functional_ext_decompositions_wavelets_numerics_interpolation_lazy_and_sampling():
    import math
    import numpy as np
    from scipy import integrate, interpolate, stats
    from torsh_b200.nn import functional_ext as X
    torch.manual_seed(0)
    dd = torch.float64
    # CP recovers a rank-3 tensor; Tucker recovers a multilinear rank-(2,3,2) tensor; TT-SVD is exact at full rank
    fac = [torch.randn(n, 3, dtype=dd) for n in (6, 5, 4)]
    t3 = X.cp_reconstruct(torch.tensor([3.0, 2.0, 1.0], dtype=dd), fac)
    assert torch.allclose(t3, torch.einsum("r,ir,jr,kr->ijk", torch.tensor([3.0, 2.0, 1.0], dtype=dd), *fac))
    w, f, err = X.cp_decomposition(t3, 3, iters=500)
    assert err < 1e-5 and torch.allclose(X.cp_reconstruct(w, f), t3, atol=1e-4) and torch.allclose(f[0].norm(dim=0), torch.ones(3, dtype=dd))
    assert X.cp_decomposition(t3, 1)[2] > 0.1
    core0 = torch.randn(2, 3, 2, dtype=dd)
    mats = [torch.linalg.qr(torch.randn(n, r, dtype=dd)).Q for n, r in ((6, 2), (5, 3), (4, 2))]
    tk = X.tucker_reconstruct(core0, mats)
    core, tf, terr = X.tucker_decomposition(tk, (2, 3, 2))
    assert terr < 1e-10 and core.shape == (2, 3, 2) and all(torch.allclose(m.t() @ m, torch.eye(m.shape[1], dtype=dd), atol=1e-10) for m in tf)
    assert X.tucker_decomposition(tk, (1, 1, 1))[2] > 0.1
    full = torch.randn(3, 4, 5, 2, dtype=dd)
    cores = X.tensor_train(full, max_rank=100)
    assert torch.allclose(X.tt_reconstruct(cores), full, atol=1e-10) and [c.shape[0] for c in cores] == [1, 3, 10, 2]
    lowrank = X.tt_reconstruct([torch.randn(1, 3, 2, dtype=dd), torch.randn(2, 4, 2, dtype=dd), torch.randn(2, 5, 1, dtype=dd)])
    c2 = X.tensor_train(lowrank, max_rank=2)
    assert torch.allclose(X.tt_reconstruct(c2), lowrank, atol=1e-10) and sum(c.numel() for c in c2) < lowrank.numel()
    # wavelets: filters are orthonormal, transforms invertible and energy preserving, db2 kills linear trends
    for name, h in X.WAVELETS.items():
        h = torch.tensor(h, dtype=dd)
        assert float(h.sum()) == pytest.approx(math.sqrt(2), abs=1e-10) and float((h * h).sum()) == pytest.approx(1.0, abs=1e-10), name
        sig = torch.randn(3, 64, dtype=dd)
        a, d = X.dwt_1d(sig, name)
        assert torch.allclose(X.idwt_1d(a, d, name), sig, atol=1e-10) and float(a.pow(2).sum() + d.pow(2).sum()) == pytest.approx(float(sig.pow(2).sum()))
        coeffs = X.wavedec(sig, name, 3)
        assert [c.shape[-1] for c in coeffs] == [8, 8, 16, 32] and torch.allclose(X.waverec(coeffs, name), sig, atol=1e-10)
        img = torch.randn(16, 32, dtype=dd)
        ll, det = X.dwt_2d(img, name)
        assert ll.shape == (8, 16) and torch.allclose(X.idwt_2d(ll, det, name), img, atol=1e-10)
    a, d = X.dwt_1d(torch.tensor([1.0, 3.0, 5.0, 9.0]), "haar")
    assert torch.allclose(a, torch.tensor([4.0, 14.0]) / math.sqrt(2)) and torch.allclose(d.abs(), torch.tensor([2.0, 4.0]) / math.sqrt(2))
    lin = torch.arange(64, dtype=dd)
    assert X.dwt_1d(lin, "db2")[1][:-1].abs().max() < 1e-10 and X.dwt_1d(lin, "haar")[1].abs().min() > 0.1     # two vanishing moments
    n = 512
    tt = torch.arange(n, dtype=dd)
    chirp = torch.sin(2 * math.pi * tt / 16) * (tt < 256) + torch.sin(2 * math.pi * tt / 64) * (tt >= 256)
    scales = [16 * 6 / (2 * math.pi), 64 * 6 / (2 * math.pi)]
    cw = X.cwt(chirp, scales).abs()
    assert cw.shape == (2, n) and cw[0, 64:192].mean() > 3 * cw[1, 64:192].mean() and cw[1, 320:448].mean() > 3 * cw[0, 320:448].mean()
    assert X.cwt(chirp, [4.0], "mexican_hat").shape == (1, n)
    clean = torch.sin(2 * math.pi * tt / 128)
    noisy = clean + 0.3 * torch.randn(n, dtype=dd)
    assert float((X.wavelet_denoise(noisy) - clean).pow(2).mean()) < 0.35 * float((noisy - clean).pow(2).mean())
    # calculus and roots against scipy
    xs = torch.linspace(0, math.pi, 101, dtype=dd)
    assert float(X.trapz(torch.sin(xs), xs)) == pytest.approx(integrate.trapezoid(np.sin(xs.numpy()), xs.numpy()))
    assert float(X.simps(torch.sin(xs), float(xs[1]))) == pytest.approx(2.0, abs=1e-7) and float(X.simps(torch.sin(xs[:100]), float(xs[1]))) == pytest.approx(float(1 - torch.cos(xs[99])), abs=1e-5)
    assert torch.allclose(X.cumtrapz(torch.sin(xs), xs), torch.from_numpy(integrate.cumulative_trapezoid(np.sin(xs.numpy()), xs.numpy())))
    assert float(X.gaussian_quad(lambda z: torch.exp(-z * z), -2.0, 3.0, 24)) == pytest.approx(integrate.quad(lambda z: math.exp(-z * z), -2, 3)[0], abs=1e-12)
    assert X.adaptive_quad(lambda z: math.sqrt(z), 0.0, 1.0, 1e-10) == pytest.approx(2 / 3, abs=1e-7)
    assert torch.allclose(X.gradient(xs ** 2, float(xs[1]))[1:-1], 2 * xs[1:-1], atol=1e-10)
    assert float(X.second_derivative(torch.sin, torch.tensor(0.7, dtype=dd))) == pytest.approx(-math.sin(0.7), abs=1e-6)
    assert float(X.partial_derivative(lambda v: (v[..., 0] ** 2 * v[..., 1]), torch.tensor([2.0, 3.0], dtype=dd), 0)) == pytest.approx(12.0, abs=1e-6)
    assert X.bisection(lambda z: z ** 3 - 2, 0.0, 2.0) == pytest.approx(2 ** (1 / 3), abs=1e-9)
    with pytest.raises(ValueError):
        X.bisection(lambda z: z * z + 1, -1.0, 1.0)
    assert float(X.newton_raphson(lambda z: z ** 3 - 2, 1.0)) == pytest.approx(2 ** (1 / 3), abs=1e-10)
    root = X.newton_raphson(lambda v: torch.stack([v[0] ** 2 + v[1] ** 2 - 4, v[0] - v[1]]), [1.0, 0.5])
    assert torch.allclose(root, torch.full((2,), math.sqrt(2), dtype=dd), atol=1e-9)
    # transformations
    m = torch.arange(6.0).reshape(2, 3)
    assert torch.equal(X.tensor_map(lambda v: v * v + 1, m), m * m + 1) and torch.equal(X.tensor_map(lambda r: r.flip(0), m, 0), m.flip(1))
    assert torch.equal(X.tensor_zip(lambda a, b: a * b, m, torch.tensor([1.0, 2.0, 3.0])), m * torch.tensor([1.0, 2.0, 3.0]))
    assert torch.equal(X.tensor_fold(lambda acc, r: acc + r, m, torch.zeros(3)), m.sum(0)) and torch.equal(X.tensor_scan(torch.maximum, m.t().contiguous(), dim=0), m.t().cummax(0).values)
    assert torch.equal(X.tensor_reduce(torch.add, torch.arange(7.0)[:, None]), torch.tensor([21.0]))
    assert X.tensor_outer(torch.ones(2), torch.ones(3), torch.ones(4)).shape == (2, 3, 4)
    assert X.tensor_contract(torch.randn(2, 3, 4), torch.randn(4, 3, 5), [1, 2], [1, 0]).shape == (2, 5)
    A_, B_, C_ = torch.randn(8, 30, dtype=dd), torch.randn(30, 4, dtype=dd), torch.randn(4, 50, dtype=dd)
    res, order, cost = X.einsum_optimized("ij,jk,kl->il", A_, B_, C_)
    assert torch.allclose(res, A_ @ B_ @ C_) and order[0][:2] == ("ij", "jk") and cost == 8 * 30 * 4 + 8 * 4 * 50
    # gradient penalties
    critic = torch.nn.Linear(5, 1, bias=False)
    real, fake = torch.randn(16, 5), torch.randn(16, 5)
    wn = float(critic.weight.detach().norm())
    assert X.gradient_penalty(critic, real, fake).item() == pytest.approx((wn - 1) ** 2, rel=1e-4)
    assert X.r1_gradient_penalty(critic, real).item() == pytest.approx(0.5 * wn * wn, rel=1e-4) == X.r2_gradient_penalty(critic, fake).item()
    X.gradient_penalty(critic, real, fake).backward()
    assert critic.weight.grad is not None
    wm = torch.randn(6, 9)
    assert float(X.spectral_gradient_penalty(wm, 200)) == pytest.approx(float(torch.linalg.svdvals(wm)[0]), rel=1e-4)
    assert X.consistency_penalty(critic, real, lambda z: z).item() == 0
    # interpolation against scipy
    xp = torch.linspace(0, 5, 11, dtype=dd); fp = torch.sin(xp)
    xq = torch.tensor([-1.0, 0.3, 2.26, 4.99, 7.0], dtype=dd)
    assert torch.allclose(X.interp1d(xq, xp, fp), torch.from_numpy(np.interp(xq.numpy(), xp.numpy(), fp.numpy())))
    assert torch.equal(X.interp1d(torch.tensor([0.2, 0.3], dtype=dd), xp, fp, "nearest"), fp[[0, 1]])
    xin = torch.linspace(0.1, 4.9, 23, dtype=dd)
    assert torch.allclose(X.spline1d(xin, xp, fp), torch.from_numpy(interpolate.CubicSpline(xp.numpy(), fp.numpy(), bc_type="natural")(xin.numpy())), atol=1e-10)
    samples = torch.sin(torch.arange(40, dtype=dd) * 0.3)
    pos = torch.tensor([5.5, 10.25, 20.0], dtype=dd)
    assert torch.allclose(X.lanczos_interp1d(pos, samples), torch.sin(pos * 0.3), atol=1e-2) and float(X.lanczos_interp1d(pos, samples)[2]) == pytest.approx(float(samples[20]))
    cheb = torch.cos(math.pi * (2 * torch.arange(12, dtype=dd) + 1) / 24)
    runge = lambda z: 1 / (1 + 25 * z * z)
    xe = torch.linspace(-0.95, 0.95, 7, dtype=dd)
    assert torch.allclose(X.barycentric_interp(xe, cheb, runge(cheb)), torch.from_numpy(interpolate.BarycentricInterpolator(cheb.numpy(), runge(cheb).numpy())(xe.numpy())), atol=1e-10)
    assert torch.allclose(X.barycentric_interp(cheb[:3], cheb, runge(cheb)), runge(cheb[:3]))
    g2 = torch.arange(12.0).reshape(3, 4)
    assert torch.allclose(X.interp2d(g2, torch.tensor([1.5, 0.0]), torch.tensor([0.5, 2.0])), torch.tensor([3.5, 8.0]))
    # counting
    data = torch.tensor([0.5, 1.5, 1.7, 2.0, 3.9, 4.0])
    hst, edges = X.histogram(data, 4, (0.0, 4.0))
    assert hst.tolist() == np.histogram(data.numpy(), 4, (0, 4))[0].tolist() == [1, 2, 1, 2]
    assert float((X.histogram(data, 4, (0.0, 4.0), density=True)[0] * 1.0).sum()) == pytest.approx(1.0)
    v, c = X.value_counts(torch.tensor([3, 1, 3, 2, 3, 1]))
    assert v.tolist() == [3, 1, 2] and c.tolist() == [3, 2, 1] and X.bincount(torch.tensor([0, 2, 2]), 4).tolist() == [1, 0, 2, 0]
    assert X.unique(torch.tensor([2, 1, 2]), return_counts=True)[1].tolist() == [1, 2]
    # lazy chains
    base = torch.randn(4, 5)
    lz = X.lazy(base).add_scalar(1).add_scalar(2).mul_scalar(2).mul_scalar(0.5).relu().relu().sub_scalar(0).tanh()
    opt = lz.optimize()
    assert lz.depth() == 8 and [o[0] for o in opt.ops] == ["add_scalar", "relu", "tanh"] and opt.ops[0][1] == 3
    assert torch.allclose(opt.evaluate(), torch.tanh(torch.relu(base + 3))) and torch.allclose(lz.evaluate(), opt.evaluate())
    assert torch.allclose(X.lazy(base).mul(X.lazy(base).exp()).sum(1).evaluate(), (base * base.exp()).sum(1)) and X.lazy(base).transpose(0, 1).reshape(-1).evaluate().shape == (20,)
    # type promotion
    assert X.promote_types(torch.int32, torch.float16) == torch.float16 and X.promote_multiple_types([torch.uint8, torch.int8, torch.bfloat16]) == torch.bfloat16
    assert X.can_cast_safely(torch.int32, torch.int64) and not X.can_cast_safely(torch.float32, torch.int32) and not X.can_cast_safely(torch.int64, torch.int32)
    assert X.get_type_category(torch.bfloat16) == "floating" and X.get_type_precision(torch.int16) == 16 and X.get_type_precision(torch.float64) == 64
    assert X.result_type(torch.ones(2, dtype=torch.int32), 2.5) == torch.float32 and X.result_type(torch.ones(2, dtype=torch.float16), 3) == torch.float16
    assert X.result_type(torch.ones(2, dtype=torch.float16), torch.tensor(1.0, dtype=torch.float64)) == torch.float16
    assert [t.dtype for t in X.promote_tensors(torch.ones(1, dtype=torch.int8), torch.ones(1, dtype=torch.float32))] == [torch.float32] * 2
    assert X.reduction_result_type(torch.int32, "mean") == torch.float32 and X.reduction_result_type(torch.int8, "sum") == torch.int64 and X.reduction_result_type(torch.float16, "sum") == torch.float16
    # fusion analysis
    pats = X.detect_fusible_patterns(["matmul", "add", "relu", "mul", "softmax", "exp", "neg", "tanh", "matmul", "sigmoid", "mul"])
    assert [(p["start"], p["kernel"]) for p in pats] == [(1, "fused_add_relu_mul"), (5, "generated_elementwise"), (9, "fused_sigmoid_mul")]
    est = X.fusion_benefit_estimate(["add", "relu", "mul", "exp"], 1 << 24)
    assert est["speedup"] == pytest.approx(2.0) and est["fused_s"] < est["unfused_s"]
    af = X.AdaptiveFusion(threshold=1.1)
    assert af.should_fuse_adaptive("p")
    af.record_performance("p", 1.0, 1.0); af.record_performance("q", 2.0, 1.0)
    assert not af.should_fuse_adaptive("p") and af.should_fuse_adaptive("q") and af.history_size() == 2
    # optimisation routines on Rosenbrock and a quadratic
    def rosen(v): return (1 - v[0]) ** 2 + 100 * (v[1] - v[0] ** 2) ** 2
    def rgrad(v): return torch.stack([-2 * (1 - v[0]) - 400 * v[0] * (v[1] - v[0] ** 2), 200 * (v[1] - v[0] ** 2)])
    x0 = torch.tensor([-1.2, 1.0], dtype=dd)
    xb, nb = X.bfgs(rosen, rgrad, x0)
    assert torch.allclose(xb, torch.ones(2, dtype=dd), atol=1e-6) and nb < 60
    xc, nc = X.conjugate_gradient_minimize(rosen, rgrad, x0, iters=2000)
    assert torch.allclose(xc, torch.ones(2, dtype=dd), atol=1e-4)
    Q = torch.tensor([[3.0, 1.0], [1.0, 2.0]], dtype=dd); bq = torch.tensor([1.0, -1.0], dtype=dd)
    xg, _ = X.gradient_descent(lambda v: 0.5 * v @ Q @ v - bq @ v, lambda v: Q @ v - bq, torch.zeros(2, dtype=dd), lr=0.3, momentum=0.3)
    assert torch.allclose(xg, torch.linalg.solve(Q, bq), atol=1e-6)
    d0 = -rgrad(x0)
    tb = X.backtracking_line_search(rosen, x0, d0, rgrad(x0))
    tw = X.wolfe_line_search(rosen, rgrad, x0, d0)
    assert rosen(x0 + tb * d0) < rosen(x0) and rosen(x0 + tw * d0) < rosen(x0) and abs(float(rgrad(x0 + tw * d0) @ d0)) <= 0.9 * abs(float(rgrad(x0) @ d0))
    # samplers: moments and Kolmogorov-Smirnov against scipy distributions
    n = 20000
    ks = lambda s, dist: stats.kstest(s.numpy().astype(np.float64), dist.cdf).pvalue
    assert ks(X.exponential((n,), 2.0, seed=0), stats.expon(scale=0.5)) > 1e-3 and ks(X.laplace((n,), 1.0, 2.0, seed=1), stats.laplace(1.0, 2.0)) > 1e-3
    assert ks(X.cauchy((n,), seed=2), stats.cauchy()) > 1e-3 and ks(X.log_normal((n,), 0.0, 0.5, seed=3), stats.lognorm(0.5)) > 1e-3
    assert ks(X.gamma((n,), 2.5, 2.0, seed=4), stats.gamma(2.5, scale=0.5)) > 1e-3 and ks(X.gamma((n,), 0.4, seed=5), stats.gamma(0.4)) > 1e-3
    assert ks(X.beta((n,), 2.0, 5.0, seed=6), stats.beta(2, 5)) > 1e-3 and ks(X.truncated_normal((n,), 0, 1, -1, 2, seed=7), stats.truncnorm(-1, 2)) > 1e-3
    assert float(X.geometric((n,), 0.25, seed=8).mean()) == pytest.approx(4.0, rel=0.05) and float(X.bernoulli((n,), 0.3, seed=9).mean()) == pytest.approx(0.3, abs=0.02)
    assert float(X.poisson((n,), 3.5, seed=10).mean()) == pytest.approx(3.5, rel=0.03) and float(X.binomial((n,), 10, 0.3, seed=11).var()) == pytest.approx(2.1, rel=0.06)
    dr = X.dirichlet(torch.tensor([1.0, 2.0, 3.0]), 5000, seed=12)
    assert torch.allclose(dr.sum(1), torch.ones(5000)) and torch.allclose(dr.mean(0), torch.tensor([1 / 6, 2 / 6, 3 / 6]), atol=0.02)
    cov = torch.tensor([[2.0, 0.6], [0.6, 1.0]])
    mv = X.multivariate_normal(torch.tensor([1.0, -1.0]), cov, n, seed=13)
    assert torch.allclose(torch.cov(mv.t()), cov, atol=0.08) and torch.allclose(mv.mean(0), torch.tensor([1.0, -1.0]), atol=0.05)
    assert torch.equal(X.uniform((5,), seed=3), X.uniform((5,), seed=3)) and sorted(X.randperm(6, seed=0).tolist()) == list(range(6)) and X.randint((9,), 2, 5, seed=0).max() < 5
    assert X.multinomial(torch.tensor([0.0, 1.0]), 4, seed=0).tolist() == [1, 1, 1, 1] and X.normal((3,), seed=1).shape == (3,)


def test_data_samplers_stratified_importance_curriculum_active_and_batching():
    from collections import Counter
    from torsh_b200.data import samplers as S
    torch.manual_seed(0)
    labels = torch.tensor([0] * 60 + [1] * 30 + [2] * 10)
    st = S.StratifiedSampler(labels, seed=0)
    order = list(st)
    assert sorted(order) == list(range(100)) and len(st) == 100
    for s in range(0, 100, 10):                                              # every block of ten holds 6 / 3 / 1
        assert Counter(labels[order[s:s + 10]].tolist()) == {0: 6, 1: 3, 2: 1}
    st.set_epoch(1)
    assert list(st) != order
    sp = S.StratifiedSplit(labels, 0.2)
    assert Counter(labels[sp.val].tolist()) == {0: 12, 1: 6, 2: 2} and not set(sp.val) & set(sp.train) and len(sp.train) == 80
    w = torch.tensor([1.0] * 90 + [10.0] * 10)
    imp = S.ImportanceSampler(w, num_samples=20000, seed=0)
    draws = torch.tensor(list(imp))
    assert float((draws >= 90).float().mean()) == pytest.approx(100 / 190, abs=0.02)
    corr = imp.correction(torch.tensor([0, 95]))
    assert corr[0] == 1.0 and float(corr[1]) == pytest.approx(0.1, rel=1e-3)
    imp.update_weights([0], [1000.0])
    assert float(imp.probabilities()[0]) > 0.8
    flat = S.ImportanceSampler(w, alpha=0.0)
    assert torch.allclose(flat.probabilities(), torch.full((100,), 0.01, dtype=torch.float64))
    diff = torch.rand(100)
    cu = S.CurriculumSampler(diff, 0.2, full_epoch=4, seed=0)
    sizes = []
    for ep in range(6):
        cu.set_epoch(ep)
        idx = list(cu)
        sizes.append(len(idx))
        assert float(diff[idx].max()) <= float(diff.sort().values[len(idx) - 1]) + 1e-9
    assert sizes == [20, 40, 60, 80, 100, 100]
    assert S.CurriculumSampler(diff, 0.2, 4, "root").fraction() == 0.2 and S.CurriculumSampler(diff, 0.2, 4, reverse=True).order[0] == diff.argmax()
    ex = S.CurriculumSampler(diff, 0.2, 4, "exponential"); ex.set_epoch(2)
    li = S.CurriculumSampler(diff, 0.2, 4); li.set_epoch(2)
    assert ex.fraction() < li.fraction()
    probs = torch.tensor([[0.99, 0.01], [0.5, 0.5], [0.7, 0.3], [0.55, 0.45], [0.9, 0.1]])
    for strat in ("uncertainty", "margin", "entropy"):
        al = S.ActiveLearningSampler(5, strat)
        assert al.query(probs, 2) == [1, 3] and al.unlabelled == {0, 2, 4} and al.query(probs, 1) == [2]
    feats = torch.tensor([[0.0, 0], [0.1, 0], [5.0, 5], [0.0, 0.1], [5.1, 5]])
    dv = S.ActiveLearningSampler(5, "diverse")
    pick = dv.query(torch.full((5, 2), 0.5), 2, feats)
    assert len({int(feats[i][0] > 2) for i in pick}) == 2                          # one from each cluster
    assert len(S.ActiveLearningSampler(5, "random").query(probs, 3)) == 3
    ad = S.AdaptiveSampler(10, explore=0.1, seed=0)
    ad.update(list(range(10)), [0.01] * 9 + [5.0])
    ad.update([9], [5.0])
    cnt = Counter()
    for ep in range(200):
        ad.set_epoch(ep)
        cnt.update(ad)
    assert cnt[9] > 5 * max(cnt[i] for i in range(9)) and min(cnt[i] for i in range(9)) > 0
    lengths = torch.randint(5, 100, (200,)).tolist()
    bb = S.BucketBatchSampler(lengths, 8, bucket_size=5, seed=0)
    batches = list(bb)
    assert sorted(i for b in batches for i in b) == list(range(200)) and len(bb) == 25
    spread = sum(max(lengths[i] for i in b) - min(lengths[i] for i in b) for b in batches) / len(batches)
    rand_spread = sum(max(lengths[i:i + 8]) - min(lengths[i:i + 8]) for i in range(0, 200, 8)) / 25
    assert spread < 0.5 * rand_spread
    tok = list(S.BucketBatchSampler(lengths, 64, bucket_size=100, max_tokens=400, seed=0))
    assert all(len(b) * max(lengths[i] for i in b) <= 400 for b in tok) and sorted(i for b in tok for i in b) == list(range(200))
    bal = S.BalancedBatchSampler(labels, classes_per_batch=2, samples_per_class=4, num_batches=5)
    for b in bal:
        c = Counter(labels[b].tolist())
        assert len(b) == 8 and len(c) == 2 and set(c.values()) == {4}
    wc = Counter(labels[list(S.WeightedClassSampler(labels, 6000, seed=0))].tolist())
    assert all(abs(wc[c] - 2000) < 200 for c in range(3))
    assert sorted(S.SubsetRandomSampler([3, 5, 7])) == [3, 5, 7]
    it = iter(S.InfiniteSampler(4, seed=0))
    first8 = [next(it) for _ in range(8)]
    assert sorted(first8[:4]) == sorted(first8[4:]) == [0, 1, 2, 3]


def test_data_pipeline_transforms_datasets_text_sql_privacy_federated_and_collate(tmp_path):
    import sqlite3
    import numpy as np
    from collections import Counter
    from torsh_b200.data import pipeline as P
    torch.manual_seed(0)
    # transform algebra
    t = P.Lambda(lambda x: x + 1, "inc") | P.Lambda(lambda x: x * 2, "dbl").when(lambda x: x.sum() > 0) | P.ToType(torch.float64)
    assert t(torch.tensor([1.0])).tolist() == [4.0] and t(torch.tensor([-5.0])).tolist() == [-4.0] and t(torch.tensor([1.0])).dtype == torch.float64 and "inc" in repr(t)
    assert torch.allclose(P.Normalize([1.0, 2.0], [2.0, 4.0])(torch.ones(2, 3, 3)), torch.tensor([0.0, -0.25]).reshape(2, 1, 1).expand(2, 3, 3))
    coin = P.Lambda(lambda x: x + 1).with_probability(0.5, seed=0)
    assert 30 < sum(int(coin(torch.zeros(()))) for _ in range(100)) < 70
    # datasets
    ds = P.TensorDataset(torch.arange(10.0), torch.arange(10))
    assert len(ds) == 10 and ds[3] == (torch.tensor(3.0), torch.tensor(3))
    with pytest.raises(ValueError):
        P.TensorDataset(torch.zeros(3), torch.zeros(4))
    td = P.TransformedDataset(ds, lambda x: x * 10, lambda y: y + 100)
    assert td[2] == (torch.tensor(20.0), torch.tensor(102))
    assert list(P.ChainDataset([1, 2], [3])) == [1, 2, 3]
    inf = iter(P.InfiniteDataset(P.TensorDataset(torch.arange(3)), shuffle=True))
    got = [int(next(inf)) for _ in range(9)]
    assert sorted(got[:3]) == sorted(got[3:6]) == [0, 1, 2]
    sh = list(P.BufferedStreamingDataset(range(100), 20, seed=0))
    assert sorted(sh) == list(range(100)) and sh != list(range(100)) and max(abs(v - i) for i, v in enumerate(sh)) < 100
    pipe = P.DataPipeline(range(100)).filter(lambda v: v % 2 == 0).map(lambda v: v * v).skip(2).take(7).batch(3)
    assert list(pipe) == [[16, 36, 64], [100, 144, 196], [256]] and list(P.DataPipeline(range(10)).shard(3, 1)) == [1, 4, 7]
    assert list(P.DataPipeline(range(7)).batch(3, drop_last=True, collate=sum)) == [3, 12] and sorted(P.DataPipeline(range(20)).shuffle(5)) == list(range(20))
    clock = iter(np.arange(0, 100, 0.5))
    pr = P.ProfiledDataset(ds, clock=lambda: float(next(clock)))
    _ = [pr[i] for i in (1, 2, 1)]
    assert pr.stats()["count"] == 3 and pr.stats()["mean"] == 0.5 and pr.stats()["total"] == 1.5
    rt = P.RealTimeDataset(capacity=3)
    for i in range(5):
        rt.push(i)
    rt.close()
    assert list(rt) == [2, 3, 4] and rt.dropped == 2
    shm = P.SharedMemoryDataset(torch.randn(8, 4), torch.arange(8))
    assert shm.is_shared() and shm[5][1] == 5
    parts = P.random_split(ds, [0.7, 0.3], seed=0)
    assert [len(p) for p in parts] == [7, 3] and sorted(int(p[i][1]) for p in parts for i in range(len(p))) == list(range(10))
    # text cleaning; Porter stemmer against the algorithm's published vocabulary pairs
    st = P.PorterStemmer()
    pairs = {"caresses": "caress", "ponies": "poni", "cats": "cat", "feed": "feed", "agreed": "agre", "plastered": "plaster", "motoring": "motor", "sing": "sing",
             "conflated": "conflat", "troubled": "troubl", "sized": "size", "hopping": "hop", "falling": "fall", "hissing": "hiss", "filing": "file", "happy": "happi",
             "relational": "relat", "conditional": "condit", "rational": "ration", "digitizer": "digit", "operator": "oper", "feudalism": "feudal", "decisiveness": "decis",
             "hopefulness": "hope", "formaliti": "formal", "triplicate": "triplic", "formative": "form", "electrical": "electr", "goodness": "good", "revival": "reviv",
             "allowance": "allow", "inference": "infer", "adjustable": "adjust", "replacement": "replac", "adoption": "adopt", "activate": "activ", "effective": "effect",
             "probate": "probat", "rate": "rate", "cease": "ceas", "controll": "control", "roll": "roll", "generalization": "gener", "running": "run"}
    wrong = {w: (st.stem(w), s) for w, s in pairs.items() if st.stem(w) != s}
    assert not wrong, wrong
    tp = P.TextPipeline().lowercase().remove_punctuation().remove_numbers().collapse_whitespace().tokenize().remove_stopwords().filter_by_length(3).stem()
    assert tp("The 3 quick foxes  were JUMPING over the lazy dogs!") == ["quick", "fox", "jump", "over", "lazi", "dog"]
    assert P.TextPipeline().tokenize().ngrams(2)("a b c") == ["a b", "b c"] and P.TextPipeline().replace_pattern(r"\d+", "<n>")("room 42") == "room <n>"
    # augmentation schedules
    pa = P.ProgressiveAugmentation(lambda s: (lambda x: x * (1 + s)), 0.0, 1.0, total_steps=10, mode="linear")
    vals = []
    for _ in range(12):
        vals.append(pa.strength()); pa.step()
    assert vals[0] == 0 and vals[5] == 0.5 and vals[-1] == 1.0 and float(pa(torch.ones(()))) == 2.0
    cosv = P.ProgressiveAugmentation(None, 0, 1, 10, "cosine"); cosv.step_count = 5
    stp = P.ProgressiveAugmentation(None, 0, 1, 10, "step", steps=2); stp.step_count = 4
    assert cosv.strength() == pytest.approx(0.5) and stp.strength() == 0.0
    aa = P.AdaptiveAugmentation(lambda s: (lambda x: x), strength=0.3, target_gap=0.05, rate=0.1)
    aa.update(0.95, 0.80); aa.update(0.95, 0.82)
    assert aa.strength == pytest.approx(0.5)
    aa.update(0.85, 0.84)
    assert aa.strength == pytest.approx(0.4) and len(aa.history) == 3
    ap = P.AugmentationPipeline(seed=0).add("flip", lambda x: x.flip(-1), 0.5).add("scale", lambda x: x * 2, 1.0)
    outs = [ap(torch.tensor([1.0, 2.0])) for _ in range(40)]
    assert ap.stats["scale"] == 40 and 10 < ap.stats["flip"] < 30 and all(o.sum() == 6 for o in outs)
    # SQL dataset
    conn = sqlite3.connect(":memory:")
    conn.execute("CREATE TABLE samples (id INTEGER PRIMARY KEY, a REAL, b REAL, label INTEGER, split TEXT)")
    conn.executemany("INSERT INTO samples VALUES (?, ?, ?, ?, ?)", [(i, i * 0.5, -i, i % 3, "train" if i % 5 else "val") for i in range(50)])
    db = P.DatabaseDataset(conn, "samples", ["a", "b"], "label", key="id", where="split = 'train'", page_size=8, cache_pages=2)
    assert len(db) == 40 and db[0][0].tolist() == [0.5, -1.0] and db[0][1] == 1 and db[39][0].tolist() == [24.5, -49.0]
    q0 = db.queries
    _ = [db[i] for i in range(8)]
    assert db.queries == q0 and len(db.cache) <= 2
    _ = [db[i] for i in (0, 10, 20, 30, 0)]
    assert db.queries == q0 + 4
    with pytest.raises(ValueError):
        P.DatabaseDataset(conn, "samples; DROP TABLE samples", ["a"])
    # privacy
    bud = P.PrivacyBudget(1.0)
    bud.spend(0.4); bud.spend(0.4)
    with pytest.raises(PermissionError):
        bud.spend(0.4)
    assert bud.remaining()[0] == pytest.approx(0.2) and len(bud.spent) == 2
    adv = P.PrivacyBudget(100.0, 1e-3, "advanced", 1e-6)
    for _ in range(100):
        adv.spend(0.1)
    assert adv.consumed()[0] < 100 * 0.1 and adv.consumed()[1] == pytest.approx(1e-6)
    g = torch.Generator().manual_seed(0)
    lap = P.laplace_mechanism(torch.zeros(20000), 1.0, 0.5, g)
    assert float(lap.abs().mean()) == pytest.approx(2.0, rel=0.05)
    gau = P.gaussian_mechanism(torch.zeros(20000), 1.0, 0.5, 1e-5, g)
    assert float(gau.std()) == pytest.approx(np.sqrt(2 * np.log(1.25e5)) / 0.5, rel=0.05)
    bits = torch.rand(20000, generator=g) < 0.3
    noisy, est = P.randomized_response(bits, 1.0, g)
    assert est == pytest.approx(0.3, abs=0.03) and 0.2 < float((noisy != bits).float().mean()) < 0.35
    ages = torch.randint(18, 90, (5000,)).float()
    pd_ = P.PrivateDataset(ages, 0, 100, P.PrivacyBudget(3.0), seed=0)
    assert pd_.mean(1.0) == pytest.approx(float(ages.mean()), abs=0.5) and pd_.count(lambda d: d > 65, 1.0) == pytest.approx(float((ages > 65).sum()), abs=15)
    assert pd_.histogram(10, 1.0).shape == (10,)
    with pytest.raises(PermissionError):
        pd_.sum(0.5)
    # federated partitions and aggregation
    labels = torch.arange(1000) % 10
    iid = P.partition_iid(1000, 10)
    assert sorted(i for p in iid for i in p) == list(range(1000)) and all(len(p) == 100 for p in iid)
    skew = P.partition_dirichlet(labels, 10, alpha=0.1, seed=0)
    assert sorted(i for p in skew for i in p) == list(range(1000))
    fd_iid, fd_skew = P.FederatedDataset(labels, iid), P.FederatedDataset(labels, skew)
    ent = lambda d: float(-(d * d.clamp(min=1e-12).log()).sum(1).mean())
    assert ent(fd_skew.label_distribution(labels)) < 0.6 * ent(fd_iid.label_distribution(labels))
    shards = P.partition_shards(labels, 10, 2, seed=0)
    assert all(len(set(labels[p].tolist())) <= 3 for p in shards) and sorted(i for p in shards for i in p) == list(range(1000))
    caps = [{"compute": 1.0 + k, "bandwidth": 1.0} for k in range(10)]
    fd = P.FederatedDataset(labels, iid, caps)
    assert fd.select_clients(3, "capable") == [9, 8, 7] and len(set(fd.select_clients(4, "random"))) == 4 and len(fd.client(2)) == 100
    assert len(set(fd.select_clients(5, "weighted"))) == 5
    states = [{"w": torch.full((3,), float(v))} for v in (1, 2, 3, 100)]
    assert P.federated_average(states[:3], [1, 1, 2])["w"].tolist() == [2.25] * 3
    assert P.federated_average(states, strategy="median")["w"].tolist() == [2.0] * 3 and P.federated_average(states, strategy="trimmed_mean", trim=0.25)["w"].tolist() == [2.5] * 3
    # pooled buffers, memory-mapped batches, device-side preprocessing
    pool = P.TensorPool()
    a = pool.acquire((4, 8)); pool.release(a)
    b = pool.acquire((4, 8)); c = pool.acquire((4, 8))
    assert b is a and c is not a and pool.allocated == 2 and pool.reused == 1
    arr = np.arange(100 * 6, dtype=np.float32).reshape(100, 6)
    np.save(tmp_path / "x.npy", arr)
    mm = P.MemoryMappedLoader(tmp_path / "x.npy", 32)
    assert len(mm) == 4 and [len(b) for b in mm] == [32, 32, 32, 4] and np.array_equal(mm.batch(1).numpy(), arr[32:64]) and np.array_equal(mm.gather([5, 2]).numpy(), arr[[2, 5]])
    u8 = torch.randint(0, 256, (4, 20, 24, 3), dtype=torch.uint8)
    dp = P.DevicePreprocessingPipeline("cpu", size=(10, 12), flip_p=0.0)
    out = dp(u8)
    ref = torch.nn.functional.interpolate(u8.permute(0, 3, 1, 2).float() / 255, size=(10, 12), mode="bilinear", antialias=True, align_corners=False)
    assert out.shape == (4, 3, 10, 12) and torch.allclose(out, (ref - dp.mean) / dp.std, atol=1e-6) and dp.bytes_uploaded == u8.numel()
    flipped = P.DevicePreprocessingPipeline("cpu", flip_p=1.0)(u8)
    assert torch.allclose(flipped, P.DevicePreprocessingPipeline("cpu")(u8).flip(-1))
    # collation
    seqs = [(torch.arange(1, 4), 0), (torch.arange(1, 6), 1), (torch.arange(1, 2), 0)]
    padded, lens, mask, ys = P.pad_sequence_collate(seqs, pad_to_multiple=4)
    assert padded.shape == (3, 8) and lens.tolist() == [3, 5, 1] and mask.sum(1).tolist() == [3, 5, 1] and padded[0].tolist() == [1, 2, 3, 0, 0, 0, 0, 0] and ys.tolist() == [0, 1, 0]
    lp, _, lm = P.pad_sequence_collate([s for s, _ in seqs], left=True)
    assert lp[0].tolist() == [0, 0, 1, 2, 3] and lm[0].tolist() == [False, False, True, True, True]
    nc = P.nested_collate([{"x": torch.ones(2), "meta": {"id": 1, "name": "a"}, "rag": torch.ones(1)}, {"x": torch.zeros(2), "meta": {"id": 2, "name": "b"}, "rag": torch.ones(3)}])
    assert nc["x"].shape == (2, 2) and nc["meta"]["id"].tolist() == [1, 2] and nc["meta"]["name"] == ["a", "b"] and isinstance(nc["rag"], list)
    assert P.nested_collate([(torch.ones(2), 1.0), (torch.ones(2), 2.0)])[1].tolist() == [1.0, 2.0]


def test_nn_research_layers_capsules_hopfield_sparse_training_and_fused_blocks():
    import math
    from torsh_b200.nn import research as R
    torch.manual_seed(0)
    # Neural ODE: dx/dt = a x integrates to exp(a); rk4 is far more accurate than euler at equal steps; gradients reach a
    a = torch.nn.Parameter(torch.tensor(0.7))
    f = lambda t, x: a * x
    x0 = torch.ones(3)
    rk, eu = R.NeuralODE(f, steps=10)(x0), R.NeuralODE(f, steps=10, method="euler")(x0)
    assert abs(rk[0].item() - math.exp(0.7)) < 1e-6 < abs(eu[0].item() - math.exp(0.7)) and abs(R.NeuralODE(f, steps=10, method="midpoint")(x0)[0].item() - math.exp(0.7)) < 2e-3
    rk.sum().backward()
    assert float(a.grad) == pytest.approx(3 * math.exp(0.7), rel=1e-5) and R.NeuralODE(f, steps=4)(x0, True).shape == (5, 3)
    # capsules: outputs have norm < 1, coupling coefficients are a distribution over output capsules, routing sharpens them
    caps = R.CapsuleLayer(12, 8, 4, 6, routing_iters=3)
    with torch.no_grad():
        caps.w.mul_(30)
    v = caps(torch.randn(5, 12, 8))
    assert v.shape == (5, 4, 6) and v.norm(dim=-1).max() < 1 and torch.allclose(caps.coupling.sum(2), torch.ones(5, 12), atol=1e-5)
    one = R.CapsuleLayer(12, 8, 4, 6, routing_iters=1); one.w = caps.w
    one(torch.randn(5, 12, 8))
    assert caps.coupling.max() > one.coupling.max() == pytest.approx(0.25)
    s = R.squash(torch.tensor([[3.0, 4.0]]))
    assert float(s.norm()) == pytest.approx(25 / 26, rel=1e-5)
    se = R.SEBlock(16, 4)
    xi = torch.randn(2, 16, 5, 5)
    assert se(xi).shape == xi.shape and ((se(xi) / xi).flatten(2).std(-1) < 1e-5).all()                       # one scale per channel
    ip = R.IPAdapterCrossAttention(32, 24, heads=4, image_ctx_dim=20, scale=0.0)
    q, txt, im = torch.randn(2, 7, 32), torch.randn(2, 5, 24), torch.randn(2, 3, 20)
    base = ip(q, txt, im)
    assert torch.equal(base, ip(q, txt)) and base.shape == (2, 7, 32)
    ip.scale = 1.0
    assert not torch.allclose(ip(q, txt, im), base)
    seq = torch.randn(2, 12, 10)
    assert torch.equal(R.PixelUnshuffle1d(3)(R.PixelShuffle1d(3)(seq)), seq) and R.PixelShuffle1d(3)(seq).shape == (2, 4, 30)
    assert R.PixelShuffle1d(2)(torch.arange(4.0).reshape(1, 2, 2)).flatten().tolist() == [0, 2, 1, 3]
    dc = R.DropConnect(64, 64, p=0.5)
    xin = torch.randn(512, 64)
    dc.eval(); ref = dc(xin)
    dc.train(); outs = torch.stack([dc(xin) for _ in range(40)]).mean(0)
    assert torch.allclose(outs, ref, atol=0.5) and not torch.equal(dc(xin), dc(xin)) and float((outs - ref).abs().mean()) < 0.15
    co = R.Cutout(5).train()
    y = co(torch.ones(8, 3, 16, 16))
    holes = (y == 0).float().sum((1, 2, 3)) / 3
    assert (holes >= 9).all() and (holes <= 25).all() and torch.equal(co.eval()(torch.ones(1, 3, 4, 4)), torch.ones(1, 3, 4, 4))
    # custom RNN equals torch's LSTM when driven by an LSTMCell with the same weights; reversed pass flips time
    lstm = torch.nn.LSTM(6, 8, batch_first=True)
    cell = torch.nn.LSTMCell(6, 8)
    cell.weight_ih, cell.weight_hh, cell.bias_ih, cell.bias_hh = lstm.weight_ih_l0, lstm.weight_hh_l0, lstm.bias_ih_l0, lstm.bias_hh_l0
    wrap = lambda x, st: (lambda hc: (hc[0], hc))(cell(x, st))
    xs = torch.randn(3, 5, 6)
    assert torch.allclose(R.CustomRNN(wrap)(xs)[0], lstm(xs)[0], atol=1e-6)
    assert torch.allclose(R.CustomRNN(wrap, reverse=True)(xs)[0], lstm(xs.flip(1))[0].flip(1), atol=1e-6)
    cl = R.ConvLSTM(2, 4)
    out, (h, c) = cl(torch.randn(2, 6, 2, 8, 8))
    assert out.shape == (2, 6, 4, 8, 8) and torch.equal(out[:, -1], h) and c.abs().max() < 6
    # Hopfield retrieval completes a corrupted pattern
    pats = torch.sign(torch.randn(6, 64))
    noisy = pats[2].clone(); noisy[:16] *= -1
    hp = R.HopfieldLayer(64, beta=1.0)
    rec = hp(noisy[None], pats)
    assert torch.equal(torch.sign(rec[0]), pats[2]) and R.HopfieldLayer(64, project=True)(noisy[None], pats).shape == (1, 64)
    # hyper-network: different conditioning vectors give different linear maps; gradients reach the generator
    hl = R.HyperLinear(4, 10, 3)
    z = torch.randn(2, 4)
    xh = torch.randn(2, 7, 10)
    yh = hl(xh, z)
    p = hl.net(z)
    manual = torch.einsum("oi,ti->to", p[1, :30].reshape(3, 10), xh[1]) + p[1, 30:]
    assert yh.shape == (2, 7, 3) and torch.allclose(yh[1], manual, atol=1e-6)
    yh.sum().backward()
    assert hl.net[0].weight.grad.abs().sum() > 0
    # adaptive softmax: a proper distribution, loss equals the NLL read from the full table
    ah = R.AdaptiveSoftmaxHead(32, 100, [10, 40])
    feats, tg = torch.randn(50, 32), torch.randint(0, 100, (50,))
    lp = ah.log_prob(feats)
    assert lp.shape == (50, 100) and torch.allclose(lp.exp().sum(1), torch.ones(50), atol=1e-5)
    assert ah(feats, tg).item() == pytest.approx(-lp.gather(1, tg[:, None]).mean().item(), rel=1e-5)
    assert sum(p.numel() for p in ah.parameters()) < 32 * 100
    # sparse layers: masks hold through training, gradual schedule follows the cubic ramp
    sl = R.SparseLinear(20, 10, sparsity=0.5)
    assert sl.sparsity() == pytest.approx(0.5) and float((sl.weight * sl.mask == 0).float().mean()) >= 0.5
    opt = torch.optim.SGD(sl.parameters(), 0.1)
    dead = sl.mask == 0
    w_dead = sl.weight.detach()[dead].clone()
    for _ in range(5):
        opt.zero_grad(); sl(torch.randn(8, 20)).pow(2).sum().backward(); opt.step()
    assert torch.equal(sl.weight.detach()[dead], w_dead) and sl.weight.grad[dead].abs().sum() == 0
    sl.prune_to(0.8)
    assert sl.sparsity() == pytest.approx(0.8) and (sl.mask[dead] == 0).all()
    sc = R.SparseConv2d(3, 8, 3, sparsity=0.75)
    assert sc.sparsity() == pytest.approx(0.75, abs=0.01) and sc(torch.randn(1, 3, 6, 6)).shape == (1, 8, 4, 4)
    net = torch.nn.Sequential(R.SparseLinear(16, 16), torch.nn.ReLU(), R.SparseLinear(16, 4))
    gp = R.GradualPruningScheduler(net, final_sparsity=0.9, begin_step=10, end_step=110, frequency=10)
    assert gp.target(0) == 0 and gp.target(60) == pytest.approx(0.9 * (1 - 0.5 ** 3)) and gp.target(500) == pytest.approx(0.9)
    hist = []
    for _ in range(130):
        gp.step(); hist.append(net[0].sparsity())
    assert hist[5] == 0 and hist[-1] == pytest.approx(0.9, abs=0.01) and all(b >= a for a, b in zip(hist, hist[1:])) and 0.5 < hist[40] < 0.8
    # lazily shaped and fused blocks
    lz = R.LazyLinear(5)
    assert not lz.is_initialized() and lz(torch.randn(3, 11)).shape == (3, 5) and lz.inner.in_features == 11 and len(list(lz.parameters())) == 2
    fl = R.FusedLinearActivation(8, 4, "gelu")
    xin = torch.randn(3, 8)
    assert torch.allclose(fl(xin), torch.nn.functional.gelu(fl.lin(xin), approximate="tanh"))
    mlp = R.StaticMLP([8, 16, 16, 2], "relu")
    assert mlp(xin).shape == (3, 2) and [m.activation for m in mlp] == ["relu", "relu", "none"]


def test_nn_tools_stability_export_conversion_zoo_update_policies_and_recording(tmp_path):
    import math
    from torsh_b200.nn import tools as T
    torch.manual_seed(0)
    # stability: a naive softmax overflows on huge inputs, the built-in one does not
    class Naive(torch.nn.Module):
        def forward(self, x): e = torch.exp(x); return e / e.sum(-1, keepdim=True)
    rep_bad, rep_ok = T.StabilityTester().test(Naive(), (4, 16)), T.StabilityTester().test(torch.nn.Softmax(-1), (4, 16))
    assert not rep_bad["passed"] and ("huge", "float32") in rep_bad["failed_cases"] and rep_ok["passed"] and len(rep_ok["results"]) == 7
    half = T.StabilityTester(dtypes=(torch.float32, torch.bfloat16)).test(torch.nn.Sequential(torch.nn.Linear(16, 8), torch.nn.LayerNorm(8)), (4, 16))
    assert half["passed"] and len(half["results"]) == 14 and half["worst_sensitivity"] < 100
    # deployment optimisation keeps outputs, folds conv+bn, removes dropout
    net = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.BatchNorm2d(8), torch.nn.ReLU(), torch.nn.Dropout(0.5), torch.nn.Conv2d(8, 4, 1)).eval()
    net[1].running_mean.normal_(); net[1].running_var.uniform_(0.5, 2)
    x = torch.randn(2, 3, 8, 8)
    opt, rep = T.DeploymentOptimizer().optimize(net)
    assert rep == {"folded_conv_bn": 1, "fused_activation": 1, "removed_dropout": 1, "traced": True} and torch.allclose(opt(x), net(x), atol=1e-5)
    assert not any(p.requires_grad for p in opt.parameters()) and T.DeploymentOptimizer().optimize(net, torch.bfloat16)[0](x.bfloat16()).dtype == torch.bfloat16
    # export formats: sizes, checksums, round trip
    mlp = torch.nn.Sequential(torch.nn.Linear(6, 12), torch.nn.ReLU(), torch.nn.Linear(12, 3))
    ex = T.ModelExporter()
    recs = ex.benchmark(mlp, torch.randn(1, 6), out_dir=tmp_path)
    assert [r["format"] for r in recs][-1] == "json" and all(r["parameters"] == 6 * 12 + 12 + 12 * 3 + 3 and len(r["sha256"]) == 64 for r in recs)
    from torsh_b200.serialize import model_state as ms
    again = torch.nn.Sequential(torch.nn.Linear(6, 12), torch.nn.ReLU(), torch.nn.Linear(12, 3))
    ms.load_model_state(again, ms.load_safetensors(tmp_path / "model.safetensors"))
    xin = torch.randn(4, 6)
    assert torch.equal(again(xin), mlp(xin))
    ts = ex.export(mlp, tmp_path / "m.pt", "torchscript", torch.randn(1, 6))
    assert ts["bytes"] > 0 and torch.allclose(torch.jit.load(str(tmp_path / "m.pt"))(xin), mlp(xin))
    onx = ex.export(mlp, tmp_path / "m.onnx", "onnx", (torch.randn(1, 6),))
    assert onx["bytes"] > 300
    with pytest.raises(ValueError):
        ex.export(mlp, tmp_path / "m.x", "coreml")
    # TensorFlow-style checkpoint into a PyTorch-layout model
    conv = torch.nn.Sequential()
    conv.add_module("block", torch.nn.Sequential())
    conv.block.add_module("conv", torch.nn.Conv2d(3, 5, 3))
    conv.block.add_module("bn", torch.nn.BatchNorm2d(5))
    conv.add_module("head", torch.nn.Linear(5, 2))
    tfw = {"block/conv/kernel:0": torch.randn(3, 3, 3, 5), "block/conv/bias:0": torch.randn(5), "block/bn/gamma:0": torch.rand(5), "block/bn/beta:0": torch.randn(5),
           "block/bn/moving_mean:0": torch.randn(5), "block/bn/moving_variance:0": torch.rand(5), "head/kernel:0": torch.randn(5, 2), "head/bias:0": torch.randn(2), "extra/w:0": torch.zeros(1)}
    mc = T.ModelConverter()
    st = mc.from_tensorflow(tfw)
    assert st["block.conv.weight"].shape == (5, 3, 3, 3) and torch.equal(st["block.conv.weight"][4, 2, 1, 0], tfw["block/conv/kernel:0"][1, 0, 2, 4]) and torch.equal(st["head.weight"], tfw["head/kernel:0"].t())
    fit = mc.fit(conv, st)
    assert fit["unexpected"] == ["extra.w"] and fit["missing"] == ["block.bn.num_batches_tracked"] and not fit["shape_mismatch"] and torch.equal(conv.block.bn.running_var, tfw["block/bn/moving_variance:0"])
    assert mc.rename({"encoder.layer.0.w": 1}, [(r"^encoder\.layer\.", "blocks.")]) == {"blocks.0.w": 1} and mc.describe(conv)[0]["name"] == "block"
    bad = dict(st); bad["head.weight"] = torch.zeros(3, 3)
    assert mc.fit(conv, bad)["shape_mismatch"] == ["head.weight"]
    src, notes = T.MigrationHelper().migrate_source("m = tf.keras.layers.Dense(4)\no = torch.optim.AdamW(p)\nz = tf.signal.fft(x)\n")
    assert "torsh_b200.nn.Linear(4)" in src and "torsh_b200.optim.AdamW" in src and "no mapping for tf.signal.fft" in notes
    # zoo
    zoo = T.ModelZoo(tmp_path / "zoo")
    zoo.register("tiny_mlp", lambda width=12: torch.nn.Sequential(torch.nn.Linear(6, width), torch.nn.ReLU(), torch.nn.Linear(width, 3)), {"width": 12}, "test model")
    info = zoo.save_weights("tiny_mlp", mlp, "v1", {"acc": 0.9})
    assert zoo.list_models() == ["tiny_mlp"] and zoo.available_weights("tiny_mlp") == ["v1"] and info["parameters"] == 123
    assert torch.equal(zoo.create("tiny_mlp", "v1")(xin), mlp(xin)) and zoo.create("tiny_mlp", width=20)[0].out_features == 20
    wf = tmp_path / "zoo" / "tiny_mlp" / "v1.safetensors"
    wf.write_bytes(wf.read_bytes()[:-4] + b"\0\0\0\0")
    with pytest.raises(IOError):
        zoo.create("tiny_mlp", "v1")
    # network report
    rp = T.NetworkOptimizer().analyze(net, x)
    assert rp["total_flops"] == 2 * (2 * 8 * 8 * 8) * 27 + 2 * (2 * 4 * 8 * 8) * 8 and any("folded" in f for f in rp["findings"]) and any("FLOPs" in f for f in rp["findings"])
    assert rp["total_params"] == sum(p.numel() for p in net.parameters())
    # per-layer policies
    model = torch.nn.ModuleDict({"embed": torch.nn.Embedding(10, 8), "blocks": torch.nn.ModuleList([torch.nn.Linear(8, 8) for _ in range(3)]), "head": torch.nn.Linear(8, 2)})
    ls = T.LayerSpecificOptimizers(model, [(r"^embed", {"freeze": True}), (r"bias$", {"weight_decay": 0.0}), (r"^head", {"lr_mult": 10.0})])
    groups = ls.param_groups(1e-3, weight_decay=0.1)
    by = {tuple(g["names"]): g for g in groups}
    assert not model["embed"].weight.requires_grad and by[("head.weight",)]["lr"] == pytest.approx(1e-2) and by[("head.weight",)]["weight_decay"] == 0.1
    assert any(g["weight_decay"] == 0.0 and "blocks.0.bias" in g["names"] and "head.bias" in g["names"] for g in groups)
    torch.optim.AdamW([{k: v for k, v in g.items() if k != "names"} for g in groups])
    lw = T.LayerSpecificOptimizers.layerwise_decay(model, 1.0, 0.5)
    lr_of = {n: g["lr"] for g in lw for n in g["names"]}
    assert lr_of["head.weight"] == 1.0 and lr_of["blocks.2.weight"] == 1.0 and lr_of["blocks.1.bias"] == 0.5 and lr_of["blocks.0.weight"] == 0.25 and lr_of["embed.weight"] == 0.125
    w = torch.nn.Parameter(torch.ones(2, 4))
    up = T.ParameterUpdater([w], lr=1.0, clip_value=0.5, max_weight_norm=1.0, ema_decay=0.5)
    w.grad = torch.tensor([[2.0, -2.0, 0.1, 0.0], [0.0, 0.0, 0.0, 0.0]])
    up.step()
    assert up.stats["value_clipped"] == 2 and up.stats["weights_rescaled"] == 2 and torch.allclose(w.detach().norm(dim=1), torch.ones(2), atol=1e-6)
    assert torch.allclose(up.ema[0], 0.5 * torch.ones(2, 4) + 0.5 * w.detach())
    live = w.detach().clone(); up.swap_in_ema()
    assert torch.allclose(w.detach(), 0.5 + 0.5 * live); up.swap_in_ema()
    assert torch.equal(w.detach(), live)
    nc = T.ParameterUpdater([w], lr=0.0, clip_norm=1.0); w.grad = torch.full((2, 4), 10.0); nc.step()
    assert nc.stats["norm_clipped"] == 1 and float(w.grad.norm()) == pytest.approx(1.0, rel=1e-4)
    # recording hooks flag a dead ReLU
    dead = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.ReLU(), torch.nn.Linear(8, 1))
    with torch.no_grad():
        dead[0].bias.fill_(-100.0)
    rec = T.ActivationRecorder(dead)
    dead(torch.randn(16, 4)).sum().backward()
    assert rec.stats["1"]["zero_fraction"] == 1.0 and any(f.startswith("1:") for f in rec.findings()) and any("vanishes" in f for f in rec.findings()) and set(rec.grads) == {"0", "1", "2"}
    rec.remove(); rec.stats.clear()
    dead(torch.randn(2, 4))
    assert not rec.stats


def test_series_ext_tests_stl_sarima_filters_changepoints_modes_imputation_cv_and_forecasters():
    import math
    import numpy as np
    from scipy import stats as sst
    from torsh_b200 import series_ext as E
    g = torch.Generator().manual_seed(0)
    rn = lambda n, s=1.0: torch.randn(n, generator=g, dtype=torch.float64) * s
    n = 400
    white, walk = rn(n), rn(n).cumsum(0)
    # stationarity and diagnostics
    assert E.adf_test(white)["stationary"] and not E.adf_test(walk)["stationary"] and E.kpss_test(white)["stationary"] and not E.kpss_test(walk)["stationary"]
    assert E.stationarity_suite(white)["verdict"] == "stationary" and E.stationarity_suite(walk)["verdict"] == "unit_root" and E.stationarity_suite(walk)["suggested_differences"] == 1
    assert E.adf_test(torch.arange(n, dtype=torch.float64) * 0.1 + white, regression="ct")["stationary"]
    ar = torch.zeros(n, dtype=torch.float64)
    for t in range(1, n):
        ar[t] = 0.8 * ar[t - 1] + white[t]
    assert E.ljung_box(white)["white_noise"] and not E.ljung_box(ar)["white_noise"] and E.ljung_box(ar)["p_value"] < 1e-6
    jb = E.jarque_bera(white)
    ref = sst.jarque_bera(white.numpy())
    assert jb["statistic"] == pytest.approx(ref.statistic, rel=1e-6) and jb["p_value"] == pytest.approx(ref.pvalue, rel=1e-5) and jb["normal"] and not E.jarque_bera(white.exp())["normal"]
    rd = E.residual_diagnostics(white)
    assert rd["homoscedastic"] and abs(rd["mean"]) < 0.2 and not E.residual_diagnostics(white * torch.linspace(0.2, 3, n, dtype=torch.float64))["homoscedastic"]
    drive = rn(n)
    resp = torch.zeros(n, dtype=torch.float64)
    for t in range(2, n):
        resp[t] = 0.3 * resp[t - 1] + 0.8 * drive[t - 1] + 0.3 * rn(1)[0]
    assert E.granger_causality(resp, drive)["causes"] and not E.granger_causality(drive, resp)["causes"]
    assert E.transfer_entropy(drive, resp) > 5 * max(E.transfer_entropy(resp, drive), 1e-3) and E.transfer_entropy(drive, resp) > 0.1
    # STL
    tt = torch.arange(240, dtype=torch.float64)
    trend, seas = 0.05 * tt + 3, 2 * torch.sin(2 * math.pi * tt / 12)
    y = trend + seas + rn(240, 0.2)
    d = E.stl(y, 12)
    assert float((d["trend"] - trend)[12:-12].abs().mean()) < 0.15 and float((d["seasonal"] - seas)[12:-12].abs().mean()) < 0.2
    assert torch.allclose(d["trend"] + d["seasonal"] + d["remainder"], y) and float(d["remainder"].std()) < 0.35
    spiky = y.clone(); spiky[[50, 120, 190]] += 15
    plain, rob = E.stl(spiky, 12), E.stl(spiky, 12, robust=True)
    assert float((rob["seasonal"] - seas)[12:-12].abs().max()) < float((plain["seasonal"] - seas)[12:-12].abs().max()) and rob["weights"][[50, 120, 190]].max() < 0.05
    # seasonal ARIMA
    m = E.SARIMA((1, 0, 0)).fit(ar)
    assert float(m.params[0]) == pytest.approx(0.8, abs=0.08) and m.sigma2 == pytest.approx(1.0, abs=0.2) and E.ljung_box(m.residuals, 10, 1)["white_noise"]
    fc = m.forecast(3)
    mu, phi = float(m.params[-1]), float(m.params[0])
    assert float(fc[0]) == pytest.approx(mu + phi * (float(ar[-1]) - mu), abs=1e-6) and abs(float(fc[2]) - mu) < abs(float(fc[0]) - mu) + 1e-9
    ma_series = white[1:] + 0.6 * white[:-1]
    mm = E.SARIMA((0, 0, 1)).fit(ma_series)
    assert float(mm.params[0]) == pytest.approx(0.6, abs=0.1)
    season = trend[:144] + seas[:144] + rn(144, 0.1)
    sm = E.SARIMA((0, 1, 1), (0, 1, 1, 12)).fit(season)
    f12 = sm.forecast(12)
    truth = 0.05 * torch.arange(144, 156, dtype=torch.float64) + 3 + 2 * torch.sin(2 * math.pi * torch.arange(144, 156, dtype=torch.float64) / 12)
    assert float((f12 - truth).abs().mean()) < 0.4
    best = E.auto_arima(walk[:200] * 0.5 + ar[:200], max_p=2, max_q=1)
    assert best.order[1] == 1 and math.isfinite(best.aic)
    assert E.auto_arima(ar[:300], max_p=2, max_q=1).order[1] == 0
    # nonlinear filters on a pendulum-like model observed through a sine
    dt = 0.05
    f = lambda s: torch.stack([s[0] + dt * s[1], s[1] - dt * 9.81 * torch.sin(s[0])])
    h = lambda s: torch.sin(s[0])[None]
    state, truth_s, obs = torch.tensor([1.0, 0.0], dtype=torch.float64), [], []
    for _ in range(150):
        state = f(state)
        truth_s.append(state); obs.append(h(state) + rn(1, 0.1))
    truth_s = torch.stack(truth_s)
    Q, R = torch.eye(2, dtype=torch.float64) * 1e-4, torch.eye(1, dtype=torch.float64) * 0.01
    for Filt in (E.ExtendedKalmanFilter, E.UnscentedKalmanFilter):
        est = Filt(f, h, Q, R, torch.tensor([0.5, 0.0]), torch.eye(2) * 0.5).filter(obs)
        assert float((est[50:, 0] - truth_s[50:, 0]).abs().mean()) < 0.08, Filt.__name__
    pf = E.ParticleFilter(lambda p, gen: torch.stack([f(s) for s in p]) + torch.randn(p.shape, generator=gen, dtype=torch.float64) * 0.02,
                          lambda z, p: torch.exp(-0.5 * (z[0] - torch.sin(p[:, 0])) ** 2 / 0.01), torch.tensor([0.5, 0.0]) + 0.5 * torch.randn(300, 2, generator=g, dtype=torch.float64), seed=1)
    pe = pf.filter(obs[:80])
    assert float((pe[40:, 0] - truth_s[40:80, 0]).abs().mean()) < 0.15 and pf.resamples > 0
    # change points
    seg = torch.cat([rn(80) + 0, rn(60) + 4, rn(100) - 2])
    cps = E.pelt(seg)
    assert len(cps) == 2 and abs(cps[0] - 80) <= 3 and abs(cps[1] - 140) <= 3 and E.pelt(rn(200)) == []
    vs = torch.cat([rn(100, 0.3), rn(100, 3.0)])
    vc = E.pelt(vs, cost="normal", min_size=10)
    assert len(vc) >= 1 and min(abs(c - 100) for c in vc) <= 8
    # mode decompositions separate two tones
    t2 = torch.arange(1024, dtype=torch.float64)
    fast, slow = torch.sin(2 * math.pi * t2 / 16), 2 * torch.sin(2 * math.pi * t2 / 200)
    imfs = E.emd(fast + slow)
    assert len(imfs) >= 3 and torch.allclose(sum(imfs), fast + slow, atol=1e-9)
    corr = lambda a, b: float(torch.corrcoef(torch.stack([a, b]))[0, 1])
    assert corr(imfs[0][100:-100], fast[100:-100]) > 0.95 and max(corr(i[100:-100], slow[100:-100]) for i in imfs[1:]) > 0.9
    modes, om = E.vmd(fast + slow + rn(1024, 0.05), k=2)
    assert om[0] == pytest.approx(1 / 200, abs=2e-3) and om[1] == pytest.approx(1 / 16, abs=2e-3) and corr(modes[1][50:-50], fast[50:-50]) > 0.97 and corr(modes[0][50:-50], slow[50:-50]) > 0.97
    # imputation and outliers
    base = torch.sin(2 * math.pi * torch.arange(120, dtype=torch.float64) / 12) + 0.01 * torch.arange(120, dtype=torch.float64)
    holes = base.clone(); holes[[0, 5, 6, 7, 50, 119]] = float("nan")
    for method, tol in (("linear", 0.6), ("spline", 0.8), ("seasonal", 0.7), ("mean", 2.0), ("ffill", 1.5), ("bfill", 1.5)):
        filled = E.impute(holes, method, 12)
        assert not torch.isnan(filled).any() and float((filled - base).abs().max()) < tol, method
    assert float((E.impute(holes, "spline")[5:8] - base[5:8]).abs().max()) < float((E.impute(holes, "mean")[5:8] - base[5:8]).abs().max())
    with pytest.raises(ValueError):
        E.impute(holes, "magic")
    dirty = base + rn(120, 0.05); dirty[[30, 77]] += torch.tensor([6.0, -5.0], dtype=torch.float64)
    for method in ("hampel", "zscore", "iqr", "isolation_forest"):
        mk = E.detect_outliers(dirty, method)
        assert mk[30] and mk[77] and int(mk.sum()) <= 6, method
    fixed = E.treat_outliers(dirty, E.detect_outliers(dirty, "hampel"))
    assert float((fixed - base).abs().max()) < 0.6 and float(E.treat_outliers(dirty, E.detect_outliers(dirty), "clip").max()) < 3
    cloud = torch.cat([rn(300).reshape(150, 2), torch.tensor([[8.0, 8.0], [-9.0, 7.0]], dtype=torch.float64)])
    sc = E.IsolationForest(seed=0).fit(cloud).score(cloud)
    assert set(sc.topk(2).indices.tolist()) == {150, 151} and float(sc[:150].median()) < 0.5 < float(sc[150])
    # rolling, features, CV, metrics
    r = E.rolling(torch.arange(10.0), 3)
    assert torch.isnan(r[:2]).all() and r[2:].tolist() == [1, 2, 3, 4, 5, 6, 7, 8] and E.rolling(torch.arange(10.0), 3, "max")[-1] == 9 and float(E.ewm(torch.ones(5), 0.3)[-1]) == 1.0
    ft = E.extract_features(y, 12)
    assert ft["seasonal_strength"] > 0.9 and ft["trend_strength"] > 0.9 and ft["linear_slope"] == pytest.approx(0.05, abs=0.01) and E.extract_features(white)["acf1"] < 0.2
    assert E.extract_features(rn(240), 12)["seasonal_strength"] < 0.5
    splits = list(E.TimeSeriesCV(3, test_size=10, gap=2).split(100))
    assert [te[0] for _, te in splits] == [70, 80, 90] and all(max(tr) == te[0] - 3 for tr, te in splits) and [len(tr) for tr, _ in splits] == [68, 78, 88]
    sl = list(E.TimeSeriesCV(3, test_size=10, mode="sliding", train_size=30).split(100))
    assert all(len(tr) == 30 and tr[-1] == te[0] - 1 for tr, te in sl)
    bl = list(E.TimeSeriesCV(4, mode="blocked").split(100))
    assert [(tr[0], te[-1]) for tr, te in bl] == [(0, 24), (25, 49), (50, 74), (75, 99)]
    em = list(E.TimeSeriesCV(3, test_size=10, embargo=5).split(100))
    assert not set(range(80, 85)) & set(em[2][0]) and set(range(85, 90)) <= set(em[2][0]) and set(range(70, 80)) <= set(em[2][0]) and len(em[2][0]) == 85
    naive = lambda tr, h: tr[-12:].repeat(h // 12 + 1)[:h]
    mean_f = lambda tr, h: tr.mean().expand(h)
    cv = E.TimeSeriesCV(4, test_size=12)
    assert sum(cv.score(y, naive)) < sum(cv.score(y, mean_f))
    fm = E.forecast_metrics(torch.tensor([10.0, 20.0]), torch.tensor([12.0, 18.0]), train=torch.tensor([1.0, 3.0, 2.0, 5.0]))
    assert fm["mae"] == 2 and fm["rmse"] == 2 and fm["mape"] == pytest.approx(15.0) and fm["bias"] == 0 and fm["mase"] == pytest.approx(1.0) and fm["smape"] == pytest.approx((4 / 22 + 4 / 38) / 2 * 100)
    # neural forecasters learn a seasonal pattern better than the mean
    wave = (torch.sin(2 * math.pi * torch.arange(200.0) / 12) + 0.05 * torch.randn(200, generator=torch.Generator().manual_seed(1)))
    for Model, kw in ((E.LSTMForecaster, {}), (E.GRUForecaster, {}), (E.CNNForecaster, {}), (E.TransformerForecaster, {"dim": 16, "heads": 2, "layers": 1})):
        fcst = Model(window=24, horizon=1, **kw).fit(wave[:176], epochs=120).forecast(24)
        assert fcst.shape == (24,) and float((fcst - wave[176:]).abs().mean()) < 0.35 < float((wave[:176].mean() - wave[176:]).abs().mean()), Model.__name__


def test_signal_ext_windows_iir_design_filtering_adaptive_audio_resampling_streaming_and_packets():
    import math
    import numpy as np
    from scipy import signal as ss
    from torsh_b200 import signal_ext as G
    torch.manual_seed(0)
    dd = torch.float64
    # windows against scipy
    for name, sci in (("hann", "hann"), ("hamming", "hamming"), ("blackman", "blackman"), ("blackman_harris", "blackmanharris"), ("nuttall", "nuttall"), ("flat_top", "flattop"),
                      ("bartlett", "bartlett"), ("bohman", "bohman"), ("cosine", "cosine"), ("rectangular", "boxcar")):
        for n in (16, 33):
            assert np.allclose(G.get_window(name, n).numpy(), ss.get_window(sci, n, fftbins=False), atol=1e-7), (name, n)
    assert np.allclose(G.get_window("hann", 16, periodic=True).numpy(), ss.get_window("hann", 16, fftbins=True))
    assert np.allclose(G.get_window("tukey", 32, alpha=0.4).numpy(), ss.windows.tukey(32, 0.4), atol=1e-12) and np.allclose(G.get_window("gaussian", 21, std=3.0).numpy(), ss.windows.gaussian(21, 3.0))
    assert np.allclose(G.get_window("kaiser", 25, beta=8.0).numpy(), ss.windows.kaiser(25, 8.0), atol=1e-6) and np.allclose(G.get_window("exponential", 21, tau=4.0).numpy(), ss.windows.exponential(21, tau=4.0))
    assert float(G.normalize_window(G.get_window("hann", 32)).sum()) == pytest.approx(1.0)
    nt, beta = G.kaiser_parameters(60.0, 0.1)
    ref_n, ref_b = ss.kaiserord(60.0, 0.1)
    assert abs(nt - ref_n) <= 1 and beta == pytest.approx(ref_b, rel=1e-3)
    # IIR designs against scipy (coefficients and magnitude response)
    cases = [("butter", dict(N=4, Wn=0.3, btype="lowpass"), lambda: G.butterworth(4, 0.3)), ("butter", dict(N=3, Wn=0.4, btype="highpass"), lambda: G.butterworth(3, 0.4, "highpass")),
             ("butter", dict(N=2, Wn=[0.2, 0.5], btype="bandpass"), lambda: G.butterworth(2, [0.2, 0.5], "bandpass")), ("butter", dict(N=2, Wn=[0.2, 0.5], btype="bandstop"), lambda: G.butterworth(2, [0.2, 0.5], "bandstop")),
             ("cheby1", dict(N=4, rp=1.0, Wn=0.3), lambda: G.chebyshev1(4, 1.0, 0.3)), ("cheby1", dict(N=5, rp=0.5, Wn=0.4, btype="highpass"), lambda: G.chebyshev1(5, 0.5, 0.4, "highpass")),
             ("cheby2", dict(N=4, rs=40.0, Wn=0.3), lambda: G.chebyshev2(4, 40.0, 0.3)), ("cheby2", dict(N=5, rs=30.0, Wn=0.5), lambda: G.chebyshev2(5, 30.0, 0.5)),
             ("ellip", dict(N=4, rp=1.0, rs=40.0, Wn=0.3), lambda: G.elliptic(4, 1.0, 40.0, 0.3))]
    for fam, kw, ours in cases:
        b_ref, a_ref = getattr(ss, fam)(**kw)
        b, a = ours()
        assert np.allclose(b.numpy(), b_ref, atol=1e-8) and np.allclose(a.numpy(), a_ref, atol=1e-8), (fam, kw)
    bb, ab = G.bessel(4, 0.3)
    w, h = G.freqz(bb, ab, 512)
    assert abs(float(h.abs()[int(0.3 * 512)]) - 1 / math.sqrt(2)) < 0.03 and float(h.abs()[0]) == pytest.approx(1.0, abs=1e-6) and G.is_stable(ab)
    gd = G.group_delay(bb, ab)[1]
    assert float(gd[:100].std()) < 0.05 * float(gd[:100].mean())                                    # maximally flat delay in the pass band
    b, a = G.butterworth(4, 0.3)
    w, h = G.freqz(b, a, 256)
    wr, hr = ss.freqz(b.numpy(), a.numpy(), 256)
    assert np.allclose(h.numpy(), hr, atol=1e-10) and np.allclose(w.numpy(), wr)
    sos = G.iir_design(6, 0.25, output="sos")
    x = torch.randn(300, dtype=dd)
    b6, a6 = G.butterworth(6, 0.25)
    assert sos.shape == (3, 6) and torch.allclose(G.sosfilt(sos, x), G.lfilter(b6, a6, x), atol=1e-9)
    assert np.allclose(G.lfilter(b, a, x).numpy(), ss.lfilter(b.numpy(), a.numpy(), x.numpy()), atol=1e-10)
    assert np.allclose(G.filtfilt(b, a, x).numpy(), ss.filtfilt(b.numpy(), a.numpy(), x.numpy(), padlen=15), atol=1e-8)
    assert np.allclose(G.impulse_response(b, a, 32).numpy(), ss.lfilter(b.numpy(), a.numpy(), np.eye(1, 32)[0]), atol=1e-12)
    st = G.stability_analysis(b, a)
    assert st["stable"] and st["max_pole_radius"] < 1 and not G.is_stable([1.0, -2.5, 1.0]) and G.is_stable([1.0])
    # FIR designs
    h2 = G.firwin2(65, [0, 0.3, 0.4, 1.0], [1, 1, 0, 0])
    assert np.allclose(h2.numpy(), ss.firwin2(65, [0, 0.3, 0.4, 1.0], [1, 1, 0, 0]), atol=1e-6)
    hr = G.remez(41, [0, 0.25, 0.35, 1.0], [1, 0], weights=[1, 10])
    mag = G.freqz(hr, 1.0, 512)[1].abs()
    assert float((mag[:int(0.25 * 512)] - 1).abs().max()) < 0.05 and float(mag[int(0.36 * 512):].max()) < 0.01 and torch.allclose(hr, hr.flip(0))
    assert np.allclose(G.savgol_coeffs(7, 2).flip(0).numpy(), ss.savgol_coeffs(7, 2)) and np.allclose(G.savgol_coeffs(7, 3, 1).flip(0).numpy(), ss.savgol_coeffs(7, 3, deriv=1), atol=1e-12)
    noisy = torch.sin(torch.linspace(0, 6, 120, dtype=dd)) + 0.1 * torch.randn(120, dtype=dd)
    assert np.allclose(G.savgol_filter(noisy, 11, 3).numpy(), ss.savgol_filter(noisy.numpy(), 11, 3), atol=1e-9)
    assert np.allclose(G.median_filter1d(noisy, 5)[2:-2].numpy(), ss.medfilt(noisy.numpy(), 5)[2:-2]) and np.allclose(G.convolve1d([1, 2, 3], [0, 1]).numpy(), [0, 1, 2, 3])
    mp = G.minimum_phase(h2)
    assert torch.allclose(G.freqz(mp, 1.0, 128)[1].abs()[:30], G.freqz(h2, 1.0, 128)[1].abs()[:30], atol=0.02) and float(mp[:10].abs().sum()) > float(h2[:10].abs().sum())
    # adaptive filters identify an unknown FIR system
    unknown = torch.tensor([0.5, -0.3, 0.2, 0.1], dtype=dd)
    src = torch.randn(3000, dtype=dd)
    des = torch.from_numpy(np.convolve(src.numpy(), unknown.numpy())[:3000]) + 0.01 * torch.randn(3000, dtype=dd)
    for fn, kw in ((G.lms_filter, dict(mu=0.01)), (G.nlms_filter, dict(mu=0.5)), (G.rls_filter, dict())):
        y, e, wts = fn(src, des, taps=4, **kw)
        assert torch.allclose(wts, unknown, atol=0.03) and float(e[-500:].pow(2).mean()) < 1e-3, fn.__name__
    assert float(G.rls_filter(src[:200], des[:200], 4)[1][100:].pow(2).mean()) < float(G.lms_filter(src[:200], des[:200], 4, 0.01)[1][100:].pow(2).mean())
    # scales, cepstra, MFCC, chroma, pitch
    for fwd, inv in ((G.hz_to_bark, G.bark_to_hz), (G.hz_to_erb, G.erb_to_hz)):
        assert torch.allclose(inv(fwd(torch.tensor([100.0, 1000.0, 8000.0]))), torch.tensor([100.0, 1000.0, 8000.0], dtype=dd))
    sr = 16000
    tt = torch.arange(4096, dtype=dd) / sr
    tone = torch.sin(2 * math.pi * 220 * tt) + 0.5 * torch.sin(2 * math.pi * 440 * tt) + 0.3 * torch.sin(2 * math.pi * 660 * tt)
    assert G.autocorr_pitch(tone, sr) == pytest.approx(220, rel=0.01)
    f0, ap = G.yin_pitch(tone, sr)
    assert f0 == pytest.approx(220, rel=0.005) and ap < 0.05 and G.yin_pitch(torch.randn(4096, dtype=dd), sr)[0] == 0.0
    assert float(G.zero_crossing_rate(torch.sin(2 * math.pi * 1000 * tt))) == pytest.approx(2 * 1000 / sr, rel=0.02)
    echo = torch.randn(1024, dtype=dd); echo[100:] += 0.6 * echo[:-100].clone()
    cep = G.real_cepstrum(echo)
    assert int(cep[20:512].argmax()) + 20 == 100 and G.power_cepstrum(echo).shape == (1024,)
    cc, nd = G.complex_cepstrum(unknown)
    ccr, ndr = ss.cceps(unknown.numpy()) if hasattr(ss, "cceps") else (cc.numpy(), nd)
    assert np.allclose(cc.numpy(), ccr, atol=1e-8) and nd == ndr
    from scipy.fft import dct
    v = torch.randn(3, 20, dtype=dd)
    assert np.allclose(G.dct2(v).numpy(), dct(v.numpy(), type=2, norm="ortho"), atol=1e-10)
    mf = G.compute_mfcc(tone.float(), sr, n_mfcc=13, n_mels=26)
    assert mf.shape[1] == 13 and torch.isfinite(mf).all() and not torch.allclose(mf[5], G.compute_mfcc(torch.randn(4096), sr, 13, 26)[5], atol=1.0)
    a440 = torch.sin(2 * math.pi * 440 * torch.arange(8192, dtype=dd) / sr)
    ch = G.chroma_features(a440.float(), sr)
    assert int(ch.mean(1).argmax()) == 9                                                             # A
    # resampling
    sig = torch.sin(2 * math.pi * 5 * torch.arange(400, dtype=dd) / 400)
    up = G.polyphase_resample(sig, 3, 2)
    ref = torch.sin(2 * math.pi * 5 * torch.arange(600, dtype=dd) / 600)
    assert up.shape == (600,) and float((up - ref)[40:-40].abs().max()) < 5e-3
    assert np.allclose(up[40:-40].numpy(), ss.resample_poly(sig.numpy(), 3, 2)[40:-40], atol=5e-3)
    assert float((G.sinc_resample(sig, 1.5) - ref)[40:-40].abs().max()) < 5e-3 and float((G.linear_resample(sig, 1.5) - torch.sin(2 * math.pi * 5 * torch.linspace(0, 399, 600, dtype=dd) / 400)).abs().max()) < 2e-3
    two = torch.sin(2 * math.pi * 10 * torch.arange(2000, dtype=dd) / 2000) + torch.sin(2 * math.pi * 400 * torch.arange(2000, dtype=dd) / 2000)
    dec = G.decimate(two, 4)
    assert dec.shape == (500,) and float((dec - torch.sin(2 * math.pi * 10 * torch.arange(500, dtype=dd) / 500))[30:-30].abs().max()) < 0.02
    # streaming equals batch
    rb = G.RingBuffer(5)
    rb.push(torch.arange(7.0))
    assert rb.is_full() and rb.peek().tolist() == [2, 3, 4, 5, 6] and rb.pop(2).tolist() == [2, 3] and len(rb) == 3
    sf = G.StreamingFilter(b, a)
    chunks = torch.cat([sf.process(c) for c in x.split(37)])
    assert torch.allclose(chunks, G.lfilter(b, a, x), atol=1e-12)
    fir = G.firwin2(33, [0, 0.2, 0.3, 1], [1, 1, 0, 0])
    oa = G.OverlapAddProcessor(fir, block=64)
    got = torch.cat([oa.process(c) for c in x.split(50)] + [oa.flush()])
    assert np.allclose(got.numpy(), np.convolve(x.numpy(), fir.numpy()), atol=1e-10)
    sst = G.StreamingSTFT(64, 16)
    frames = torch.cat([sst.push(c) for c in x.split(23)], 1)
    full = torch.stft(x, 64, 16, window=torch.hann_window(64, dtype=dd), center=False, return_complex=True)
    assert torch.allclose(frames, full, atol=1e-10)
    smooth = lambda v: G.savgol_filter(v, 11, 2)
    assert torch.allclose(G.process_chunked(smooth, noisy, 32, overlap=8), smooth(noisy), atol=1e-9)
    # lifting and packets
    for wv in ("haar", "cdf53"):
        for n in (64, 63):
            s_ = torch.randn(2, n, dtype=dd)
            a_, d_ = G.lifting_dwt(s_, wv)
            assert torch.allclose(G.lifting_idwt(a_, d_, wv), s_, atol=1e-12), (wv, n)
    ramp = torch.arange(64, dtype=dd)
    assert G.lifting_dwt(ramp, "cdf53")[1][:-1].abs().max() < 1e-12 and G.lifting_dwt(ramp, "haar")[1].abs().min() > 0.5
    s_ = torch.randn(128, dtype=dd)
    tree = G.wavelet_packet(s_, "db2", 3)
    assert len(tree) == 15 and tree["ada"].shape == (16,) and torch.allclose(G.wavelet_packet_reconstruct(tree, "db2"), s_, atol=1e-10)
    assert sum(float(tree[p].pow(2).sum()) for p in tree if len(p) == 3) == pytest.approx(float(s_.pow(2).sum()))
    hf = torch.sin(2 * math.pi * 0.45 * torch.arange(256, dtype=dd))
    basis = G.best_basis(G.wavelet_packet(hf, "db4", 3))
    leaves_energy = sum(float(G.wavelet_packet(hf, "db4", 3)[p].pow(2).sum()) for p in basis)
    assert leaves_energy == pytest.approx(float(hf.pow(2).sum()), rel=1e-9) and any(p.startswith("d") for p in basis) and basis != [""]
    assert G.scale_to_frequency(G.frequency_to_scale(0.1)) == pytest.approx(0.1) and G.cone_of_influence(100, 8.0) == (12, 88) and G.scalogram(hf, [2.0, 4.0]).shape == (2, 256)


def test_sparse_ext_arithmetic_factorisations_solvers_exchange_analysis_layers_and_optimizers(tmp_path):
    import numpy as np
    import scipy.sparse as sps
    import scipy.sparse.linalg as spla
    from torsh_b200 import sparse_ext as Z
    from torsh_b200.sparse import CooTensor
    torch.manual_seed(0)
    dd = torch.float64
    def rand_sparse(m, n, density, seed):
        g = torch.Generator().manual_seed(seed)
        d = torch.randn(m, n, generator=g, dtype=dd) * (torch.rand(m, n, generator=g) < density)
        return CooTensor.from_dense(d), d
    a, da = rand_sparse(12, 9, 0.3, 1)
    b, db = rand_sparse(12, 9, 0.3, 2)
    c, dc = rand_sparse(9, 7, 0.3, 3)
    assert torch.allclose(Z.sparse_add(a, b, -2.0).to_dense(), da - 2 * db) and torch.allclose(Z.sparse_mul(a, b).to_dense(), da * db)
    assert torch.allclose(Z.spgemm(a, c).to_dense(), da @ dc) and Z.spgemm(a, c).nnz == int((da @ dc != 0).sum())
    assert torch.allclose(Z.sparse_sum(a, 0), da.sum(0)) and torch.allclose(Z.sparse_sum(a, 1), da.sum(1)) and float(Z.sparse_sum(a)) == pytest.approx(float(da.sum()))
    for k in ("fro", "1", "inf"):
        assert Z.sparse_norm(a, k) == pytest.approx(float(torch.linalg.matrix_norm(da, {"fro": "fro", "1": 1, "inf": float("inf")}[k])))
    assert torch.allclose(Z.triu(a, 1).to_dense(), da.triu(1)) and torch.allclose(Z.tril(a, -1).to_dense(), da.tril(-1)) and torch.allclose(Z.diagonal(a), da.diagonal())
    assert torch.allclose(Z.kron(a, c).to_dense(), torch.kron(da, dc)) and torch.equal(Z.identity(3).to_dense(), torch.eye(3, dtype=dd))
    # SPD system: 2-D Laplacian
    n = 8
    lap = sps.kron(sps.eye(n), sps.diags([-1, 2, -1], [-1, 0, 1], shape=(n, n))) + sps.kron(sps.diags([-1, 2, -1], [-1, 0, 1], shape=(n, n)), sps.eye(n))
    A = Z.from_scipy(lap.tocoo())
    rhs = torch.randn(n * n, dtype=dd)
    exact = torch.from_numpy(spla.spsolve(lap.tocsc(), rhs.numpy()))
    x, info = Z.conjugate_gradient(A, rhs)
    assert info["converged"] and torch.allclose(x, exact, atol=1e-8)
    chol = Z.SparseCholesky(A)
    Lf = chol.factor().to_dense()
    assert torch.allclose(Lf @ Lf.t(), A.to_dense(), atol=1e-10) and torch.allclose(chol.solve(rhs), exact, atol=1e-9)
    ic = Z.SparseCholesky(A, incomplete=True)
    assert ic.factor().nnz == Z.tril(A).nnz < chol.factor().nnz
    xp, ip = Z.conjugate_gradient(A, rhs, precond=ic.solve)
    xj, ij = Z.conjugate_gradient(A, rhs, precond=Z.jacobi_preconditioner(A))
    assert ip["converged"] and ip["iterations"] < 0.7 * info["iterations"] and torch.allclose(xp, exact, atol=1e-8) and ij["converged"]
    with pytest.raises(ValueError):
        Z.SparseCholesky(Z.sparse_add(A, Z.identity(n * n), -10.0))
    # non-symmetric system: convection-diffusion
    conv = lap + 0.8 * sps.kron(sps.eye(n), sps.diags([-1, 1], [-1, 1], shape=(n, n)))
    B = Z.from_scipy(conv.tocoo())
    exact_b = torch.from_numpy(spla.spsolve(conv.tocsc(), rhs.numpy()))
    ilu = Z.IncompleteLU(B)
    L, U = ilu.factors()
    pat = B.to_dense() != 0
    assert torch.allclose((L.to_dense() @ U.to_dense())[pat], B.to_dense()[pat], atol=1e-10) and L.nnz + U.nnz == B.nnz + n * n
    for solver in (Z.bicgstab, Z.gmres):
        x0, i0 = solver(B, rhs)
        x1, i1 = solver(B, rhs, precond=ilu.solve)
        assert i0["converged"] and i1["converged"] and i1["iterations"] < i0["iterations"] and torch.allclose(x1, exact_b, atol=1e-7), solver.__name__
    tri = Z.tril(B)
    assert torch.allclose(Z.solve_triangular(tri, rhs), torch.linalg.solve_triangular(tri.to_dense(), rhs[:, None], upper=False)[:, 0], atol=1e-10)
    assert torch.allclose(Z.solve_triangular(Z.triu(B), rhs, lower=False), torch.linalg.solve_triangular(Z.triu(B).to_dense(), rhs[:, None], upper=True)[:, 0], atol=1e-10)
    # reordering
    perm0 = torch.randperm(n * n, generator=torch.Generator().manual_seed(5))
    shuffled = Z.permute(A, perm0)
    rcm = Z.reverse_cuthill_mckee(shuffled)
    again = Z.permute(shuffled, rcm)
    assert sorted(rcm.tolist()) == list(range(n * n)) and Z.bandwidth(again) < 0.4 * Z.bandwidth(shuffled) and Z.bandwidth(again) <= 2 * n
    assert torch.allclose(torch.linalg.eigvalsh(again.to_dense()), torch.linalg.eigvalsh(A.to_dense()), atol=1e-9)
    # exchange formats
    Z.write_matrix_market(a, tmp_path / "a.mtx", comment="test matrix")
    back = Z.read_matrix_market(tmp_path / "a.mtx")
    assert torch.allclose(back.to_dense(), da) and "%test matrix" in (tmp_path / "a.mtx").read_text()
    from scipy.io import mmread
    assert np.allclose(mmread(str(tmp_path / "a.mtx")).toarray(), da.numpy())
    Z.write_matrix_market(A, tmp_path / "s.mtx", symmetric=True)
    assert "symmetric" in (tmp_path / "s.mtx").read_text().splitlines()[0] and torch.allclose(Z.read_matrix_market(tmp_path / "s.mtx").to_dense(), A.to_dense())
    (tmp_path / "p.mtx").write_text("%%MatrixMarket matrix coordinate pattern skew-symmetric\n3 3 1\n2 1\n")
    assert Z.read_matrix_market(tmp_path / "p.mtx").to_dense().tolist() == [[0, -1, 0], [1, 0, 0], [0, 0, 0]]
    assert np.allclose(Z.to_scipy(a).toarray(), da.numpy()) and torch.allclose(Z.from_scipy(Z.to_scipy(a, "csc")).to_dense(), da)
    Z.save_matlab(a, tmp_path / "a.mat")
    assert torch.allclose(Z.load_matlab(tmp_path / "a.mat").to_dense(), da)
    # analysis
    rep = Z.analyze_pattern(A)
    assert rep["symmetric"] and rep["diagonals"] == 5 and rep["bandwidth"] == n and rep["diagonal_dominant"] and rep["recommended_format"] == "dia" and rep["row_nnz_max"] == 5
    blocks = CooTensor.from_dense(torch.kron((torch.rand(6, 6) < 0.3).double(), torch.ones(4, 4, dtype=dd)) + 0)
    assert Z.analyze_pattern(blocks)["block_size"] == 4 and Z.analyze_pattern(blocks)["recommended_format"] == "bsr"
    reg, _ = rand_sparse(200, 200, 0.02, 7)
    assert Z.analyze_pattern(reg)["recommended_format"] in ("csr", "ell") and not Z.analyze_pattern(reg)["symmetric"]
    mem = Z.memory_report(reg)
    assert mem["csr"] < mem["coo"] < mem["dense"] and mem["best"] == "csr"
    skew = torch.zeros(50, 50, dtype=dd); skew[torch.arange(50), torch.arange(50)] = 1.0; skew[0] = 1.0
    hy = Z.HybridTensor(CooTensor.from_dense(skew))
    v = torch.randn(50, 3, dtype=dd)
    assert hy.k == 1 and hy.coo.nnz == 49 and torch.allclose(hy.matmul(v), skew @ v) and torch.allclose(hy.to_dense(), skew) and torch.allclose(hy.matmul(v[:, 0]), skew @ v[:, 0])
    sy = Z.SymmetricTensor(A)
    assert sy.nnz_stored == (A.nnz + n * n) // 2 and torch.allclose(sy.matmul(rhs), A.matmul(rhs)) and torch.allclose(sy.to_coo().to_dense(), A.to_dense())
    with pytest.raises(ValueError):
        Z.SymmetricTensor(a if a.shape[0] == a.shape[1] else B)
    # layers
    act = Z.SparseActivation("relu")(a)
    assert torch.allclose(act.to_dense(), da.relu()) and act.nnz == int((da > 0).sum()) and torch.allclose(Z.SparseActivation("tanh")(a).to_dense(), da.tanh())
    ln = Z.SparseLayerNorm()(a)
    row = ln.values[ln.rows == 3]
    assert abs(float(row.mean())) < 1e-9 and float(row.var(unbiased=False)) == pytest.approx(1.0, abs=1e-3)
    sm = Z.sparse_softmax(a)
    masked = da.masked_fill(da == 0, float("-inf")).softmax(1).nan_to_num(0.0)
    assert torch.allclose(sm.to_dense(), masked, atol=1e-12)
    att = Z.SparseAttention(16, heads=2)
    xs = torch.randn(10, 16)
    r_full, c_full = torch.arange(10).repeat_interleave(10), torch.arange(10).repeat(10)
    q, k, vv = (f(xs).reshape(10, 2, 8).transpose(0, 1) for f in (att.q, att.k, att.v))
    dense = att.o(torch.nn.functional.scaled_dot_product_attention(q, k, vv).transpose(0, 1).reshape(10, 16))
    assert torch.allclose(att(xs, r_full, c_full), dense, atol=1e-5)
    r_loc, c_loc = Z.SparseAttention.local_pattern(10, 1, global_tokens=1)
    assert len(r_loc) == 28 + 16 and att(xs, r_loc, c_loc).shape == (10, 16)
    mask = torch.full((10, 10), float("-inf")); mask[r_loc, c_loc] = 0
    dense_l = att.o(torch.nn.functional.scaled_dot_product_attention(q, k, vv, attn_mask=mask).transpose(0, 1).reshape(10, 16))
    assert torch.allclose(att(xs, r_loc, c_loc), dense_l, atol=1e-5)
    sp = torch.sparse_coo_tensor(torch.tensor([[0, 1, 5, 7], [0, 1, 2, 7]]), torch.tensor([1.0, 3.0, 2.0, -1.0]), (8, 8))
    mp = Z.sparse_max_pool2d(sp, 2).coalesce()
    assert mp.shape == (4, 4) and mp.indices().t().tolist() == [[0, 0], [2, 1], [3, 3]] and mp.values().tolist() == [3.0, 2.0, -1.0]
    sc = Z.SparseConv1d(4, 6, 3)
    pos, feats = torch.tensor([2, 3, 10]), torch.randn(3, 4)
    op, of = sc(pos, feats)
    dense_in = torch.zeros(1, 4, 12); dense_in[0, :, pos] = feats.t()
    ref = torch.nn.functional.conv1d(dense_in, sc.weight.permute(2, 1, 0), sc.bias, padding=1)[0].t()
    assert op.tolist() == [2, 3, 10] and torch.allclose(of, ref[pos], atol=1e-6)
    # row-wise optimizers
    emb = Z.SparseEmbedding(100, 8)
    before = emb.inner.weight.detach().clone()
    opt = Z.SparseSGD(emb.parameters(), lr=0.5, momentum=0.9)
    emb(torch.tensor([3, 7, 3])).sum().backward()
    assert emb.inner.weight.grad.is_sparse
    opt.step()
    changed = (emb.inner.weight.detach() != before).any(1).nonzero().flatten().tolist()
    assert changed == [3, 7] and opt.rows_touched == 2 and torch.allclose(emb.inner.weight.detach()[3], before[3] - 0.5 * 2)
    e2 = Z.SparseEmbedding(50, 4); e3 = torch.nn.Embedding(50, 4); e3.weight.data.copy_(e2.inner.weight.data)
    oa, ob = Z.SparseAdamW(e2.parameters(), lr=0.01), torch.optim.Adam(e3.parameters(), lr=0.01)
    for _ in range(3):                                                       # rows hit every step follow dense Adam exactly
        for e, o in ((e2, oa), (e3, ob)):
            o.zero_grad(); (e(torch.tensor([1, 2])) ** 2).sum().backward(); o.step()
    assert torch.allclose(e2.inner.weight.detach()[[1, 2]], e3.weight.detach()[[1, 2]], atol=1e-6) and torch.equal(e2.inner.weight.detach()[5], e3.weight.detach()[5])
    acc = Z.SparseGradientAccumulator((100, 8))
    for ids in ([1, 2], [2, 9]):
        emb.inner.weight.grad = None
        emb(torch.tensor(ids)).sum().backward()
        acc.add(emb.inner.weight.grad)
    tot = acc.result()
    assert tot.indices()[0].tolist() == [1, 2, 9] and tot.values()[1].tolist() == [2.0] * 8


def test_graph_ext_pooling_geometric_hetero_kg_explain_kernels_transport_analysis_and_loaders(tmp_path):
    import json
    import math
    import numpy as np
    nx = pytest.importorskip("scipy")
    from torsh_b200 import graph as G, graph_ext as X
    torch.manual_seed(0)
    # two cliques joined by one edge
    k = 6
    a = torch.combinations(torch.arange(k)).t()
    ei = torch.cat([a, a + k, torch.tensor([[0], [k]])], 1)
    ei = torch.cat([ei, ei.flip(0)], 1)
    n = 2 * k
    truth = torch.arange(n) // k
    x = torch.randn(n, 8)
    dp = X.DiffPool(8, 16, 2)
    xp, ap = dp(x, ei)
    assert xp.shape == (2, 16) and ap.shape == (2, 2) and torch.allclose(dp.assignment.sum(1), torch.ones(n), atol=1e-6) and dp.link_loss > 0 and dp.entropy_loss > 0
    mc = X.MinCutPool(8, 2)
    feats = torch.nn.functional.one_hot(truth, 2).float() @ torch.randn(2, 8) + 0.1 * torch.randn(n, 8)
    opt = torch.optim.Adam(mc.parameters(), 0.05)
    for _ in range(150):
        mc(feats, ei)
        loss = mc.cut_loss + mc.ortho_loss
        opt.zero_grad(); loss.backward(); opt.step()
    assign = mc.assignment.argmax(1)
    assert (assign[:k] == assign[0]).all() and (assign[k:] == assign[k]).all() and assign[0] != assign[k] and float(mc.cut_loss) < -0.9
    tk = X.TopKPool(8, 0.5)
    xs, es, keep = tk(x, ei)
    assert xs.shape == (6, 8) and es.max() < 6 and len(keep) == 6 and es.shape[1] == int(((torch.isin(ei[0], keep)) & (torch.isin(ei[1], keep))).sum())
    batch = truth.clone()
    gap = X.GlobalAttentionPool(8)
    assert gap(x, batch).shape == (2, 8)
    perm = torch.randperm(k)
    s2s = X.Set2Set(8, 3)
    assert s2s(x, batch).shape == (2, 16) and torch.allclose(s2s(x[:k]), s2s(x[:k][perm]), atol=1e-5)
    # geometric layers: EGNN is rotation / translation equivariant, SchNet invariant
    pos = torch.randn(10, 3)
    h = torch.randn(10, 8)
    rg = X.radius_graph(pos, 2.5)
    kg = X.knn_graph(pos, 3)
    assert (torch.cdist(pos, pos)[rg[0], rg[1]] <= 2.5).all() and (rg[0] != rg[1]).all() and kg.shape == (2, 30) and torch.bincount(kg[1]).tolist() == [3] * 10
    q, _ = torch.linalg.qr(torch.randn(3, 3))
    shift = torch.randn(3)
    eg = X.EGNNLayer(8)
    h1, p1 = eg(h, pos, kg)
    h2, p2 = eg(h, pos @ q.t() + shift, kg)
    assert torch.allclose(h1, h2, atol=1e-4) and torch.allclose(p1 @ q.t() + shift, p2, atol=1e-4)
    sn = X.SchNetConv(8)
    assert torch.allclose(sn(h, pos, kg), sn(h, pos @ q.t() + shift, kg), atol=1e-4) and X.RBFLayer(16)(torch.tensor([0.0, 2.5])).shape == (2, 16)
    mp = X.MPNNConv(8, 4)
    assert mp(h, kg, torch.randn(30, 4)).shape == (10, 8)
    # heterogeneous, hypergraph, temporal
    hg = X.HeteroGraphData()
    hg.add_nodes("author", torch.randn(4, 5)); hg.add_nodes("paper", torch.randn(6, 7))
    hg.add_edges("author", "writes", "paper", torch.tensor([[0, 1, 1, 3], [0, 0, 2, 5]]))
    hg.add_edges("paper", "cites", "paper", torch.tensor([[0, 2], [2, 4]]))
    out = X.HeteroConv({"author": 5, "paper": 7}, 9, hg.edge_types())(hg)
    assert out["author"].shape == (4, 9) and out["paper"].shape == (6, 9) and hg.node_types() == ["author", "paper"]
    reach = hg.metapath_reachable([("author", "writes", "paper"), ("paper", "cites", "paper")])
    assert sorted(map(tuple, reach.t().tolist())) == [(0, 2), (1, 2), (1, 4)]
    inc = torch.tensor([[0, 1, 2, 2, 3, 4], [0, 0, 0, 1, 1, 1]])
    hc = X.HypergraphConv(3, 3)
    with torch.no_grad():
        hc.lin.weight.copy_(torch.eye(3)); hc.lin.bias.zero_()
    xh = torch.randn(5, 3)
    H = torch.zeros(5, 2); H[inc[0], inc[1]] = 1
    dv, de = H.sum(1).rsqrt(), H.sum(0)
    assert torch.allclose(hc(xh, inc), (dv[:, None] * H / de[None]) @ H.t() @ (dv[:, None] * xh), atol=1e-6)
    tm = X.TemporalGraphMemory(6, 8, 3)
    tm.update(torch.tensor([0, 1]), torch.tensor([2, 3]), torch.tensor([1.0, 2.0]), torch.randn(2, 3))
    assert tm.embedding(torch.tensor([0, 2])).abs().sum() > 0 and tm.embedding(torch.tensor([4])).abs().sum() == 0 and tm.last.tolist() == [1, 2, 1, 2, 0, 0]
    # knowledge graph embeddings rank true tails near the top
    ents, rels = 12, 2
    triples = torch.tensor([(i, 0, i + 1) for i in range(ents - 1)] + [(i, 1, i + 3) for i in range(ents - 3)])       # chains: translations can represent them
    for model in ("transe", "distmult", "rotate"):
        torch.manual_seed(1)
        kge = X.KnowledgeGraphEmbedding(ents, rels, 16, model)
        opt = torch.optim.Adam(kge.parameters(), 0.05)
        g = torch.Generator().manual_seed(0)
        for _ in range(300):
            opt.zero_grad(); kge.loss(triples, g).backward(); opt.step()
        ranks = [kge.rank_tail(*t) for t in triples.tolist()]
        assert np.mean(ranks) < (2.5 if model != "distmult" else 5.0), (model, np.mean(ranks))
    # explanations pick the edges that carry the signal
    class WGCN(torch.nn.Module):
        def __init__(self): super().__init__(); self.l1, self.l2 = torch.nn.Linear(2, 8), torch.nn.Linear(8, 2)
        def forward(self, x, edge_index, edge_weight=None):
            w = torch.ones(edge_index.shape[1]) if edge_weight is None else edge_weight
            agg = lambda t: t + torch.zeros_like(t).index_add_(0, edge_index[1], t[edge_index[0]] * w[:, None])
            return self.l2(torch.relu(agg(self.l1(x))))
    star = torch.tensor([[1, 2, 3, 4], [0, 0, 0, 0]])
    xs_ = torch.tensor([[0.0, 0], [5.0, 0], [0.0, 0.1], [0.0, 0.1], [0.0, 0.1]])
    wg = WGCN()
    with torch.no_grad():
        wg.l1.weight.zero_(); wg.l1.weight[0, 0] = 1; wg.l1.bias.zero_(); wg.l2.weight.zero_(); wg.l2.weight[1, 0] = 1; wg.l2.bias.zero_(); wg.l2.bias[0] = 1.0
    assert wg(xs_, star).argmax(-1)[0] == 1
    attr = X.gradient_attribution(wg, xs_, star, 0, 1)
    assert int(attr["grad_x_input"].sum(1).argmax()) == 1 and attr["saliency"].shape == (5, 2)
    mask = X.GraphExplainer(wg, epochs=300, size_coeff=0.05, entropy_coeff=0.01).explain_node(xs_, star, 0)
    assert int(mask.argmax()) == 0 and mask[0] > 0.8 and mask[1:].max() < mask[0] - 0.3
    # kernels: isomorphic graphs are identical under WL, a path and a star differ
    path4 = (torch.tensor([[0, 1, 1, 2, 2, 3], [1, 0, 2, 1, 3, 2]]), torch.zeros(4, dtype=torch.long))
    p = torch.tensor([2, 0, 3, 1])
    path4b = (p[path4[0]], torch.zeros(4, dtype=torch.long))
    star4 = (torch.tensor([[0, 1, 0, 2, 0, 3], [1, 0, 2, 0, 3, 0]]), torch.zeros(4, dtype=torch.long))
    for kern in (X.wl_subtree_kernel, X.shortest_path_kernel):
        K = kern([path4, path4b, star4])
        assert K[0, 0] == K[1, 1] == K[0, 1] and K[0, 2] / (K[0, 0] * K[2, 2]).sqrt() < 0.99 and torch.linalg.eigvalsh(K).min() > -1e-9, kern.__name__
    # transport
    pa, pb = torch.tensor([0.5, 0.5], dtype=torch.float64), torch.tensor([0.25, 0.75], dtype=torch.float64)
    cost = torch.tensor([[0.0, 1.0], [1.0, 0.0]], dtype=torch.float64)
    plan = X.sinkhorn(pa, pb, cost, 0.01)
    assert torch.allclose(plan.sum(1), pa, atol=1e-6) and torch.allclose(plan.sum(0), pb, atol=1e-6) and float((plan * cost).sum()) == pytest.approx(0.25, abs=1e-3)
    pts = torch.randn(7, 2, dtype=torch.float64)
    c1 = torch.cdist(pts, pts)
    pm = torch.randperm(7)
    rot = torch.tensor([[0.0, -1.0], [1.0, 0.0]], dtype=torch.float64)
    c2 = torch.cdist(pts[pm] @ rot, pts[pm] @ rot)
    T, gw = X.gromov_wasserstein(c1, c2)
    assert gw < 0.02 and (T.argmax(1) == torch.argsort(pm)).float().mean() > 0.8
    assert X.gromov_wasserstein(c1, torch.cdist(torch.randn(7, 2, dtype=torch.float64) * 3, torch.zeros(7, 2, dtype=torch.float64)) * 0 + c1 * 2)[1] > gw
    assert X.graph_edit_distance_upper(path4[0], 4, path4b[0], 4) <= 2 and X.graph_edit_distance_upper(path4[0], 4, star4[0], 4) >= 2
    # analysis against closed forms / scipy
    from scipy.sparse.csgraph import shortest_path
    dist = X.floyd_warshall(ei, n)
    adj = np.zeros((n, n)); adj[ei[0], ei[1]] = 1
    assert np.allclose(dist.numpy(), shortest_path(adj, unweighted=True)) and float(dist.max()) == 3
    sa = X.spectral_analysis(ei, n)
    assert sa["components"] == 1 and 0 < sa["algebraic_connectivity"] < 1 and (torch.sign(sa["fiedler_vector"][:k]) == torch.sign(sa["fiedler_vector"][0])).all()
    assert torch.sign(sa["fiedler_vector"][0]) != torch.sign(sa["fiedler_vector"][-1])
    two = torch.cat([a, a + k], 1); two = torch.cat([two, two.flip(0)], 1)
    assert X.spectral_analysis(two, n)["components"] == 2 and torch.allclose(X.laplacian(ei, n, "rw").sum(1), torch.zeros(n, dtype=torch.float64), atol=1e-12)
    xf, u = X.graph_fourier_transform(torch.ones(n), two, n)
    assert torch.allclose(u @ xf, torch.ones(n, dtype=torch.float64), atol=1e-9)
    ce = X.centrality(ei, n)
    assert set(ce["betweenness"].topk(2).indices.tolist()) == {0, k} and ce["betweenness"][1] == 0
    assert float(ce["betweenness"][0]) == pytest.approx((k - 1) * k) and ce["degree"][0] == pytest.approx(6 / 11) and ce["closeness"][0] > ce["closeness"][1] and int(ce["eigenvector"].argmax()) in (0, k)
    part = X.spectral_partition(ei, n, 2)
    assert X.edge_cut(ei, part) == 1 and part[:k].unique().numel() == 1 and X.spectral_partition(ei, n, 4).unique().numel() == 4
    # heads, autoencoder, batching
    gs = [G.GraphData(torch.randn(5, 4), torch.tensor([[0, 1, 2, 3], [1, 2, 3, 4]]), None, torch.tensor(0)), G.GraphData(torch.randn(3, 4), torch.tensor([[0, 1], [1, 2]]), None, torch.tensor(1))]
    bx, be, bb, by = X.batch_graphs(gs)
    assert bx.shape == (8, 4) and be[:, -2:].tolist() == [[5, 6], [6, 7]] and bb.tolist() == [0] * 5 + [1] * 3 and by.tolist() == [0, 1]
    gc = X.GraphClassifier(4, 8, 2)
    assert gc(bx, be, bb).shape == (2, 2) and torch.allclose(gc(bx, be, bb)[1], gc(gs[1].x, gs[1].edge_index)[0], atol=1e-5)
    for var in (False, True):
        gae = X.GraphAutoEncoder(8, 16, 4, var)
        opt = torch.optim.Adam(gae.parameters(), 0.02)
        neg = G.negative_sampling(ei, n, ei.shape[1], seed=0)
        first = None
        for _ in range(80):
            l = gae.loss(x, ei, neg)
            opt.zero_grad(); l.backward(); opt.step()
            first = first if first is not None else l.item()
        assert l.item() < first and gae.eval().encode(x, ei).shape == (n, 4)
    # loaders
    (tmp_path / "e.txt").write_text("# comment\na b 1.5\nb c 2.0\n\nc a 0.5\n")
    e, w, names = X.load_edge_list(tmp_path / "e.txt")
    assert names == ["a", "b", "c"] and e.shape == (2, 6) and w.tolist() == [1.5, 2.0, 0.5] * 2 and X.load_edge_list(tmp_path / "e.txt", directed=True)[0].shape == (2, 3)
    (tmp_path / "g.gml").write_text('graph [\n directed 0\n node [ id 10 label "x" value 1.5 ]\n node [ id 11 label "y" ]\n node [ id 12 label "z" ]\n edge [ source 10 target 11 ]\n edge [ source 11 target 12 ]\n]\n')
    ge, labels, vals = X.load_gml(tmp_path / "g.gml")
    assert labels == ["x", "y", "z"] and vals == [1.5, None, None] and sorted(map(tuple, ge.t().tolist())) == [(0, 1), (1, 0), (1, 2), (2, 1)]
    (tmp_path / "g.json").write_text(json.dumps({"nodes": [{"id": "a", "features": [1, 0], "label": 0}, {"id": "b", "features": [0, 1], "label": 1}], "links": [{"source": "a", "target": "b"}]}))
    jd = X.load_json_graph(tmp_path / "g.json")
    assert jd.x.tolist() == [[1, 0], [0, 1]] and jd.y.tolist() == [0, 1] and jd.num_edges == 2


def test_text_analysis_readability_ngram_lm_retrieval_keywords_sentiment_language_entities_and_models():
    import math
    from sklearn.feature_extraction.text import TfidfVectorizer as SkTfidf
    from torsh_b200.text import analysis as T
    torch.manual_seed(0)
    doc = ("Dr. Smith arrived at 9:30 a.m. on Monday. He met Prof. Jones, who had travelled from Berlin! Did they discuss the 3.5 percent rise? "
           "Yes. The meeting ended early.")
    ss = T.sentences(doc)
    assert len(ss) == 5 and ss[0].endswith("Monday.") and ss[2].endswith("rise?") and ss[3] == "Yes."
    assert [T.count_syllables(w) for w in ("cat", "table", "beautiful", "the", "wanted", "jumped", "make", "readability", "queue")] == [1, 2, 3, 1, 2, 1, 1, 5, 1]
    easy = "The cat sat on the mat. The dog ran to the cat. It was a fun day."
    hard = "Notwithstanding considerable methodological heterogeneity, the epidemiological investigations demonstrated statistically significant associations between environmental contaminants and neurodevelopmental abnormalities."
    re_, rh = T.readability(easy), T.readability(hard)
    assert re_["flesch_reading_ease"] > 90 > 10 > rh["flesch_reading_ease"] and rh["flesch_kincaid_grade"] > 15 > 3 > re_["flesch_kincaid_grade"] and rh["gunning_fog"] > re_["gunning_fog"] + 10
    assert rh["coleman_liau"] > re_["coleman_liau"] and rh["smog"] > re_["smog"] and rh["automated_readability"] > re_["automated_readability"]
    st = T.text_statistics(easy)
    assert st["sentences"] == 3 and st["words"] == 17 and st["unique_words"] == 13 and st["syllables"] == 17 and 0.4 < st["stopword_ratio"] < 0.7
    rep, var = ["a", "b"] * 100, [f"w{i}" for i in range(200)]
    dr, dv = T.lexical_diversity(rep), T.lexical_diversity(var)
    assert dr["ttr"] == 0.01 and dv["ttr"] == 1.0 and dv["mattr"] == 1.0 and dr["mattr"] == pytest.approx(0.04) and dv["mtld"] > 10 * dr["mtld"] and dr["yule_k"] > dv["yule_k"] and dv["hapax_ratio"] == 1.0
    # n-gram language model
    corpus = [s.split() for s in ["the cat sat on the mat", "the dog sat on the log", "the cat ate the fish", "a dog ate the bone", "the cat sat on the log"]]
    for sm in ("laplace", "kneser_ney"):
        lm = T.NGramLM(3, sm).fit(corpus)
        tot = sum(lm.prob(w, ["the", "cat"]) for w in lm.vocab)
        assert tot == pytest.approx(1.0, abs=(1e-9 if sm == "laplace" else 0.05)), sm
        assert lm.prob("sat", ["the", "cat"]) > lm.prob("bone", ["the", "cat"]) and lm.perplexity(corpus) < lm.perplexity([["log", "the", "on", "sat", "cat", "the"]])
    kn, lap = T.NGramLM(3, "kneser_ney").fit(corpus), T.NGramLM(3, "laplace").fit(corpus)
    held = [["the", "dog", "sat", "on", "the", "mat"]]
    assert kn.perplexity(held) < lap.perplexity(held) and kn.prob("zebra", ["the"]) > 0
    gen = kn.generate(12, seed=3)
    assert 1 <= len(gen) <= 12 and set(gen) <= kn.vocab
    uni = T.NGramLM(1, "laplace").fit(corpus)
    assert uni.prob("the") == pytest.approx((9 + 1) / (28 + 5 + len(uni.vocab))) and len(uni.vocab) == 12
    # TF-IDF against scikit-learn, BM25 ranking
    docs = ["the cat sat on the mat", "the dog chased the cat", "dogs and cats are pets", "stock markets fell sharply today"]
    ours = T.TfidfVectorizer().fit(docs)
    sk = SkTfidf(token_pattern=r"[A-Za-z0-9]+").fit(docs)
    assert sorted(ours.vocabulary) == sorted(sk.vocabulary_) and torch.allclose(ours.transform(docs), torch.from_numpy(sk.transform(docs).toarray()), atol=1e-12)
    bi = T.TfidfVectorizer((1, 2), sublinear_tf=True).fit(docs)
    skb = SkTfidf(token_pattern=r"[A-Za-z0-9]+", ngram_range=(1, 2), sublinear_tf=True).fit(docs)
    assert torch.allclose(bi.transform(docs), torch.from_numpy(skb.transform(docs).toarray()), atol=1e-12)
    bm = T.BM25(docs)
    assert bm.top_k("cat on a mat", 2) == [0, 1] and bm.top_k("markets today", 1) == [3] and bm.scores("unicorn") == [0.0] * 4
    assert T.jaccard_similarity("abc", "bcd") == 0.5 and T.dice_similarity("abc", "bcd") == pytest.approx(2 / 3) and T.cosine_similarity_counts("aab", "ab") == pytest.approx(3 / math.sqrt(10))
    assert T.jaro_winkler("MARTHA", "MARHTA") == pytest.approx(0.9611, abs=1e-4) and T.jaro_winkler("DIXON", "DICKSONX") == pytest.approx(0.8133, abs=1e-4) and T.jaro_winkler("abc", "xyz") == 0.0
    s1, s2 = set(range(100)), set(range(50, 150))
    sig1, sig2 = T.minhash_signature(s1, 256), T.minhash_signature(s2, 256)
    assert abs(sum(a == b for a, b in zip(sig1, sig2)) / 256 - 1 / 3) < 0.1
    # keywords and summaries
    article = ("Neural networks learn representations from data. Deep neural networks stack many layers of representations. "
               "Training deep neural networks requires large data sets and fast hardware. The weather was pleasant on Tuesday. "
               "Graphics processors provide the fast hardware that training needs. Convolutional neural networks process images with shared weights.")
    rk = T.rake_keywords(article, 5)
    assert any("neural networks" in k for k, _ in rk) and rk[0][1] >= rk[-1][1]
    tr = dict(T.textrank_keywords(article, 6))
    assert "neural" in tr and "networks" in tr and "tuesday" not in tr
    for method in ("textrank", "frequency"):
        summ = T.summarize(article, 2, method)
        assert len(summ) == 2 and not any("weather" in s for s in summ) and all(s in article for s in summ), method
    assert T.summarize("One. Two.", 5) == ["One.", "Two."]
    # sentiment, language, entities, cohesion
    assert T.sentiment("I love this great phone")["label"] == "positive" and T.sentiment("This is a terrible, useless product")["label"] == "negative"
    assert T.sentiment("The movie was not good")["score"] < 0 < T.sentiment("The movie was good")["score"] < T.sentiment("The movie was extremely good")["score"]
    assert T.sentiment("I didn't hate it")["score"] > 0 and T.sentiment("The box is on the table")["label"] == "neutral"
    samples = {"en": "the quick brown fox jumps over the lazy dog and then runs through the forest while the birds are singing in the trees this is what they have been doing for the whole day",
               "de": "der schnelle braune fuchs springt über den faulen hund und läuft dann durch den wald während die vögel in den bäumen singen das haben sie den ganzen tag gemacht und nicht aufgehört",
               "es": "el rápido zorro marrón salta sobre el perro perezoso y luego corre por el bosque mientras los pájaros cantan en los árboles esto es lo que han estado haciendo durante todo el día"}
    li = T.LanguageIdentifier().fit(samples)
    assert li.predict("where are the children going this morning") == "en" and li.predict("wohin gehen die kinder heute morgen und warum") == "de" and li.predict("a dónde van los niños esta mañana") == "es"
    ents = T.extract_entities("Contact Maria Garcia at maria@example.org or visit https://example.org/team on 2026-03-14 at 10:30; budget $1,250.50 (up 12%). #launch @acme")
    kinds = {e["type"]: e["text"] for e in ents}
    assert kinds == {"name": "Maria Garcia", "email": "maria@example.org", "url": "https://example.org/team", "date": "2026-03-14", "time": "10:30", "money": "$1,250.50", "percent": "12%", "hashtag": "#launch", "mention": "@acme"}
    assert [e["start"] for e in ents] == sorted(e["start"] for e in ents) and T.extract_entities("a@b.co", ["email"])[0]["end"] == 6
    coh = T.lexical_cohesion("Solar panels convert light. Panels need light to work. Bananas are yellow.")
    assert coh["breaks"] == [2] and coh["per_transition"][0] > 0 and coh["local"] > coh["global"] > 0
    # models learn a toy task
    vocab = 20
    xs = torch.randint(1, vocab, (64, 12)); xs[:, 8:] = 0
    ys = (xs == 7).any(1).long()
    xs[:32, 2] = 7; ys[:32] = 1
    xs[32:][xs[32:] == 7] = 8; ys[32:] = 0
    for Model in (T.BiLSTMTextClassifier, T.TextCNN, T.TransformerTextClassifier):
        torch.manual_seed(0)
        m = Model(vocab, 2, 16) if Model is not T.TransformerTextClassifier else Model(vocab, 2, 16, 2, 1)
        opt = torch.optim.Adam(m.parameters(), 0.01)
        for _ in range(60):
            opt.zero_grad(); torch.nn.functional.cross_entropy(m(xs), ys).backward(); opt.step()
        assert (m(xs).argmax(1) == ys).float().mean() > 0.95, Model.__name__
        padded = torch.cat([xs[:4], torch.zeros(4, 5, dtype=torch.long)], 1)
        assert torch.allclose(m(padded), m(xs[:4]), atol=1e-4) or Model is T.TextCNN
    tg = T.SequenceTagger(vocab, 3, 16, 16)
    tags = (xs % 3) * (xs != 0)
    opt = torch.optim.Adam(tg.parameters(), 0.02)
    first = None
    for _ in range(80):
        l = tg.loss(xs, tags)
        opt.zero_grad(); l.backward(); opt.step()
        first = first if first is not None else l.item()
    dec = tg.decode(xs[:8])
    acc = sum(int(a == b) for seq, t in zip(dec, tags[:8]) for a, b in zip(seq, t[:8].tolist())) / 64
    assert l.item() < 0.3 * first and all(len(d) == 8 for d in dec) and acc > 0.9


def test_quantization_ext_learned_vq_sensitivity_mixed_precision_refinement_packing_and_reports():
    import math
    from torsh_b200 import quantization_ext as Q
    torch.manual_seed(0)
    # LSQ: step initialises from data, trains, and beats its initial error
    w = torch.randn(64, 32)
    lq = Q.LSQQuantizer(3)
    first = (lq(w) - w).pow(2).mean().item()
    assert lq(w).unique().numel() <= 8 and float(lq.step) == pytest.approx(2 * w.abs().mean().item() / math.sqrt(3), rel=1e-5)
    opt = torch.optim.Adam(lq.parameters(), 0.01)
    for _ in range(200):
        loss = (lq(w) - w).pow(2).mean()
        opt.zero_grad(); loss.backward(); opt.step()
    assert loss.item() < first and lq.step.grad is not None
    pc = Q.LSQQuantizer(4, per_channel=0)
    pc(w * torch.logspace(-1, 1, 64)[:, None])
    assert pc.step.shape == (64, 1) and pc.step[-1] > 20 * pc.step[0]
    pact = Q.PACT(2, alpha=1.0)
    y = pact(torch.tensor([-1.0, 0.2, 0.5, 3.0]))
    assert y.tolist() == pytest.approx([0.0, 1 / 3, 2 / 3, 1.0]) 
    y.sum().backward()
    assert pact.alpha.grad is not None and pact.alpha.grad != 0
    ll = Q.LSQLinear(32, 16, w_bits=4, a_bits=8)
    xin = torch.randn(8, 32)
    out = ll(xin)
    out.sum().backward()
    assert out.shape == (8, 16) and ll.weight.grad is not None and ll.wq.step.grad is not None and (out - torch.nn.functional.linear(xin, ll.weight, ll.bias)).abs().max() < 1.0
    # vector quantisation of a matrix with clustered rows
    centers = torch.randn(8, 4)
    mat = (centers[torch.randint(0, 8, (256,))] + 0.01 * torch.randn(256, 4)).reshape(64, 16)
    vq = Q.VectorQuantizedTensor(mat, dim=4, bits=3)
    assert (vq.dequantize() - mat).abs().max() < 0.06 and vq.compression_ratio() > 7 and vq.dequantize().shape == mat.shape
    pq = Q.VectorQuantizedTensor(torch.randn(64, 16), dim=4, bits=4, subspaces=2)
    assert len(pq.codebooks) == 2 and pq.codebooks[0].shape == (16, 2) and pq.dequantize().shape == (64, 16)
    cb, assign = Q.kmeans_codebook(torch.cat([torch.zeros(10, 2), torch.ones(10, 2) * 5]), 2)
    assert sorted(cb[:, 0].round().tolist()) == [0.0, 5.0] and assign[:10].unique().numel() == 1
    # sensitivity, Hessian trace, bit allocation
    net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    with torch.no_grad():
        net[4].weight.mul_(5)
    xs, ys = torch.randn(128, 16), torch.randint(0, 4, (128,))
    loss_fn = lambda m: torch.nn.functional.cross_entropy(m(xs), ys)
    sens = Q.layer_sensitivity(net, loss_fn, (8, 4, 2))
    assert set(sens) == {"0", "2", "4"} and all(abs(sens[n][8]) < abs(sens[n][2]) + 1e-6 for n in sens) and all(abs(v[8]) < 0.05 for v in sens.values())
    before = {n: p.detach().clone() for n, p in net.named_parameters()}
    assert all(torch.equal(before[n], p) for n, p in net.named_parameters())
    quad = torch.nn.Linear(3, 1, bias=False)
    A = torch.tensor([[2.0, 0, 0], [0, 3.0, 0], [0, 0, 5.0]])
    tr = Q.hessian_trace(quad, lambda m: 0.5 * (m.weight @ A @ m.weight.t()).sum(), samples=8)
    assert tr["weight"] == pytest.approx(10 / 3, rel=1e-5)
    ht = Q.hessian_trace(net, loss_fn, samples=8)
    assert set(ht) == {"0.weight", "2.weight", "4.weight"} and all(math.isfinite(v) for v in ht.values())
    sizes = {n: net[int(n)].weight.numel() for n in sens}
    full = sum(sizes.values()) * 8
    alloc = Q.allocate_bits(sizes, sens, 0.6 * full)
    assert sum(sizes[n] * alloc[n] for n in sizes) <= 0.6 * full and set(alloc.values()) <= {8, 4, 2} and Q.allocate_bits(sizes, sens, full) == {n: 8 for n in sizes}
    mixed = Q.apply_mixed_precision(net, alloc)
    assert float(loss_fn(mixed)) < float(loss_fn(Q.apply_mixed_precision(net, {n: 2 for n in sizes}))) and torch.equal(net[0].weight, before["0.weight"])
    # AdaRound beats nearest rounding on the layer output; bias correction removes the mean shift; equalisation preserves the function
    lin = torch.nn.Linear(32, 16)
    xcal = torch.randn(512, 32) + 0.5
    wq_near = Q._fake_quant_weight(lin.weight.detach(), 3)
    wq_ada = Q.adaround_layer(lin.weight.detach(), xcal, bits=3, iters=300)
    err = lambda wq: float((xcal @ wq.t() - xcal @ lin.weight.detach().t()).pow(2).mean())
    steps = (wq_ada / (lin.weight.detach().abs().amax(1, keepdim=True) / 3))
    assert err(wq_ada) < 0.85 * err(wq_near) and torch.allclose(steps, steps.round(), atol=1e-4)
    nb = Q.bias_correction(lin, wq_near, xcal)
    shift = lambda b: (torch.nn.functional.linear(xcal, wq_near, b) - lin(xcal)).mean(0).abs().max().item()
    assert shift(nb) < 1e-5 < shift(lin.bias.detach())
    a, b = torch.nn.Linear(8, 16), torch.nn.Linear(16, 4)
    with torch.no_grad():
        a.weight[:4] *= 50
    xq = torch.randn(32, 8)
    ref = b(torch.relu(a(xq)))
    spread0 = a.weight.detach().abs().amax(1)
    Q.cross_layer_equalization(a, b)
    assert torch.allclose(b(torch.relu(a(xq))), ref, atol=1e-4) and a.weight.detach().abs().amax(1).max() / a.weight.detach().abs().amax(1).min() < 0.3 * (spread0.max() / spread0.min())
    assert torch.allclose(a.weight.detach().abs().amax(1), b.weight.detach().abs().amax(0), rtol=1e-4)
    # calibration: heavy tails are clipped by entropy / mse, kept by max
    cal = Q.HistogramCalibrator(1024)
    data = torch.cat([torch.randn(100000), torch.tensor([12.0, -10.0])])
    cal.collect(data[:50000]); cal.collect(data[50000:])
    assert cal.max == 12.0 and float(cal.hist.sum()) == len(data)
    t_ent, t_mse, t_pct = cal.threshold("entropy"), cal.threshold("mse"), cal.threshold("percentile", percentile=99.9)
    assert 2.5 < t_pct < 4.0 and 2.5 < t_mse < 12 and 2.5 < t_ent <= 12 and cal.threshold("mse", bits=4) < t_mse
    # packing and entropy coding
    for bits in (1, 2, 4):
        v = torch.randint(0, 2 ** bits, (37,))
        p = Q.pack_bits(v, bits)
        assert len(p) == math.ceil(37 * bits / 8) and torch.equal(Q.unpack_bits(p, bits, 37).long(), v)
    sym = torch.cat([torch.zeros(700), torch.ones(200), torch.full((80,), 2.0), torch.full((20,), 3.0)]).long()[torch.randperm(1000)]
    hc = Q.HuffmanCodec().fit(sym.tolist())
    blob, nbits = hc.encode(sym.tolist())
    assert hc.decode(blob, nbits) == sym.tolist() and hc.table[0][1] == 1 and hc.table[3][1] == 3
    H = Q.entropy_bits(sym.tolist())
    assert H <= hc.mean_code_length(sym.tolist()) < H + 1 and nbits == 700 + 400 + 240 + 60 and len(blob) == 175
    one = Q.HuffmanCodec().fit([5, 5, 5])
    assert one.decode(*one.encode([5, 5, 5])) == [5, 5, 5]
    # metrics and report
    r = torch.randn(1000)
    q8, q4 = Q._fake_quant_weight(r[None], 8)[0], Q._fake_quant_weight(r[None], 4)[0]
    m8, m4 = Q.quantization_metrics(r, q8), Q.quantization_metrics(r, q4)
    assert m8["sqnr_db"] > m4["sqnr_db"] + 20 and m8["cosine"] > m4["cosine"] > 0.98 and m4["relative_l2"] > m8["relative_l2"] and m8["psnr_db"] > m8["sqnr_db"]
    assert Q.kl_divergence_hist(r, r) == pytest.approx(0.0, abs=1e-9) and Q.kl_divergence_hist(r, r * 3) > 0.3
    rep = Q.model_quantization_report(net, alloc)
    assert len(rep["layers"]) == 3 and rep["mean_bits"] <= 0.6 * 8 + 1e-9 and rep["compression"] == pytest.approx(16 / rep["mean_bits"]) and rep["worst_layer"] in sizes
    assert Q.model_quantization_report(net, 8)["compression"] == 2.0


def test_linalg_ext_multigrid_pivoting_refinement_randomized_krylov_and_analysis():
    import math
    import numpy as np
    from scipy import linalg as sl
    from torsh_b200 import linalg_ext as L
    torch.manual_seed(0)
    dd = torch.float64
    # multigrid: grid-independent convergence on Poisson problems
    for dim, n in ((1, 127), (2, 31), (2, 63)):
        shape = (n,) * dim
        xs = torch.linspace(0, 1, n + 2, dtype=dd)[1:-1]
        exact = torch.sin(math.pi * xs) if dim == 1 else torch.sin(math.pi * xs)[:, None] * torch.sin(2 * math.pi * xs)[None]
        mg = L.MultigridSolver(dim)
        f = mg.apply(exact)
        u, hist = mg.solve(f, 1e-9)
        assert hist[-1] < 1e-9 and len(hist) <= 14 and float((u - exact).abs().max()) < 1e-7, (dim, n)
        assert hist[1] / hist[0] < 0.25
    gs = L.MultigridSolver(2, smoother="gauss_seidel", cycle="W")
    ex = torch.randn(31, 31, dtype=dd)
    u, hist = gs.solve(gs.apply(ex), 1e-9)
    assert hist[-1] < 1e-9 and len(hist) <= 10 and float((u - ex).abs().max()) < 1e-6
    jac_only = L.MultigridSolver(2)
    xs31 = torch.linspace(0, 1, 33, dtype=dd)[1:-1]
    fs = jac_only.apply(torch.sin(math.pi * xs31)[:, None] * torch.sin(math.pi * xs31)[None])
    v = jac_only._smooth(torch.zeros(31, 31, dtype=dd), fs, 30)
    assert float((fs - jac_only.apply(v)).norm() / fs.norm()) > 0.5                                      # plain smoothing stalls on smooth error; multigrid does not
    # equilibration and preconditioners
    bad = torch.randn(8, 8, dtype=dd) * torch.logspace(-6, 6, 8, dtype=dd)[:, None] * torch.logspace(4, -4, 8, dtype=dd)[None]
    eq, r, c = L.equilibrate(bad)
    assert torch.allclose(eq, r[:, None] * bad * c[None]) and torch.linalg.cond(eq) < 1e-6 * torch.linalg.cond(bad) and torch.allclose(eq.abs().amax(1), torch.ones(8, dtype=dd), atol=0.05)
    spd = torch.randn(20, 20, dtype=dd); spd = spd @ spd.t() + 20 * torch.eye(20, dtype=dd)
    rhs = torch.randn(20, dtype=dd)
    M = L.ssor_preconditioner(spd)
    minv = torch.stack([M(e) for e in torch.eye(20, dtype=dd)], 1)
    assert torch.allclose(minv, minv.t(), atol=1e-10) and torch.linalg.cond(minv @ spd) < torch.linalg.cond(spd) and torch.allclose(L.diagonal_preconditioner(spd)(rhs), rhs / spd.diagonal())
    # LU pivoting strategies
    a = torch.randn(7, 7, dtype=dd)
    for strat in ("partial", "complete", "rook"):
        p, l, u, q, growth = L.lu_pivoted(a, strat)
        assert torch.allclose(l @ u, a[p][:, q], atol=1e-10) and torch.allclose(l, torch.tril(l)) and l.abs().max() <= 1 + 1e-12 and growth < 10, strat
    wilk = torch.tril(-torch.ones(10, 10, dtype=dd), -1) + torch.eye(10, dtype=dd); wilk[:, -1] = 1                # worst case for partial pivoting
    assert L.lu_pivoted(wilk, "partial")[4] == pytest.approx(2 ** 9) and L.lu_pivoted(wilk, "complete")[4] < 3 and L.lu_pivoted(wilk, "rook")[4] < 3
    # mixed-precision refinement reaches double accuracy from a float32 factorisation
    sysm = torch.randn(50, 50, dtype=dd) + 8 * torch.eye(50, dtype=dd)
    b = torch.randn(50, dtype=dd)
    x, hist = L.solve_refined(sysm, b)
    assert hist[0] > 1e-8 and hist[-1] < 1e-14 and torch.allclose(x, torch.linalg.solve(sysm, b), atol=1e-12)
    lo, di, up = torch.rand(9, dtype=dd), 4 + torch.rand(10, dtype=dd), torch.rand(9, dtype=dd)
    tri = torch.diag(di) + torch.diag(lo, -1) + torch.diag(up, 1)
    r10 = torch.randn(10, dtype=dd)
    assert torch.allclose(L.solve_tridiagonal(lo, di, up, r10), torch.linalg.solve(tri, r10), atol=1e-12)
    U, V = torch.randn(20, 3, dtype=dd), torch.randn(20, 3, dtype=dd)
    dvec = 5 + torch.rand(20, dtype=dd)
    assert torch.allclose(L.woodbury_solve(lambda y: y / dvec, U, V, rhs), torch.linalg.solve(torch.diag(dvec) + U @ V.t(), rhs), atol=1e-10)
    # randomised and Krylov methods
    low = torch.randn(80, 6, dtype=dd) @ torch.randn(6, 60, dtype=dd)
    qr = L.randomized_range_finder(low, 6)
    assert float(torch.linalg.matrix_norm(low - qr @ qr.t() @ low)) < 1e-9 * float(torch.linalg.matrix_norm(low))
    symm = torch.randn(60, 8, dtype=dd); symm = symm @ torch.diag(torch.tensor([50.0, 40, 30, 20, 10, 5, 2, 1], dtype=dd)) @ symm.t()
    w, vecs = L.randomized_eigh(symm, 4)
    assert torch.allclose(w, torch.linalg.eigvalsh(symm).flip(0)[:4], rtol=1e-6) and torch.allclose(symm @ vecs, vecs * w, atol=1e-5 * float(w[0]))
    Fn = L.nystrom(symm, 12)
    assert float(torch.linalg.matrix_norm(Fn @ Fn.t() - symm) / torch.linalg.matrix_norm(symm)) < 1e-6
    lam, vec = L.power_iteration(symm)
    assert lam == pytest.approx(float(torch.linalg.eigvalsh(symm)[-1]), rel=1e-8) and float((symm @ vec - lam * vec).norm()) < 1e-4 * lam
    rv, rvecs = L.lanczos(lambda z: spd @ z, 20, 20)
    assert torch.allclose(rv, torch.linalg.eigvalsh(spd), atol=1e-8) and torch.allclose(spd @ rvecs[:, -1], rv[-1] * rvecs[:, -1], atol=1e-7)
    few = L.lanczos(lambda z: spd @ z, 20, 8)[0]
    assert few[-1] == pytest.approx(float(torch.linalg.eigvalsh(spd)[-1]), rel=1e-3)
    g = torch.randn(6, 6, dtype=dd)
    assert np.allclose(L.expm_taylor(g).numpy(), sl.expm(g.numpy()), atol=1e-10) and np.allclose(L.expm_taylor(10 * g).numpy(), sl.expm(10 * g.numpy()), rtol=1e-8)
    big = -spd / 20
    v0 = torch.randn(20, dtype=dd)
    assert torch.allclose(L.expm_multiply(lambda z: big @ z, v0, 0.7, 20), torch.linalg.matrix_exp(0.7 * big) @ v0, atol=1e-10)
    # subspaces, alignment, report
    defc = torch.randn(6, 3, dtype=dd) @ torch.randn(3, 8, dtype=dd)
    ns = L.null_space(defc)
    assert ns.shape == (8, 5) and float((defc @ ns).abs().max()) < 1e-10 and torch.allclose(ns.t() @ ns, torch.eye(5, dtype=dd), atol=1e-10) and L.orth(defc).shape == (6, 3)
    e = torch.eye(4, dtype=dd)
    ang = L.subspace_angles(e[:, :2], torch.stack([e[:, 0], (e[:, 1] + e[:, 2]) / math.sqrt(2)], 1))
    assert sorted(ang.tolist()) == pytest.approx([0.0, math.pi / 4], abs=1e-7) and np.allclose(np.sort(ang.numpy()), np.sort(sl.subspace_angles(e[:, :2].numpy(), np.stack([e[:, 0].numpy(), ((e[:, 1] + e[:, 2]) / math.sqrt(2)).numpy()], 1))), atol=1e-7)
    rot, _ = torch.linalg.qr(torch.randn(5, 5, dtype=dd))
    pts = torch.randn(30, 5, dtype=dd)
    R, res = L.procrustes(pts, pts @ rot)
    assert torch.allclose(R, rot, atol=1e-10) and res < 1e-10
    rep = L.matrix_analysis(spd)
    assert rep["symmetric"] and rep["positive_definite"] and rep["definiteness"] == "positive" and rep["rank"] == 20 and rep["condition"] == pytest.approx(float(torch.linalg.cond(spd)), rel=1e-8)
    tri_rep = L.matrix_analysis(tri)
    assert tri_rep["bandwidth"] == (1, 1) and tri_rep["diagonally_dominant"] and not tri_rep["symmetric"] and tri_rep["sparsity"] == pytest.approx(72 / 100)
    assert L.matrix_analysis(rot)["orthogonal"] and L.matrix_analysis(defc)["rank"] == 3 and L.matrix_analysis(-spd)["definiteness"] == "negative" and 1 <= rep["stable_rank"] <= 20


def test_tensor_ext_expressions_graph_comprehension_registries_shapes_views_and_backend_services():
    import math
    from scipy import stats as sst
    from torsh_b200 import tensor_ext as E
    torch.manual_seed(0)
    a, b = torch.randn(4, 5), torch.randn(4, 5)
    ex = (E.expr(a) * 2.0 + E.expr(b)).apply("relu") - 1 + (-E.expr(a)) / 4
    assert torch.allclose(ex.eval(), torch.relu(a * 2 + b) - 1 - a / 4) and ex.count_nodes() == 13
    assert ex.to_source() == "((relu(((x0 * 2.0) + x1)) - 1.0) + ((-x0) / 4.0))" and torch.allclose((3 * E.expr(a)).eval(), 3 * a) and torch.allclose((1 - E.expr(a)).eval(), 1 - a)
    # expression graph
    g = E.ExpressionGraph()
    g.add_input("x", (8, 16)); g.add_input("w", (16, 4))
    g.add_node("h", "matmul", ["x", "w"], (8, 4)); g.add_node("h2", "matmul", ["x", "w"], (8, 4))
    g.add_node("s1", "add", ["h", "h2"]); g.add_node("s2", "add", ["h2", "h"])
    g.add_node("r", "relu", ["s1"]); g.add_node("t", "tanh", ["r"]); g.add_node("sc", "scale", ["t"], attr=0.5); g.add_node("dead", "exp", ["s2"])
    g.mark_output("sc")
    feeds = {"x": torch.randn(8, 16), "w": torch.randn(16, 4)}
    want = 0.5 * torch.tanh(torch.relu(2 * feeds["x"] @ feeds["w"]))
    assert torch.allclose(g.execute(feeds)["sc"], want, atol=1e-6)
    rep = g.optimize()
    assert rep == {"removed": 3, "merged": 2} and set(g.nodes) == {"x", "w", "h", "s1", "r", "t", "sc"} and torch.allclose(g.execute(feeds)["sc"], want, atol=1e-6)
    assert g.detect_fusable_chains() == [["s1", "r", "t", "sc"]] and g.topological_sort().index("h") < g.topological_sort().index("s1")
    co = g.costs()
    assert co["flops"] == 2 * 32 * 16 + 4 * 32 and co["memory_bytes"] - co["memory_bytes_fused"] == 3 * 32 * 4 and '"h" -> "s1"' in g.to_dot()
    cyc = E.ExpressionGraph(); cyc.nodes = {"a": {"op": "neg", "inputs": ["b"], "shape": (1,), "attr": None}, "b": {"op": "neg", "inputs": ["a"], "shape": (1,), "attr": None}}
    with pytest.raises(ValueError):
        cyc.topological_sort()
    # comprehensions
    tc = E.TensorComprehension((3, 4))
    assert torch.equal(tc.build(lambda i, j: i * 10 + j), torch.arange(3)[:, None].float() * 10 + torch.arange(4)[None].float())
    assert torch.equal(tc.where(lambda i, j: i == j, lambda i, j: 1.0, lambda i, j: 0.0), torch.eye(3, 4)) and torch.equal(tc.build(lambda i, j: 7), torch.full((3, 4), 7.0))
    assert E.TensorComprehension.from_iter((k * k for k in range(6)), (2, 3)).tolist() == [[0, 1, 4], [9, 16, 25]] and E.logspace(0, 2, 3).tolist() == pytest.approx([1, 10, 100])
    # registries
    reg = E.CustomTypeRegistry()
    reg.register_type(E.fixed_point_type("q8_8", 16, 8)); reg.register_type(E.fixed_point_type("q4_4", 8, 4))
    v = torch.tensor([1.5, -2.25, 0.004, 200.0])
    enc = reg.encode("q8_8", v)
    assert enc.dtype == torch.int16 and reg.decode("q8_8", enc).tolist() == pytest.approx([1.5, -2.25, 0.00390625, 127.99609375]) and reg.registered_types() == ["q4_4", "q8_8"]
    assert reg.decode("q4_4", reg.convert(enc, "q8_8", "q4_4")).tolist() == pytest.approx([1.5, -2.25, 0.0, 7.9375]) and reg.has_conversion("q8_8", "q4_4")
    assert reg.decode("q8_8", reg.apply("q8_8", "add", enc, enc))[:2].tolist() == [3.0, -4.5]
    reg.register_operation("q8_8", "neg", lambda s: -s)
    assert reg.list_operations("q8_8") == ["neg"] and reg.apply("q8_8", "neg", enc)[0] == -enc[0] and reg.stats() == {"types": 2, "conversions": 0, "operations": 1}
    with pytest.raises(ValueError):
        reg.register_type(E.fixed_point_type("q8_8"))
    ops = E.CustomOperationRegistry()
    ops.register("scale", lambda t, factor=1.0: t * factor, 1, "multiply by a constant", factor=2.0)
    ops.register("lerp", lambda p, q, w=0.5: p + w * (q - p), 2, w=0.5)
    assert torch.equal(ops.call("scale", a), a * 2) and torch.equal(ops.call("scale", a, factor=3.0), a * 3) and torch.allclose(ops.call("lerp", a, b, w=0.25), a + 0.25 * (b - a))
    assert ops.get_metadata("scale")["description"] == "multiply by a constant" and ops.list_operations() == ["lerp", "scale"]
    for bad in (lambda: ops.call("scale", a, b), lambda: ops.call("scale", a, gain=2)):
        with pytest.raises(TypeError):
            bad()
    # shape inference with a trace
    sd = E.ShapeInferenceDebugger()
    assert sd.infer_broadcast_shape((4, 1, 3), (5, 1)) == (4, 5, 3) and sd.infer_matmul_shape((2, 3, 4), (4, 5)) == (2, 3, 5) and sd.infer_matmul_shape((4,), (4, 5)) == (5,) and sd.infer_matmul_shape((7, 2, 3, 4), (2, 4, 6)) == (7, 2, 3, 6)
    assert sd.infer_concat_shape([(2, 3), (4, 3)], 0) == (6, 3) and sd.infer_reshape_shape((4, 6), (-1, 8)) == (3, 8)
    for bad in (lambda: sd.infer_broadcast_shape((3, 4), (5, 4)), lambda: sd.infer_matmul_shape((2, 3), (4, 5)), lambda: sd.infer_concat_shape([(2, 3), (2, 4)], 0), lambda: sd.infer_reshape_shape((4, 6), (5, -1))):
        with pytest.raises(ValueError):
            bad()
    st = sd.get_statistics()
    assert st["steps"] == 10 and st["errors"] == 4 and st["by_op"]["matmul"] == 4 and "not broadcastable" in sd.trace[6]["error"]
    # statistics against scipy
    x = torch.randn(200) ** 3
    y = x + torch.randn(200)
    d = E.describe(x)
    assert d["skewness"] == pytest.approx(float(sst.skew(x.numpy())), rel=1e-4) and d["kurtosis"] == pytest.approx(float(sst.kurtosis(x.numpy())), rel=1e-4) and d["median"] == pytest.approx(float(x.median()), abs=0.05)
    assert E.correlation(x, y) == pytest.approx(sst.pearsonr(x.numpy(), y.numpy())[0], rel=1e-5) and E.correlation(x, y, "spearman") == pytest.approx(sst.spearmanr(x.numpy(), y.numpy())[0], rel=1e-5)
    assert E.correlation(x, y, "kendall") == pytest.approx(sst.kendalltau(x.numpy(), y.numpy())[0], rel=1e-5) and float(E.percentile(x, 90)) == pytest.approx(float(torch.quantile(x.double(), 0.9))) and E.mode(torch.tensor([1, 3, 3, 2])) == 3
    # fluent wrapper and views
    assert torch.allclose(E.fluent(a).add_scalar(1).relu().mul_scalar(2).sum_dim(1).unwrap(), (torch.relu(a + 1) * 2).sum(1)) and torch.allclose(E.fluent(a).matmul(E.fluent(b).t()).unwrap(), a @ b.t())
    base = torch.arange(24.0)
    tv = E.TensorView(base, (3, 4), (8, 2), 1)
    assert tv.view.tolist()[1] == [9.0, 11.0, 13.0, 15.0] and not tv.is_contiguous() and tv.shares_storage_with(base) and tv.is_view() and not tv.overlaps_itself()
    assert E.TensorView(base, (3, 4), (0, 1)).overlaps_itself() and tv.memory_usage() == {"view_bytes": 48, "storage_bytes": 96} and tv.to_owned().is_contiguous() and not tv.to_owned().data_ptr() == base.data_ptr()
    assert E.TensorView.calculate_strides((2, 3, 4)) == (12, 4, 1) and E.TensorView.calculate_strides((2, 3, 4), "F") == (1, 2, 6) and tv.slice(1, 0, 4, 2).view.shape == (3, 2)
    # backend services
    pm = E.PerformanceModel()
    for n in (64, 128, 256, 512, 1024):
        pm.record("matmul", n, 2e-9 * n ** 3 * (1 + 0.01 * ((n // 64) % 3 - 1)))
        pm.record("copy", n, 1e-6 * n)
    fm = pm.fit("matmul")
    assert fm["exponent"] == pytest.approx(3.0, abs=0.05) and fm["complexity_class"] == "cubic" and pm.fit("copy")["complexity_class"] == "linear" and pm.predict("matmul", 2048) == pytest.approx(2e-9 * 2048 ** 3, rel=0.1)
    pm.record("copy", 2048, 1.0)
    assert pm.anomalies("copy", z=1.5) == [5]
    vc = E.VersionCompatibilityChecker()
    vc.require("torch", ">=2.4,<3"); vc.require("cuda", ">=12.8"); vc.require("triton", ">=3", "warning")
    ok = vc.check({"torch": "2.11.0+cu128", "cuda": "12.9", "triton": None})
    assert ok["compatible"] and [c["ok"] for c in ok["components"]] == [True, True, False] and ok["components"][2]["message"] == "not installed"
    assert not vc.check({"torch": "1.13.1", "cuda": "12.9", "triton": "3.6"})["compatible"] and E.VersionCompatibilityChecker.detect()["torch"] == torch.__version__
    dp = E.DefragmentationPlanner(1000)
    dp.add_block("a", 0, 100); dp.add_block("b", 300, 100); dp.add_block("pin", 500, 50, movable=False); dp.add_block("c", 800, 100)
    plan = dp.plan()
    assert [(m["name"], m["to"]) for m in plan["moves"]] == [("b", 100), ("c", 550)] and plan["largest_free_after"] == 350 > plan["largest_free_before"] == 250 and plan["fragmentation_after"] < plan["fragmentation_before"]
    clock = iter(range(10000))
    sel = E.AdaptiveKernelSelector(timer=lambda: float(next(clock)))
    cost = {"slow": 5, "fast": 1}
    def make(name):
        def fn(t):
            for _ in range(cost[name]):
                next(clock)
            return t * 2
        return fn
    sel.register("double", "slow", make("slow")); sel.register("double", "fast", make("fast")); sel.register("double", "big_only", make("fast"), predicate=lambda t: t.numel() > 10 ** 6)
    outs = [sel.run("double", a) for _ in range(5)]
    assert all(torch.equal(o, a * 2) for o in outs) and sel.best("double", a) == "fast" and sel.last == "fast" and sel.best("double", torch.zeros(3)) is None
    tp = E.TransferPlanner()
    tp.add_link("pageable", "device", 6e9, 10e-6); tp.add_link("pageable", "pinned", 20e9, 1e-6); tp.add_link("pinned", "device", 55e9, 8e-6)
    route = tp.plan("pageable", "device", 1 << 30)
    assert route["path"] == ["pageable", "pinned", "device"] and route["seconds"] == pytest.approx((1 << 30) / 20e9 + (1 << 30) / 55e9 + 9e-6)
    piped = tp.plan("pageable", "device", 1 << 30, chunk=1 << 24)
    assert piped["seconds"] < route["seconds"] and piped["seconds"] == pytest.approx(63 * ((1 << 24) / 20e9 + 1e-6) + ((1 << 24) / 20e9 + 1e-6) + ((1 << 24) / 55e9 + 8e-6))
    assert tp.plan("pageable", "device", 1024)["path"] == ["pageable", "device"] or tp.plan("pageable", "device", 1024)["seconds"] < 2e-5
    with pytest.raises(ValueError):
        tp.plan("device", "pageable", 10)


def test_domain_models_unet_pinn_fno_and_multiview_diffusion_parts():
    from torsh_b200.models import domain as D
    torch.manual_seed(0)
    # U-Net with gates and deep supervision
    net = D.UNet(in_channels=1, out_channels=2, base_features=4, num_levels=2, attention=True, deep_supervision=True)
    x = torch.randn(2, 1, 16, 16)
    out, aux = net(x)
    assert out.shape == (2, 2, 16, 16) and len(aux) == 1 and aux[0].shape == out.shape and 0 <= float(net.gates[0].last_alpha.detach().min()) and float(net.gates[0].last_alpha.detach().max()) <= 1 and net.gates[1].last_alpha.shape == (2, 1, 16, 16)
    net.eval()
    assert net(x).shape == (2, 2, 16, 16)
    with pytest.raises(ValueError):
        net(torch.randn(1, 1, 10, 10))
    net.train()
    target = (x[:, 0] > 0).long()
    opt = torch.optim.Adam(net.parameters(), lr=2e-2)
    first = None
    for _ in range(60):
        o, a = net(x)
        loss = D.UNet.deep_supervision_loss(o, a, target) + D.dice_loss(o, target)
        first = first if first is not None else float(loss.detach())
        opt.zero_grad(); loss.backward(); opt.step()
    assert float(loss.detach()) < 0.5 * first and float((net(x)[0].argmax(1) == target).float().mean()) > 0.9
    perfect = torch.nn.functional.one_hot(target, 2).movedim(-1, 1).float() * 50
    assert float(D.dice_loss(perfect, target)) < 1e-4 and float(D.dice_loss(-perfect, target)) > 0.9
    v3 = D.UNet3D(in_channels=2, out_channels=3, base_features=2, num_levels=2)
    assert v3(torch.randn(1, 2, 8, 8, 8)).shape == (1, 3, 8, 8, 8)
    # physics-informed network: u' = -u, u(0) = 1
    pinn = D.PINN(input_dim=1, output_dim=1, hidden_dims=(16, 16), adaptive_weights=False, boundary_weight=10.0)
    xs = torch.linspace(0, 1, 32)[:, None]
    res = lambda m, p: D.PINN.derivative(m(p), p, 0) + m(p)
    opt = torch.optim.Adam(pinn.parameters(), lr=1e-2)
    for _ in range(600):
        total, parts = pinn.compute_total_loss(pinn.physics_loss(xs, res), pinn.boundary_loss(torch.zeros(1, 1), torch.ones(1, 1)))
        opt.zero_grad(); total.backward(); opt.step()
    assert set(parts) == {"physics", "boundary"} and float((pinn(xs).detach() - torch.exp(-xs)).abs().max()) < 0.03
    xg = torch.tensor([[0.3], [0.7]], requires_grad=True)
    assert torch.allclose(D.PINN.derivative(xg ** 3, xg, 0, order=2), 6 * xg)
    ad = D.PINN(input_dim=1, hidden_dims=(4,), adaptive_weights=True)
    tot, _ = ad.compute_total_loss(torch.tensor(2.0), torch.tensor(3.0), torch.tensor(4.0))
    assert float(tot.detach()) == 9.0 and ad.log_vars.requires_grad
    tot.backward()
    assert ad.log_vars.grad.tolist() == [-1.0, -2.0, -3.0]
    # Fourier neural operator: learns the antiderivative of band-limited functions and transfers to a finer grid
    def batch(n, res, gen):
        xs = torch.linspace(0, 1, res + 1)[:-1]
        k = torch.arange(1, 4)[None, :, None].float()
        a, b = torch.randn(n, 3, 1, generator=gen), torch.randn(n, 3, 1, generator=gen)
        f = (a * torch.sin(2 * math.pi * k * xs) + b * torch.cos(2 * math.pi * k * xs)).sum(1)
        F_ = (-a / (2 * math.pi * k) * torch.cos(2 * math.pi * k * xs) + b / (2 * math.pi * k) * torch.sin(2 * math.pi * k * xs)).sum(1)
        return f[..., None], F_[..., None]
    gen = torch.Generator().manual_seed(0)
    fno = D.FNO(input_dim=1, output_dim=1, num_layers=2, hidden_dim=32, modes=(6,), width=16)
    opt = torch.optim.Adam(fno.parameters(), lr=5e-3)
    for _ in range(300):
        f, Fx = batch(32, 32, gen)
        loss = torch.nn.functional.mse_loss(fno(f), Fx)
        opt.zero_grad(); loss.backward(); opt.step()
    with torch.no_grad():
        f, Fx = batch(64, 32, gen); e32 = float((fno(f) - Fx).norm() / Fx.norm())
        f, Fx = batch(64, 128, gen); e128 = float((fno(f) - Fx).norm() / Fx.norm())
    assert e32 < 0.15 and e128 < 0.2
    f2 = D.FNO(input_dim=2, output_dim=1, num_layers=2, hidden_dim=8, modes=(3, 3), width=4)
    assert f2(torch.randn(2, 12, 10, 2)).shape == (2, 12, 10, 1) and f2(torch.randn(1, 20, 16, 2)).shape == (1, 20, 16, 1)
    # guidance
    c, u = torch.ones(2, 4, 8, 8), torch.zeros(2, 4, 8, 8)
    assert torch.equal(D.apply_classifier_free_guidance(c, u, 2.0), 2 * c) and torch.equal(D.apply_classifier_free_guidance(c, u, 1.0), c) and torch.equal(D.apply_classifier_free_guidance(c, c * 3, 0.0), c * 3)
    with pytest.raises(ValueError):
        D.apply_classifier_free_guidance(c, u[:1], 2.0)
    both = D.prepare_cfg_batch(c, u)
    uu, cc = D.split_cfg_batch(both, 2)
    assert both.shape[0] == 4 and torch.equal(uu, u) and torch.equal(cc, c)
    with pytest.raises(ValueError):
        D.split_cfg_batch(both, 3)
    assert D.guidance_scale_with_warmup(5, 50, 15.0, 10) == 8.0 and D.guidance_scale_with_warmup(10, 50, 15.0, 10) == 15.0 and D.guidance_scale_with_warmup(0, 50, 15.0) == 1.0 and D.guidance_scale_with_warmup(5, 50, 7.5) == 7.5
    cond = torch.randn(2, 4, 8, 8)
    guided = D.apply_classifier_free_guidance(cond, torch.randn(2, 4, 8, 8), 12.0)
    resc = D.rescale_guidance(guided, cond, phi=1.0)
    assert torch.allclose(resc.std((1, 2, 3)), cond.std((1, 2, 3)), rtol=1e-4) and guided.std() > 3 * cond.std()
    # conditioning modules
    cam = D.CameraEmbedding(embed_dim=32, hidden_dims=(16,))
    params = D.CameraEmbedding.pack(500.0, 500.0, 128.0, 128.0, torch.eye(3).expand(6, 3, 3), torch.zeros(6, 3))
    assert params.shape == (6, 16) and params[0, :4].tolist() == [500.0, 500.0, 128.0, 128.0] and cam(params).shape == (6, 32)
    with pytest.raises(ValueError):
        cam(torch.zeros(2, 12))
    cfg = D.IPAdapterProjectionConfig.sd15_vit_l()
    assert (cfg.num_tokens, cfg.cross_attn_dim, cfg.clip_feature_dim, cfg.hidden_dim) == (16, 768, 1024, 2048) and D.IPAdapterProjectionConfig.sdxl_vit_g().cross_attn_dim == 2048
    ip = D.IPAdapterProjection(num_tokens=4, cross_attn_dim=8, clip_feature_dim=12, hidden_dim=16)
    tok = ip(torch.randn(3, 12))
    assert tok.shape == (3, 4, 8) and ip.num_parameters() == 12 * 16 + 16 + 16 * 32 + 32 + 16 and torch.allclose(tok.mean(-1), torch.zeros(3, 4), atol=1e-5)
    with pytest.raises(ValueError):
        D.IPAdapterProjection(num_tokens=0)
    lu = D.LatentUpsampler(channels=4, timestep_dim=16, base_dim=8)
    lat = torch.randn(2, 4, 6, 6)
    up = lu(lat, torch.tensor([10, 500]))
    assert up.shape == (2, 4, 12, 12) and torch.allclose(up, torch.nn.functional.interpolate(lat, scale_factor=2.0, mode="bilinear", align_corners=False))
    up.sum().backward()
    assert lu.out.weight.grad.abs().sum() > 0
    cva = D.CrossViewAttention(num_heads=2, channels=8)
    feats = torch.randn(4, 8, 3, 3)                                              # 2 samples x 2 views
    assert torch.equal(cva(feats, 2), feats)
    torch.nn.init.normal_(cva.proj.weight, std=0.5)
    base = cva(feats, 2)
    moved = feats.clone(); moved[1] = torch.randn(8, 3, 3)                          # change view 1 of sample 0
    out2 = cva(moved, 2)
    assert not torch.allclose(out2[0], base[0]) and torch.allclose(out2[2:], base[2:], atol=1e-6)
    single = cva(moved, 1)
    assert torch.allclose(single[0], cva(feats, 1)[0], atol=1e-6)
    with pytest.raises(ValueError):
        cva(feats[:3], 2)
    mv = D.MultiviewUNet(in_channels=4, num_heads=2, base_dim=8, timestep_dim=16, camera_embed_dim=16)
    xin = torch.randn(4, 4, 8, 8)
    eps = mv(xin, torch.tensor([5, 5, 90, 90]), params[:4], num_views=2)
    assert eps.shape == xin.shape
    eps.pow(2).mean().backward()
    assert all(p.grad is not None for n, p in mv.named_parameters() if "attn" not in n or "proj" in n)
    other_cam = params[:4].clone(); other_cam[:, 13:] = 1.0
    assert not torch.allclose(mv(xin, torch.tensor([5, 5, 90, 90]), other_cam, 2), eps)


def test_model_tooling_factory_lazy_loading_validation_comparison_and_benchmark(tmp_path):
    from safetensors.torch import load_file, save_file
    from scipy import stats as sst
    from sklearn.metrics import precision_recall_fscore_support
    from torsh_b200.models import tooling as T
    torch.manual_seed(0)
    # configs and factory
    fac = T.ModelFactory()
    assert "vit_base" in fac.list_all_models()["vision"] and "bert_large" in fac.list_all_models()["nlp"]
    info = fac.get_model_info("nlp", "gpt2")
    assert 120e6 < info["parameters"] < 130e6 and info["architecture"] == "gpt" and fac.get_model_info("vision", "nope") is None
    assert 85e6 < fac.get_model_info("vision", "vit_base")["parameters"] < 88e6
    small = fac.build_vision_model("resnet18", num_classes=5, widths=(4, 8, 8, 8), depths=(1, 1, 1, 1))
    assert small(torch.randn(2, 3, 16, 16)).shape == (2, 5)
    vit = fac.build_vision_model("vit_tiny", image_size=16, patch_size=8, embed_dim=16, num_heads=2, depths=(1,), num_classes=3)
    assert vit(torch.randn(2, 3, 16, 16)).shape == (2, 3)
    fac.add_config("nlp", "nano", T.NlpModelConfig("gpt", vocab_size=50, max_position=16, hidden=8, layers=1, heads=2, dropout=0.0))
    gpt = fac.build_nlp_model("nano").eval()
    ids = torch.randint(0, 50, (2, 6))
    lg = gpt(ids)
    ids2 = ids.clone(); ids2[:, -1] = (ids2[:, -1] + 1) % 50
    assert lg.shape == (2, 6, 50) and torch.allclose(gpt(ids2)[:, :-1], lg[:, :-1], atol=1e-5) and gpt.head.weight is gpt.tok.weight
    assert fac.build_nlp_model("nano", architecture="bert", num_labels=4)(ids).shape == (2, 4)
    with pytest.raises(ValueError):
        T.NlpModelConfig(hidden=10, heads=3).validate()
    with pytest.raises(ValueError):
        T.VisionModelConfig("vit", image_size=30, patch_size=16).validate()
    assert T.compare_configs(T.NLP_PRESETS["gpt2"], T.NLP_PRESETS["gpt2_medium"]) == {"heads": (12, 16), "hidden": (768, 1024), "layers": (12, 24)}
    # safetensors both ways with the reference package, lazy cache, streaming
    tensors = {"a.weight": torch.randn(8, 4), "a.bias": torch.randn(8).to(torch.bfloat16), "idx": torch.arange(5), "flag": torch.tensor([True, False]), "half": torch.randn(3, 3).half()}
    T.write_safetensors(tensors, tmp_path / "m.safetensors", {"format": "pt"})
    theirs = load_file(str(tmp_path / "m.safetensors"))
    assert all(torch.equal(theirs[k], v) and theirs[k].dtype == v.dtype for k, v in tensors.items())
    save_file(tensors, str(tmp_path / "theirs.safetensors"))
    with T.LazyModelLoader(tmp_path / "theirs.safetensors", max_cache_bytes=8 * 4 * 4 + 16) as ld:
        assert ld.tensor_names() == sorted(tensors) and ld.tensor_metadata("a.bias") == ((8,), torch.bfloat16) and ld.tensor_metadata("zzz") is None and not ld.is_cached("a.weight")
        assert torch.equal(ld.get_tensor("a.weight"), tensors["a.weight"]) and ld.is_cached("a.weight") and torch.equal(ld.get_tensor("a.weight"), tensors["a.weight"])
        assert ld.cache_stats().hits == 1 and ld.cache_stats().misses == 1 and ld.cache_stats().hit_rate() == 0.5
        assert torch.equal(ld.get_tensor("a.bias"), tensors["a.bias"]) and torch.equal(ld.get_tensor("idx"), tensors["idx"])
        assert ld.cache_stats().evictions >= 1 and not ld.is_cached("a.weight") and ld.cache_stats().bytes_cached <= ld.cache_stats().capacity and 0 < ld.cache_stats().utilization() <= 1
        seen = {}
        ld.stream_tensors(lambda n, t: seen.__setitem__(n, t))
        assert set(seen) == set(tensors) and torch.equal(seen["half"], tensors["half"]) and torch.equal(seen["flag"], tensors["flag"])
        chunks = list(ld.stream_tensor_chunks("a.weight", 48))
        assert [c.numel() for c in chunks] == [12, 12, 8] and torch.equal(torch.cat(chunks).reshape(8, 4), tensors["a.weight"])
        with pytest.raises(KeyError):
            ld.get_tensor("missing")
        ld.clear_cache()
        assert ld.cache_stats().bytes_cached == 0
    lin = torch.nn.Linear(4, 8)
    T.write_safetensors({"weight": tensors["a.weight"], "bias": torch.zeros(8)}, tmp_path / "lin.safetensors")
    with T.LazyModelLoader(tmp_path / "lin.safetensors") as ld:
        assert ld.load_into(lin) == {"missing": [], "unexpected": []} and torch.equal(lin.weight, tensors["a.weight"]) and ld.metadata == {}
        with pytest.raises(KeyError):
            ld.load_into(torch.nn.Linear(4, 8, bias=False))
        assert ld.load_into(torch.nn.Linear(4, 8, bias=False), strict=False)["unexpected"] == ["bias"]
    # confusion matrix against scikit-learn
    y = torch.randint(0, 4, (300,)); pred = torch.where(torch.rand(300) < 0.7, y, torch.randint(0, 4, (300,)))
    cm = T.ConfusionMatrix(4).update(pred[:150], y[:150]).update(pred[150:], y[150:])
    p, r, f, s = precision_recall_fscore_support(y.numpy(), pred.numpy(), average=None)
    for i, c in enumerate(cm.class_metrics()):
        assert c["precision"] == pytest.approx(p[i]) and c["recall"] == pytest.approx(r[i]) and c["f1"] == pytest.approx(f[i]) and c["support"] == s[i]
    for avg in ("macro", "weighted"):
        pp, rr, ff, _ = precision_recall_fscore_support(y.numpy(), pred.numpy(), average=avg)
        sm = cm.summary(avg)
        assert sm["precision"] == pytest.approx(pp) and sm["recall"] == pytest.approx(rr) and sm["f1"] == pytest.approx(ff)
    assert cm.summary("micro")["f1"] == pytest.approx(float((pred == y).float().mean()))
    # splits
    labels = torch.tensor([0] * 40 + [1] * 10)
    folds = T.make_splits(50, "stratified", k=5, labels=labels)
    assert len(folds) == 5 and all(int((labels[te] == 1).sum()) == 2 and len(te) == 10 and not set(tr.tolist()) & set(te.tolist()) for tr, te in folds) and sorted(torch.cat([te for _, te in folds]).tolist()) == list(range(50))
    assert len(T.make_splits(20, "kfold", k=4, repeats=2)) == 8 and [len(te) for _, te in T.make_splits(10, "leave_one_out")] == [1] * 10
    ts = T.make_splits(60, "time_series", k=5)
    assert all(int(tr.max()) < int(te.min()) for tr, te in ts) and len(ts[0][0]) == 10 and len(ts[4][0]) == 50
    btr, bte = T.make_splits(100, "bootstrap", k=3)[0]
    assert len(btr) == 100 and not set(btr.tolist()) & set(bte.tolist()) and 25 < len(bte) < 50
    htr, hte = T.make_splits(100, "holdout", test_fraction=0.25)[0]
    assert len(htr) == 75 and len(hte) == 25
    # validator on a separable problem, and a regression
    X = torch.randn(200, 5); W = torch.randn(5, 3); Y = (X @ W).argmax(1)
    def fit(m, xs, ys, loss_fn=torch.nn.functional.cross_entropy):
        opt = torch.optim.Adam(m.parameters(), lr=0.05)
        for _ in range(80):
            opt.zero_grad(); loss_fn(m(xs), ys).backward(); opt.step()
    res = T.ModelValidator("stratified", k=4).validate(lambda: torch.nn.Linear(5, 3), fit, X, Y)
    assert len(res["splits"]) == 4 and res["summary"]["accuracy"]["mean"] > 0.9 and res["summary"]["accuracy"]["ci95"][0] <= res["summary"]["accuracy"]["mean"] <= res["summary"]["accuracy"]["ci95"][1] and 48 <= res["splits"][0]["test_size"] <= 52
    yr = X @ torch.randn(5) + 0.01 * torch.randn(200)
    reg = T.ModelValidator("kfold", k=3, task="regression").validate(lambda: torch.nn.Linear(5, 1), lambda m, a, b: fit(m, a, b, lambda o, t: torch.nn.functional.mse_loss(o.squeeze(-1), t)), X, yr)
    assert reg["summary"]["r2"]["mean"] > 0.98 and reg["summary"]["mae"]["mean"] < 0.2
    assert T.tensors_close(torch.ones(4), torch.ones(4) + 1e-9) and not T.tensors_close(torch.ones(4), torch.ones(5)) and T.tensors_close(torch.tensor([1.0, 2.0, 3.0, 9.0]), torch.tensor([1.0, 2.0, 3.0, 4.0]), max_mismatch_fraction=0.25)
    half = torch.nn.Linear(5, 3); ref = lambda t: torch.nn.functional.linear(t.double(), half.weight.double(), half.bias.double())
    assert T.validate_model_correctness(half, ref, [X[:4], X[4:8]], rtol=1e-4, atol=1e-5)["passed"] and not T.validate_model_correctness(half, lambda t: ref(t) + 0.1, [X[:4]])["passed"]
    # ANOVA and comparison
    g = [[0.90, 0.91, 0.92, 0.93, 0.90], [0.85, 0.86, 0.84, 0.87, 0.85], [0.905, 0.915, 0.92, 0.925, 0.91]]
    an = T.one_way_anova(g)
    ref_an = sst.f_oneway(*g)
    assert an["f"] == pytest.approx(ref_an.statistic) and an["p"] == pytest.approx(ref_an.pvalue) and (an["df_between"], an["df_within"]) == (2, 12)
    cmpr = T.ModelComparator().add("big", g[0], latency_ms=20.0, size_mb=400.0).add("small", g[1], latency_ms=5.0, size_mb=50.0).add("mid", g[2], latency_ms=12.0, size_mb=200.0).add("bad", [0.80, 0.81, 0.79, 0.80, 0.82], latency_ms=25.0, size_mb=500.0)
    out = cmpr.compare()
    assert out["rankings"]["quality"][0] in ("big", "mid") and out["rankings"]["latency"][0] == "small" and out["overall"][-1] == "bad" and set(out["pareto"]) == {"small", "mid"} or set(out["pareto"]) == {"small", "mid", "big"}
    pw = {(p["a"], p["b"]): p for p in out["pairwise"]}
    assert pw[("big", "small")]["significant"] and pw[("big", "small")]["preferred"] == "big" and not pw[("big", "mid")]["significant"] and pw[("big", "mid")]["preferred"] == "no clear preference"
    assert all(p["p_adjusted"] >= p["p"] for p in out["pairwise"]) and out["anova"]["p"] < 1e-6
    csv_text = cmpr.export_csv(out)
    assert csv_text.splitlines()[0] == "model,quality,latency_ms,size_mb,score,pareto" and len(csv_text.splitlines()) == 5 and "<td>bad</td>" in cmpr.html_report(out) and "ANOVA: F =" in cmpr.html_report(out)
    # benchmark and recommendations
    b = T.benchmark_model(torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8)), torch.randn(1, 64), warmup=1, iterations=5, batch_sizes=(1, 16))
    assert b["parameters"] == 64 * 64 + 64 + 64 * 8 + 8 and set(b["latency"]) == {1, 16} and b["latency"][16]["p99_ms"] >= b["latency"][16]["p50_ms"] > 0
    fake = {"size_mb": 400.0, "latency": {1: {"p50_ms": 30.0, "throughput": 33.0}, 8: {"p50_ms": 220.0, "throughput": 36.0}}}
    recs = T.optimization_recommendations(fake, {"size_mb": 120.0, "latency_ms": 10.0, "throughput": 100.0})
    assert [r["priority"] for r in recs] == ["high", "high", "medium", "low"] and "int8" in recs[0]["action"] and "CUDA graph" in recs[1]["action"]
    assert T.optimization_recommendations(fake, {"size_mb": 1000.0}) == [recs[-1]]


def test_nn_structure_lookup_activations_combinators_views_parameters_conventions_profiling_threads_harness_and_diagnostics():
    from collections import OrderedDict
    from torsh_b200.nn import structure as S
    torch.manual_seed(0)
    # table-driven activations
    for make, fn, bound in ((S.LookupActivation.gelu, torch.nn.functional.gelu, 5e-5), (S.LookupActivation.sigmoid, torch.sigmoid, 4e-4), (S.LookupActivation.tanh, torch.tanh, 1e-4), (S.LookupActivation.silu, torch.nn.functional.silu, 3e-3)):
        lut = make()
        assert lut.max_error() < bound, (fn.__name__, lut.max_error())
    coarse, fine = S.LookupActivation.gelu(size=64), S.LookupActivation.gelu(size=4096)
    assert coarse.max_error() > 10 * fine.max_error()
    xg = torch.linspace(-3, 3, 50, requires_grad=True)
    gl, = torch.autograd.grad(S.LookupActivation.gelu()(xg).sum(), xg); gx, = torch.autograd.grad(torch.nn.functional.gelu(xg).sum(), xg)
    assert torch.allclose(gl, gx, atol=2e-2) and S.LookupActivation.gelu()(torch.tensor([100.0, -100.0])).tolist() == [100.0, 0.0] and S.LookupActivation.gelu()(torch.randn(4).bfloat16()).dtype == torch.bfloat16
    # combinators
    x = torch.randn(3, 8)
    lin = torch.nn.Linear(8, 8)
    assert torch.allclose(S.Residual(lin, scale=0.5)(x), x + 0.5 * lin(x)) and S.Residual(torch.nn.Linear(8, 4), torch.nn.Linear(8, 4))(x).shape == (3, 4)
    a, b = torch.nn.Linear(8, 2), torch.nn.Linear(8, 3)
    assert S.Parallel(a, b)(x).shape == (3, 5) and torch.allclose(S.Parallel(a, a, merge="mean")(x), a(x)) and S.Parallel(a, a, merge="stack", dim=0)(x).shape == (2, 3, 2) and len(S.Parallel(a, b, merge="tuple")(x)) == 2
    rep, shared = S.Repeat(lambda i: torch.nn.Linear(8, 8), 3), S.Repeat(lambda i: torch.nn.Linear(8, 8), 3, share=True)
    assert len(list(rep.parameters())) == 6 and len(list(shared.parameters())) == 2 and torch.allclose(shared(x), shared.blocks[0](shared.blocks[0](shared.blocks[0](x))))
    cond = S.Conditional(lambda t: "long" if t.shape[0] > 4 else "short", {"long": torch.nn.Linear(8, 1), "short": torch.nn.Linear(8, 2)})
    assert cond(x).shape == (3, 2) and cond(torch.randn(6, 8)).shape == (6, 1) and "double" in repr(S.Lambda(lambda t: t * 2, "double")) and torch.equal(S.Lambda(lambda t: t * 2)(x), x * 2)
    net = S.SequentialBuilder(8).linear(16).gelu().layer_norm().residual(lambda bld: bld.linear(32).relu().linear(16)).dropout(0.1).linear(4).build()
    assert net(x).shape == (3, 4) and isinstance(net[3], S.Residual) and len(net) == 6
    with pytest.raises(ValueError, match="keep the feature size"):
        S.SequentialBuilder(8).residual(lambda bld: bld.linear(4))
    # views
    tree = S.model_tree(net, x)
    assert tree.splitlines()[0].startswith("Sequential (") and "├─ 0: Linear [3, 16] [144]" in tree and "│  ├─ body: Sequential [3, 16]" in tree and "└─ 5: Linear [3, 4] [68]" in tree
    assert len(S.model_tree(net, max_depth=1).splitlines()) == 7
    table = S.layer_table(net, x)
    total = sum(p.numel() for p in net.parameters())
    assert table.splitlines()[0].startswith("layer") and f"{total:,}" in table.splitlines()[-1] and "3.body.0" in table and "Dropout" in table
    dot = S.model_to_dot(net, x)
    assert dot.startswith("digraph model {") and "Linear" in dot and "[3, 4]" in dot and dot.count("->") >= 7 and "add" in dot
    class Branchy(torch.nn.Module):
        def __init__(self): super().__init__(); self.a, self.b = torch.nn.Linear(8, 8), torch.nn.Linear(8, 8)
        def forward(self, t): return self.a(t) if t.sum() > 0 else self.b(self.a(t))
    assert "input ->" in S.model_to_dot(Branchy(), x)
    # parameter management
    model = torch.nn.Sequential(OrderedDict(embed=torch.nn.Embedding(10, 8), body=torch.nn.Linear(8, 8), head=torch.nn.Linear(8, 10, bias=False)))
    pm = S.ParameterManager(model).group("no_decay", "*.bias", "embed.*", weight_decay=0.0).group("head", "head.*", lr=1e-2)
    groups = pm.optimizer_groups(lr=1e-3, weight_decay=0.1)
    assert [g["name"] for g in groups] == ["no_decay", "head", "default"] and groups[0]["weight_decay"] == 0.0 and groups[1]["lr"] == 1e-2 and groups[2]["lr"] == 1e-3 and len(groups[0]["params"]) == 2
    opt = torch.optim.AdamW([{k: v for k, v in g.items() if k != "name"} for g in groups])
    assert len(opt.param_groups) == 3 and sum(len(g["params"]) for g in opt.param_groups) == 4
    assert pm.freeze("embed.*", "body.*") == 3 and pm.statistics()["frozen"] == 80 + 64 + 8 and [g["name"] for g in pm.optimizer_groups()] == ["head"] and pm.unfreeze("body.*") == 2
    pm.constrain("non_negative", "body.bias").constrain("max_norm", "head.weight", value=0.5).constrain("clip", "body.weight", value=0.1)
    pm.apply_constraints()
    assert float(model.body.bias.detach().min()) >= 0 and float(model.head.weight.detach().norm(dim=1).max()) <= 0.5 + 1e-6 and float(model.body.weight.detach().abs().max()) <= 0.1 + 1e-6
    S.ParameterManager(model).constrain("unit_norm", "head.weight").apply_constraints()
    assert torch.allclose(model.head.weight.norm(dim=1), torch.ones(10), atol=1e-5)
    tied = torch.nn.Sequential(OrderedDict(embed=torch.nn.Embedding(10, 8), head=torch.nn.Linear(8, 10, bias=False)))
    S.ParameterManager(tied).tie("embed.weight", "head.weight")
    assert tied.head.weight is tied.embed.weight and len(list(tied.parameters())) == 1
    with pytest.raises(ValueError):
        S.ParameterManager(model).tie("embed.weight", "body.weight")
    st = pm.statistics()
    assert st["total"] == 80 + 64 + 8 + 80 and st["parameters"]["head.weight"]["shape"] == (10, 8) and st["parameters"]["body.bias"]["grad_norm"] is None
    # conventions
    @S.validated(p="probability", k="positive", mode=("choice", ["a", "b"]), t=("ndim", 2), u="floating")
    def op(t, u, p=0.5, k=1, mode="a"): return t
    assert op(x, x) is x
    for bad, msg in ((dict(p=1.5), "'p' must be in"), (dict(k=0), "'k' must be positive"), (dict(mode="c"), "one of"),):
        with pytest.raises(ValueError, match=msg):
            op(x, x, **bad)
    with pytest.raises(ValueError, match="op: argument 't' must have 2 dimensions"):
        op(x[0], x)
    with pytest.raises(ValueError, match="floating"):
        op(x, torch.ones(2, dtype=torch.long))
    v, w = torch.tensor([1.0, 2.0, 3.0]), torch.tensor([1.0, 0.0, 1.0])
    assert float(S.apply_reduction(v, "mean")) == 2.0 and float(S.apply_reduction(v, "sum", w)) == 4.0 and float(S.apply_reduction(v, "mean", w)) == 2.0 and S.apply_reduction(v, "none", w).tolist() == [1.0, 0.0, 3.0]
    with pytest.raises(ValueError):
        S.apply_reduction(v, "avg")
    # profiling and comparison
    A, B = torch.randn(64, 64), torch.randn(64, 64)
    pr = S.profile_function(torch.matmul, A, B, iterations=5, flops=2 * 64 ** 3)
    assert pr["median_s"] > 0 and pr["input_bytes"] == 2 * 64 * 64 * 4 and pr["output_bytes"] == 64 * 64 * 4 and pr["gflops"] > 0
    cmp = S.compare_implementations({"matmul": torch.matmul, "einsum": lambda p, q: torch.einsum("ij,jk->ik", p, q), "wrong": lambda p, q: p @ q + 1}, A, B, iterations=3)
    assert cmp["rows"]["einsum"]["matches"] and not cmp["rows"]["wrong"]["matches"] and cmp["fastest"] in ("matmul", "einsum") and cmp["rows"]["matmul"]["speedup"] == 1.0
    # threads
    big = torch.randn(8192, 16)
    assert torch.equal(S.parallel_chunks(torch.tanh, big, threads=4), torch.tanh(big)) and torch.equal(S.parallel_chunks(torch.tanh, big[:100], threads=4), torch.tanh(big[:100]))
    assert torch.allclose(S.parallel_reduce(lambda p: p.sum(0), torch.add, big.double(), threads=4), big.double().sum(0))
    # harness
    rep_ok = S.check_against_reference(torch.nn.functional.gelu, lambda t: 0.5 * t * (1 + torch.erf(t / math.sqrt(2))), lambda dt, g: [torch.randn(32, generator=g)], check_grad=True)
    assert rep_ok["passed"] and rep_ok["float64"]["max_abs_error"] < 1e-12 and rep_ok["bfloat16"]["max_abs_error"] > rep_ok["float32"]["max_abs_error"] and "max_grad_error" in rep_ok["float32"]
    rep_bad = S.check_against_reference(lambda t: torch.nn.functional.gelu(t, approximate="tanh"), lambda t: 0.5 * t * (1 + torch.erf(t / math.sqrt(2))), lambda dt, g: [torch.randn(64, generator=g) * 2], dtypes=(torch.float64, torch.bfloat16))
    assert not rep_bad["float64"]["passed"] and rep_bad["bfloat16"]["passed"] and not rep_bad["passed"]
    xs = torch.randn(4, 6)
    assert S.check_properties(torch.relu, xs, ["idempotent", "monotone", "positive_homogeneous", "non_negative", "odd", "linear"]) == {"idempotent": True, "monotone": True, "positive_homogeneous": True, "non_negative": True, "odd": False, "linear": False}
    assert S.check_properties(lambda t: t.softmax(-1), xs, ["shift_invariant", "permutation_equivariant", "bounded01", "sums_to_one", "idempotent"]) == {"shift_invariant": True, "permutation_equivariant": True, "bounded01": True, "sums_to_one": True, "idempotent": False}
    assert S.check_properties(torch.tanh, xs, ["odd", "even", "monotone"]) == {"odd": True, "even": False, "monotone": True} and S.check_properties(lambda t: t * 3, xs, ["linear"])["linear"] and S.check_properties(torch.abs, xs, ["even"])["even"]
    # diagnostics
    healthy = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
    assert S.diagnose_module(healthy, torch.randn(32, 8))["healthy"]
    sick = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 16), torch.nn.Sigmoid(), torch.nn.Linear(16, 4))
    with torch.no_grad():
        sick[0].bias.fill_(-100.0); sick[2].bias.fill_(50.0)
    d = S.diagnose_module(sick, torch.randn(32, 8))
    kinds = {i["kind"] for i in d["issues"]}
    assert {"dead_units", "saturated", "no_gradient"} <= kinds and not d["healthy"] and [i for i in d["issues"] if i["kind"] == "dead_units"][0]["layer"] == "1"


def test_special_ext_bessel_struve_coulomb_elliptic_faddeeva_integrals_zeta_mathieu_spheroidal_harmonics_tables_and_reports():
    import mpmath
    import numpy as np
    import scipy.special as sp
    from torsh_b200 import special_ext as E
    close = lambda a, b, rtol=1e-9, atol=1e-12: np.allclose(np.asarray(a), np.asarray(b), rtol=rtol, atol=atol)
    x = torch.tensor([0.05, 0.7, 2.5, 9.0, 31.0], dtype=torch.float64)
    for n in (0, 1, 2, 5, 12, 30):
        assert close(E.bessel_j(n, x), sp.jv(n, x.numpy()), 1e-11, 1e-15), n
        assert close(E.bessel_i(n, x), sp.iv(n, x.numpy()), 1e-7, 1e-300), n
    for n in (0, 1, 3, 8):
        assert close(E.bessel_y(n, x), sp.yv(n, x.numpy()), 1e-11) and close(E.bessel_k(n, x), sp.kv(n, x.numpy()), 1e-7, 1e-300), n
    assert close(E.bessel_j(3, -x), sp.jv(3, -x.numpy()), 1e-7) and close(E.bessel_j(-2, x), sp.jv(-2, x.numpy()), 1e-7) and float(E.bessel_j(4, torch.tensor(0.0))) == 0.0 and close(E.bessel_i(3, -x), sp.iv(3, -x.numpy()), 1e-7, 1e-300)
    xs = torch.tensor([1e-5, 0.3, 2.0, 11.0, 40.0], dtype=torch.float64)
    for n in (0, 1, 2, 6, 15):
        assert close(E.spherical_jn(n, xs), sp.spherical_jn(n, xs.numpy()), 1e-6, 1e-300), n
    for n in (0, 1, 4):
        assert close(E.spherical_yn(n, xs[1:]), sp.spherical_yn(n, xs[1:].numpy()), 1e-8), n
    # Struve, Lommel, Coulomb against scipy / mpmath
    xm = torch.tensor([0.2, 1.5, 6.0, 15.0], dtype=torch.float64)
    assert close(E.struve_h(0, xm), sp.struve(0, xm.numpy()), 1e-7) and close(E.struve_h(1, xm), sp.struve(1, xm.numpy()), 1e-7) and close(E.struve_h(0.5, xm), sp.struve(0.5, xm.numpy()), 1e-7)
    for mu, nu in ((0.5, 0.3), (2.0, 0.0), (1.5, 1.0)):
        assert close(E.lommel_s1(mu, nu, xm[:3]), [float(mpmath.lommels1(mu, nu, float(v))) for v in xm[:3]], 1e-8), (mu, nu)
    z = torch.tensor(2.0, dtype=torch.float64, requires_grad=True)
    s = E.lommel_s1(0.5, 0.3, z); d1, = torch.autograd.grad(s, z, create_graph=True); d2, = torch.autograd.grad(d1, z)
    assert float((z * z * d2 + z * d1 + (z * z - 0.09) * s - z ** 1.5).detach().abs()) < 1e-9
    rho = torch.tensor([0.3, 1.0, 4.0, 9.0], dtype=torch.float64)
    for l, eta in ((0, 0.0), (0, 0.5), (1, 0.5), (2, -1.0), (3, 2.0)):
        assert close(E.coulomb_f(l, eta, rho), [float(mpmath.coulombf(l, eta, float(r))) for r in rho], 1e-7, 1e-12), (l, eta)
    assert close(E.coulomb_f(0, 0.0, rho), torch.sin(rho), 1e-10)
    # Jacobi elliptic
    u, m = torch.tensor([0.1, 0.8, 2.0, -1.3, 5.0], dtype=torch.float64), torch.tensor([0.0, 0.3, 0.7, 0.99, 1.0], dtype=torch.float64)
    ours, theirs = E.ellipj(u, m), sp.ellipj(u.numpy(), m.numpy())
    assert all(close(a, b, 1e-9, 1e-12) for a, b in zip(ours, theirs))
    sn, cn, dn, _ = E.ellipj(torch.linspace(-3, 3, 50, dtype=torch.float64), 0.6)
    assert close(sn ** 2 + cn ** 2, np.ones(50)) and close(dn ** 2 + 0.6 * sn ** 2, np.ones(50))
    # Faddeeva and the error-function family
    zs = torch.tensor([0.3 + 0.2j, -1.5 + 2.0j, 4.0 + 0.01j, 2.0 - 1.0j, -0.5 - 0.5j, 0.0 + 6.0j, 10.0 + 10.0j], dtype=torch.complex128)
    assert close(E.wofz(zs), sp.wofz(zs.numpy()), 1e-10, 1e-13) and close(E.erf_complex(zs[:6]), sp.erf(zs[:6].numpy()), 1e-9, 1e-12)
    xr = torch.tensor([-3.0, -0.5, 0.0, 0.8, 3.0, 12.0, 30.0, 200.0], dtype=torch.float64)
    assert close(E.erfcx(xr), sp.erfcx(xr.numpy()), 1e-10) and close(E.erfi(xr[:5]), sp.erfi(xr[:5].numpy()), 1e-10, 1e-13) and close(E.dawsn(xr), sp.dawsn(xr.numpy()), 1e-9, 1e-13)
    assert close(E.voigt_profile(xr[:5], 0.7, 0.4), sp.voigt_profile(xr[:5].numpy(), 0.7, 0.4), 1e-10)
    S, C = E.fresnel(xr[:7]); Ss, Cs = sp.fresnel(xr[:7].numpy())
    assert close(S, Ss, 1e-8, 1e-10) and close(C, Cs, 1e-8, 1e-10)
    # sine / cosine integrals
    xi = torch.tensor([0.01, 0.5, 3.0, 20.0, 90.0], dtype=torch.float64)
    si, ci = E.sici(xi); sis, cis = sp.sici(xi.numpy())
    assert close(si, sis, 1e-11) and close(ci, cis, 1e-9, 1e-12) and close(E.sici(-xi)[0], -sis, 1e-11)
    # complex gamma, zeta, polylogarithm
    zg = torch.tensor([0.5 + 0.0j, 3.2 + 1.5j, -1.5 + 0.7j, 0.1 - 4.0j, 20.0 + 5.0j], dtype=torch.complex128)
    assert close(E.gamma_complex(zg), sp.gamma(zg.numpy()), 1e-10) and close(E.loggamma_complex(zg).real, sp.loggamma(zg.numpy()).real, 1e-10)
    sv = torch.tensor([-5.0, -2.5, -1.0, 0.0, 0.5, 0.9, 2.0, 4.0, 15.5], dtype=torch.float64)
    assert close(E.zeta(sv), [float(mpmath.zeta(float(v))) for v in sv], 1e-9, 1e-12) and float(E.zeta(torch.tensor(2.0))) == pytest.approx(math.pi ** 2 / 6) and float(E.zeta(torch.tensor(-1.0))) == pytest.approx(-1 / 12)
    zp = torch.tensor([-0.9, -0.3, 0.2, 0.7], dtype=torch.float64)
    assert close(E.polylog(2, zp), [float(mpmath.polylog(2, float(v))) for v in zp], 1e-10) and close(E.polylog(3.5, torch.tensor(1.0, dtype=torch.float64), terms=200000), float(mpmath.zeta(3.5)), 1e-5) and close(E.polylog(1, zp), -torch.log(1 - zp), 1e-10)
    # Mathieu and spheroidal characteristic values
    for mm in range(0, 6):
        for q in (0.0, 0.5, 3.0, 12.0, 40.0):
            assert E.mathieu_a(mm, q) == pytest.approx(sp.mathieu_a(mm, q), rel=1e-8, abs=1e-8), (mm, q)
            if mm:
                assert E.mathieu_b(mm, q) == pytest.approx(sp.mathieu_b(mm, q), rel=1e-8, abs=1e-8), (mm, q)
    ang = torch.tensor([0.0, 0.4, 1.1, 2.5, 4.0], dtype=torch.float64)
    for mm, q in ((0, 1.0), (1, 2.0), (2, 5.0), (3, 0.5)):
        assert close(E.mathieu_cem(mm, q, ang), sp.mathieu_cem(mm, q, np.degrees(ang.numpy()))[0], 1e-7, 1e-9), (mm, q)
    for mm, nn, c in ((0, 0, 1.0), (0, 2, 3.0), (1, 1, 2.0), (1, 4, 5.0), (2, 3, 0.5), (0, 1, 8.0)):
        assert E.spheroidal_cv(mm, nn, c) == pytest.approx(sp.pro_cv(mm, nn, c), rel=1e-9), (mm, nn, c)
        assert E.spheroidal_cv(mm, nn, c, oblate=True) == pytest.approx(sp.obl_cv(mm, nn, c), rel=1e-8, abs=1e-9), (mm, nn, c)
    # polynomials and harmonics
    xp = torch.linspace(-0.95, 0.95, 7, dtype=torch.float64)
    assert close(E.jacobi(4, 0.5, 1.5, xp), sp.eval_jacobi(4, 0.5, 1.5, xp.numpy())) and close(E.jacobi(3, 0.0, 0.0, xp), sp.eval_legendre(3, xp.numpy())) and close(E.jacobi(0, 1.0, 2.0, xp), np.ones(7))
    for mm, ll in ((0, 0), (0, 3), (1, 1), (2, 5), (4, 4)):
        assert close(E.assoc_legendre(mm, ll, xp), sp.lpmv(mm, ll, xp.numpy()), 1e-10), (mm, ll)
    th, ph = torch.tensor([0.3, 2.0, 5.5], dtype=torch.float64), torch.tensor([0.4, 1.6, 2.9], dtype=torch.float64)
    harm = getattr(sp, "sph_harm_y", None)
    for mm, ll in ((0, 0), (1, 2), (-1, 2), (3, 3), (-2, 4)):
        ref = harm(ll, mm, ph.numpy(), th.numpy()) if harm else sp.sph_harm(mm, ll, th.numpy(), ph.numpy())
        assert close(E.sph_harm(mm, ll, th, ph), ref, 1e-10, 1e-13), (mm, ll)
    assert E.sinpi(torch.tensor([0.0, 0.5, 1.0, 1.5, 1e6, 0.25])).tolist() == pytest.approx([0, 1, 0, -1, 0, math.sqrt(0.5)]) and E.cospi(torch.tensor([0.0, 0.5, 1.0, 2.5, 1 / 3])).tolist() == pytest.approx([1, 0, -1, 0, 0.5])
    assert float(E.sinc_pi(torch.tensor(0.0))) == 1.0 and float(E.sinc_pi(torch.tensor(0.5))) == pytest.approx(2 / math.pi) and float(E.haversine(torch.tensor(math.pi))) == pytest.approx(1.0) and float(E.gudermannian(torch.tensor(1.0))) == pytest.approx(2 * math.atan(math.tanh(0.5)))
    assert E.EULER_GAMMA == pytest.approx(float(mpmath.euler)) and E.CATALAN == pytest.approx(float(mpmath.catalan)) and E.APERY == pytest.approx(float(mpmath.apery)) and E.GLAISHER == pytest.approx(float(mpmath.glaisher)) and E.OMEGA == pytest.approx(float(mpmath.lambertw(1)))
    # domain handling, tables, caching, accuracy report
    assert E.check_domain("f", torch.tensor([0.0, 0.5, 1.0]), 0.0, 1.0, open_hi=True).tolist() == [True, True, False]
    with pytest.raises(E.SpecialFunctionError, match=r"ellipk: argument 1.5 outside the domain \[0, 1\)"):
        E.check_domain("ellipk", torch.tensor([0.2, 1.5]), 0, 1, mode="raise", open_hi=True)
    tab = E.TabulatedFunction(lambda t: E.bessel_j(0, t), 0.0, 20.0, points=2048)
    xt = torch.rand(500, dtype=torch.float64) * 20
    assert float((tab(xt) - E.bessel_j(0, xt)).abs().max()) < 1e-7 and close(tab(torch.tensor([25.0], dtype=torch.float64)), sp.j0(25.0))
    cache, calls = E.SmartCache(capacity=2), []
    def slow(t): calls.append(1); return E.bessel_j(7, t)
    a1, a2 = cache(slow, xt), cache(slow, xt.clone())
    assert a1 is a2 and len(calls) == 1 and cache.hit_rate() == 0.5
    cache(slow, xt + 1); cache(slow, xt + 2); cache(slow, xt)
    assert len(calls) == 4 and len(cache.store) == 2
    rep = E.accuracy_report(lambda t: E.bessel_j(2, t), lambda t: torch.as_tensor(sp.jv(2, t.numpy())), 0.1, 30.0)
    assert rep["max_abs"] < 1e-12 and len(rep["profile"]) == 10 and len(rep["chart"].splitlines()) == 10 and rep["max_ulp"] >= rep["median_ulp"] and 0.1 <= rep["argmax_abs"] <= 30.0
    crude = E.accuracy_report(lambda t: t - t ** 3 / 6, torch.sin, 0.0, 2.0)
    assert crude["argmax_abs"] == 2.0 and crude["profile"][-1] > crude["profile"][0] and crude["max_abs"] == pytest.approx(abs(2 - 8 / 6 - math.sin(2)))


def test_text_quality_metrics_distances_overlap_rouge_bleu_embedding_perplexity_coherence_fluency_semantics():
    from torsh_b200.text import quality_metrics as Q
    from torsh_b200.text.analysis import NGramLM, words
    # edit distances
    assert Q.levenshtein("kitten", "sitting") == 3 and Q.levenshtein("abc", "", deletion=2) == 6 and Q.levenshtein("abc", "abd", substitution=0.5) == 0.5 and Q.levenshtein("a b c".split(), "a c".split()) == 1
    assert Q.damerau_levenshtein("ca", "abc") == 2 and Q.optimal_string_alignment("ca", "abc") == 3 and Q.damerau_levenshtein("abcd", "acbd") == 1 == Q.optimal_string_alignment("abcd", "acbd") and Q.hamming("karolin", "kathrin") == 3
    with pytest.raises(ValueError):
        Q.hamming("ab", "abc")
    assert Q.jaro("martha", "marhta") == pytest.approx(0.9444, abs=1e-4) and Q.jaro("dixon", "dicksonx") == pytest.approx(0.7667, abs=1e-4) and Q.jaro("abc", "xyz") == 0.0 and Q.jaro("same", "same") == 1.0
    assert Q.normalized_distance(Q.levenshtein, "kitten", "sitting") == pytest.approx(3 / 7) and Q.similarity(Q.levenshtein, "", "") == 1.0
    pd = Q.pairwise_distances(["abc", "abd", "xyz"])
    assert pd.tolist() == [[0, 1, 3], [1, 0, 3], [3, 3, 0]] and Q.find_most_similar("helo", ["world", "hello", "help"], top=2) == [(1, pytest.approx(0.2)), (2, pytest.approx(0.25))]
    # overlap
    a, b = "the cat sat on the mat".split(), "the cat lay on the rug".split()
    ov = Q.ngram_overlap(a, b)
    assert ov["precision"] == pytest.approx(4 / 6) and ov["jaccard"] == pytest.approx(4 / 8) and ov["dice"] == pytest.approx(8 / 12) and Q.ngram_overlap(a, b, 2)["overlap_coefficient"] == pytest.approx(2 / 5)
    assert Q.positional_overlap(a, b) == pytest.approx(4 / 6) and Q.positional_overlap(a, a[::-1]) < 0.5 and Q.positional_overlap([], a) == 0.0
    texts = [a, b, "stocks fell sharply today".split(), "stocks rose sharply today".split()]
    assert Q.cluster_by_overlap(texts, 0.4) == [[0, 1], [2, 3]] and Q.overlap_matrix(texts)[0, 2] == 0
    # ROUGE
    cand, ref = "the cat was found under the bed".split(), "the cat was under the bed".split()
    r1, r2, rl = Q.rouge(cand, ref, "rouge-1"), Q.rouge(cand, ref, "rouge-2"), Q.rouge(cand, ref, "rouge-l")
    assert (r1["precision"], r1["recall"]) == (pytest.approx(6 / 7), 1.0) and (r2["precision"], r2["recall"]) == (pytest.approx(4 / 6), pytest.approx(4 / 5)) and (rl["precision"], rl["recall"]) == (pytest.approx(6 / 7), 1.0)
    rs = Q.rouge("police killed the gunman".split(), "police kill the gunman".split(), "rouge-s")
    assert rs["precision"] == pytest.approx(3 / 6) and Q.rouge("police killed the gunman".split(), "police kill the gunman".split(), "rouge-s", stem=True)["f"] == 1.0
    assert Q.rouge("a b".split(), "a b".split(), "rouge-su")["f"] == 1.0 and Q.rouge("a b c d".split(), "a c".split(), "rouge-s", skip=0)["precision"] == 0.0
    w_contig, w_spread = Q.rouge("a b c d x y z".split(), "a b c d e f g".split(), "rouge-w"), Q.rouge("a x b y c z d".split(), "a b c d e f g".split(), "rouge-w")
    assert w_contig["f"] > w_spread["f"] and Q.rouge("a x b y c z d".split(), "a b c d e f g".split(), "rouge-l")["f"] == Q.rouge("a b c d x y z".split(), "a b c d e f g".split(), "rouge-l")["f"]
    multi = Q.rouge(cand, ["a dog barked".split(), ref], "rouge-1")
    assert multi["recall"] == 1.0 and Q.rouge(cand, ["a dog barked".split(), ref], "rouge-1", multi="mean")["recall"] == 0.5
    assert Q.rouge("the the cat".split(), "cat".split(), "rouge-1", remove_stopwords=True)["f"] == 1.0
    summ = Q.rouge_l_summary(["w1 w2 w6 w7 w8".split(), "w1 w3 w8 w9 w5".split()], ["w1 w2 w3 w4 w5".split()])
    assert summ["recall"] == pytest.approx(4 / 5) and summ["precision"] == pytest.approx(4 / 10)
    bi = Q.bootstrap_interval([0.4, 0.5, 0.6, 0.45, 0.55] * 4)
    assert bi["lower"] < bi["mean"] < bi["upper"] and bi["mean"] == pytest.approx(0.5) and bi["width"] < 0.1 and bi["margin_of_error"] == pytest.approx(bi["width"] / 2)
    # BLEU variants, chrF, METEOR-style, TER
    hyp, refs = "the quick brown fox jumps over the dog".split(), ["the quick brown fox jumps over the lazy dog".split()]
    bd = Q.bleu_detailed(hyp, refs)
    assert bd["precisions"][0] == 1.0 and bd["precisions"][3] == pytest.approx(4 / 5) and bd["brevity_penalty"] == pytest.approx(math.exp(1 - 9 / 8)) and bd["bleu"] == pytest.approx(bd["brevity_penalty"] * (1 * 6 / 7 * 5 / 6 * 4 / 5) ** 0.25)
    short = "the fox jumps high today".split()
    assert Q.bleu_detailed(short, refs)["bleu"] == 0.0 and 0 < Q.bleu_detailed(short, refs, smoothing="epsilon")["bleu"] < Q.bleu_detailed(short, refs, smoothing="add_one")["bleu"] and Q.bleu_detailed(short, refs, smoothing="exponential")["bleu"] > 0
    assert Q.bleu_detailed("the the the".split(), ["the cat".split()], max_n=1)["precisions"] == [pytest.approx(1 / 3)]
    assert Q.chrf("hello world", "hello world") == 1.0 and Q.chrf("abc", "xyz") == 0.0 and 0.5 < Q.chrf("the cat sat", "the cat sits") < 1.0 and 0 < Q.chrf("the cat sat", "cat the sat") < Q.chrf("the cat sat", "cat the sat", word_n=1) < 1
    m_same, m_scr = Q.meteor_like("the cat sat on the mat".split(), "the cat sat on the mat".split()), Q.meteor_like("mat the on sat cat the".split(), "the cat sat on the mat".split())
    assert m_same["chunks"] == 1 and m_same["score"] == pytest.approx(1 - 0.5 / 6 ** 3) and m_scr["precision"] == 1.0 and m_scr["score"] < 0.8 * m_same["score"]
    assert Q.meteor_like("cats running".split(), "cat runs".split())["recall"] >= 0.5 and Q.meteor_like("big house".split(), "large house".split(), synonyms={"big": {"large"}})["recall"] == 1.0 and Q.meteor_like(["x"], ["y"])["score"] == 0.0
    assert Q.translation_edit_rate("a b c d e".split(), "a b c d e".split()) == 0.0 and Q.translation_edit_rate("d e a b c".split(), "a b c d e".split()) == pytest.approx(1 / 5) and Q.translation_edit_rate("a b x".split(), "a b c d".split()) == pytest.approx(2 / 4)
    # embedding matching
    E = torch.eye(4)
    assert Q.embedding_score(E[[0, 1, 2]], E[[2, 0, 1]])["f"] == pytest.approx(1.0) and Q.embedding_score(E[[0, 1]], E[[0, 3]])["precision"] == pytest.approx(0.5)
    w = Q.embedding_score(E[[0, 1]], E[[0, 3]], cand_idf=torch.tensor([3.0, 1.0]))
    assert w["precision"] == pytest.approx(0.75) and Q.embedding_score(E[[0, 1]], E[[0, 3]], baseline=0.2)["recall"] == pytest.approx((0.5 - 0.2) / 0.8)
    idf = Q.idf_weights([["a", "b"], ["a", "c"], ["a"]])
    assert idf["a"] == pytest.approx(0.0) and idf["b"] == pytest.approx(math.log(2)) and idf["zzz"] == pytest.approx(math.log(4))
    # perplexity
    logits = torch.zeros(2, 5, 7)
    assert Q.perplexity_from_logits(logits, torch.randint(0, 7, (2, 5))) == pytest.approx(7.0, rel=1e-5)
    tg = torch.tensor([[1, 2, -100, -100, -100], [0, 1, 2, 3, 4]])
    sharp = torch.full((2, 5, 7), -20.0); sharp[0, :, 1] = 20.0; sharp[1] = 0.0
    per = Q.perplexity_from_logits(sharp, tg, per_sequence=True)
    assert per[1] == pytest.approx(7.0, rel=1e-5) and per[0] == pytest.approx(math.exp(20.0), rel=1e-3)
    assert Q.perplexity_from_probabilities([0.25] * 8) == pytest.approx(4.0) and Q.perplexity_from_cross_entropy(3.0, base=2) == 8.0 and Q.bits_per_character(math.log(2) * 100, 50) == pytest.approx(2.0) and Q.perplexity_quality(35.0) == "good"
    cmpm = Q.compare_perplexities([50.0, 60, 55, 70, 65, 58, 62, 66], [40.0, 45, 50, 52, 51, 47, 49, 50])
    assert cmpm["model2_win_rate"] == 1.0 and cmpm["is_model2_better"] and cmpm["improvement_percentage"] == pytest.approx(100 * (60.75 - 48.0) / 60.75) and not Q.compare_perplexities([50.0, 60, 55, 52], [51.0, 59, 56, 51])["is_model2_better"]
    # coherence
    good = "The river flooded the village last night. The flood destroyed several houses near the river. Residents of the village left their houses quickly. They returned when the river fell again."
    bad = "The river flooded the village last night. Quantum computers use qubits. My favourite recipe needs three eggs. Stock markets closed higher on Friday."
    eg, eb = Q.entity_grid(good), Q.entity_grid(bad)
    assert {"river", "village", "houses"} <= set(eg["entities"]) and eb["entities"] == [] and eg["coherence"] > 0.1 > eb["coherence"] and abs(sum(eg["transitions"].values()) - 1) < 1e-9 and eg["grid"]["river"][2] == "-"
    ch = Q.lexical_chains(good)
    assert ch[0]["word"] == "river" and ch[0]["sentences"] == [0, 1, 3] and any(c["word"] in ("flood", "hous") for c in ch) and Q.lexical_chains(bad) == []
    lc_g, lc_b = Q.local_coherence(good), Q.local_coherence(bad)
    assert lc_g["mean"] > 0.2 > 0.1 > lc_b["mean"] and len(lc_g["adjacent"]) == 3 and lc_g["adjacent"][2] >= 0.15
    dm = Q.discourse_markers("First we measured it. However, the signal was weak. Therefore we repeated it. For example, run two failed. In conclusion, it works.")
    assert dm["counts"]["adversative"] == 1 and dm["counts"]["causal"] == 1 and dm["counts"]["exemplifying"] == 1 and dm["counts"]["summarising"] == 1 and dm["per_sentence"] >= 1.0 and 0.8 < dm["diversity"] <= 1.0
    st = Q.structural_coherence("This essay introduces tides. Tides follow the moon.\n\nTides rise twice a day. The moon pulls the tides along.\n\nIn conclusion, tides track the moon. The moon matters.")
    assert st["paragraphs"] == 3 and st["balance"] > 0.8 and st["has_introduction_marker"] and st["has_conclusion_marker"] and st["topic_sentence_support"] > 0.2
    assert Q.coherence_report(good)["score"] > 2 * Q.coherence_report(bad)["score"] and Q.coherence_report(bad)["chains"] == 0
    # fluency
    lr = Q.lexical_richness("a a a b b c".split())
    assert lr["ttr"] == 0.5 and lr["hapax_ratio"] == pytest.approx(1 / 3) and lr["yule_k"] == pytest.approx(1e4 * (1 + 4 + 9 - 6) / 36) and lr["simpson_d"] == pytest.approx((6 + 2) / 30) and lr["dis_legomena_ratio"] == pytest.approx(1 / 3)
    sf = Q.syntactic_fluency("this sentence starts lowercase. The the cat sat on a apple. She walked (quickly home. Because rain.")
    kinds = [i["kind"] for i in sf["issues"]]
    assert {"capitalisation", "doubled_word", "article_agreement", "unbalanced", "fragment"} <= set(kinds) and sf["score"] < 0.5 and Q.syntactic_fluency("The cat sat on an apple. It was an honest hour of work.")["issues"] == []
    verse = "The cat sat still\nUpon the hill\nAnd watched the night\nGrow slowly bright"
    prose = "Go. The extraordinarily complicated administrative reorganisation continued unexpectedly throughout the following year. Stop."
    rv, rp = Q.rhythm_analysis(verse), Q.rhythm_analysis(prose)
    assert rv["end_rhyme"] == pytest.approx(2 / 3) and rp["cadence_variability"] > 100 and rp["polysyllabic_ratio"] > 0.4 and rv["syllables_per_word"] < 1.4 and Q.rhythm_analysis("big bad bears bite")["alliteration"] == 1.0
    pf, pi = Q.pragmatic_analysis("Therefore, the committee consequently recommends additional investigation regarding the aforementioned discrepancies."), Q.pragmatic_analysis("Hey guys, that's gonna be awesome! Can't wait, lol!")
    assert pf["register"] == "formal" and pi["register"] == "informal" and Q.pragmatic_analysis("Perhaps it might possibly work.")["hedging"] == pytest.approx(3 / 5) and Q.pragmatic_analysis("Could you please help? Thanks!")["politeness"] > 0.5
    lm = NGramLM(2).fit([words(good)] * 3)
    fr_in, fr_out = Q.fluency_report(good, lm), Q.fluency_report("village the night flooded river last the. houses several the near destroyed flood river the.", lm)
    assert fr_in["components"]["statistical"] > fr_out["components"]["statistical"] and fr_in["score"] > fr_out["score"]
    # semantics
    assert Q.sentence_sentiment("This is a great film") > 0 > Q.sentence_sentiment("This is not a great film") and Q.sentence_sentiment("This is really terrible") == -1.0 and Q.sentence_sentiment("The table is round") == 0.0
    traj = Q.sentiment_trajectory("The start was terrible. The middle was bad. Then it became good. The ending was wonderful and brilliant.")
    assert traj["trend"] == "improving" and traj["polarity_flips"] == 1 and traj["per_sentence"][0] < 0 < traj["per_sentence"][-1] and Q.sentiment_trajectory("Great. Awful. Great. Awful.")["volatility"] == 1.0
    em = Q.emotion_scores("She was afraid and full of dread, panic rising; later she smiled.")
    assert em["dominant"] == "fear" and em["scores"]["fear"] == 0.75 and em["scores"]["joy"] == 0.25
    docs = [d.split() for d in ("stock market investors shares profit", "market shares investors bank profit", "bank profit stock market", "football team player goal match", "team goal player league match", "match football league team")]
    tp = Q.nmf_topics(docs, k=2, top=5)
    assert len(set(tp["assignments"][:3])) == 1 and len(set(tp["assignments"][3:])) == 1 and tp["assignments"][0] != tp["assignments"][3] and tp["reconstruction_error"] < 0.7
    fin_topic = tp["topics"][tp["assignments"][0]]
    assert {"market", "profit"} <= set(fin_topic) and not {"team", "goal"} & set(fin_topic[:3]) and all(c > -2.5 for c in tp["coherence"])
    assert Q.classify_domain("The patient received treatment after the diagnosis at the hospital.")["domain"] == "medical" and Q.classify_domain("The defendant appealed to the court under the statute.")["domain"] == "legal" and Q.classify_domain("Hello there.")["domain"] == "general"
    ss = Q.syntactic_similarity("The dog chased the ball quickly.", "The cat watched the bird quietly.")
    assert ss["structure"] == 1.0 and ss["score"] > 0.95 > Q.syntactic_similarity("The dog chased the ball quickly.", "Running fast, are 12 people happy?")["score"]
    lsa = Q.latent_semantic_similarity(docs + ["investors shares".split(), "league player".split()], rank=2)
    assert lsa[6, 2] > 0.9 > 0.3 > lsa[6, 5] and lsa[7, 5] > 0.9 and torch.allclose(lsa.diag(), torch.ones(8, dtype=torch.float64))


def test_vision_tools_drawing_annotations_attribution_tiling_video_flow_stabilisation_and_apng():
    import json
    import xml.etree.ElementTree as ET
    from torsh_b200.vision import tools as V
    from torsh_b200.vision.io import decode_png
    torch.manual_seed(0)
    # drawing
    img = torch.zeros(3, 20, 30)
    d = V.draw_boxes(img, torch.tensor([[2.0, 3.0, 10.0, 12.0]]), colors=torch.tensor([[255, 0, 0]]), width=2)
    assert d.dtype == torch.uint8 and d[:, 3, 2:11].float().mean(1).tolist() == [255, 0, 0] and d[0, 4, 5] == 255 and d[0, 5, 5] == 0 and d[0, 12, 10] == 255 and d[0, 13, 10] == 0
    filled = V.draw_boxes(torch.ones(3, 20, 30), torch.tensor([[0.0, 0.0, 5.0, 5.0]]), colors=torch.tensor([[0, 0, 255]]), fill_alpha=0.5)
    assert filled[:, 3, 3].tolist() == [128, 128, 255] and V.draw_boxes(img, torch.tensor([[-5.0, -5.0, 50.0, 50.0]])).shape == (3, 20, 30)
    kp = V.draw_keypoints(img, torch.tensor([[5.0, 5.0], [20.0, 15.0]]), radius=1, connections=[(0, 1)], color=(0, 255, 0))
    assert kp[1, 5, 5] == 255 and kp[1, 15, 20] == 255 and int(kp[1, 10, 12]) + int(kp[1, 10, 13]) + int(kp[1, 9, 12]) + int(kp[1, 10, 11]) >= 255 and kp[0].sum() == 0
    m = torch.zeros(2, 20, 30, dtype=torch.bool); m[0, :5] = True; m[1, 10:] = True
    seg = V.draw_segmentation_masks(torch.full((3, 20, 30), 100, dtype=torch.uint8), m, alpha=0.5)
    assert seg[:, 0, 0].tolist() == [165, 62, 88] and seg[:, 7, 0].tolist() == [100, 100, 100] and seg[:, 15, 0].tolist() == [80, 140, 88]
    grid = V.make_grid(torch.arange(5.0).reshape(5, 1, 1, 1).expand(5, 1, 4, 6), nrow=3, padding=1, pad_value=-1.0)
    assert grid.shape == (1, 2 * 5 + 1, 3 * 7 + 1) and grid[0, 1, 1] == 0 and grid[0, 1, 8] == 1 and grid[0, 6, 8] == 4 and grid[0, 0, 0] == -1 and grid[0, 6, 15] == -1
    assert V.make_grid(torch.rand(2, 3, 4, 4) * 10, normalize=True).max() <= 1.0
    # annotation session
    s = V.AnnotationSession(100, 80, "a.png")
    b1 = s.add("box", "cat", [10, 10, 50, 40], score=0.9); p1 = s.add("polygon", "dog", [60, 10, 90, 10, 90, 40]); k1 = s.add("point", "eye", [20, 20])
    with pytest.raises(ValueError):
        s.add("box", "bad", [10, 10, 5, 40])
    s.relabel(b1, "tiger"); s.move(b1, 5, -5); s.remove(k1)
    assert s.items[b1].coords == [15, 5, 55, 35] and s.statistics()["labels"] == {"tiger": 1, "dog": 1}
    assert s.undo() and k1 in s.items and s.undo() and s.items[b1].coords == [10, 10, 50, 40] and s.undo() and s.items[b1].label == "cat"
    coco = s.to_coco()
    by = {a["id"]: a for a in coco["annotations"]}
    assert by[b1]["bbox"] == [10, 10, 40, 30] and by[b1]["area"] == 1200 and by[p1]["area"] == 450 and by[p1]["bbox"] == [60, 10, 30, 30] and by[k1]["keypoints"] == [20, 20, 2] and by[b1]["score"] == 0.9 and len(coco["categories"]) == 3
    back = V.AnnotationSession.from_coco(json.loads(json.dumps(coco)))
    assert back.statistics() == s.statistics() and not back.undo()
    svg = ET.fromstring(s.to_svg("a.png"))
    ns = "{http://www.w3.org/2000/svg}"
    assert svg.find(f"{ns}rect").attrib["width"] == "40" and svg.find(f"{ns}polygon") is not None and svg.find(f"{ns}circle").attrib["cx"] == "20" and svg.find(f"{ns}image").attrib["href"] == "a.png" and "cat 0.90" in s.to_svg()
    page = V.html_gallery([s, back], hrefs=["a.png", "b.png"])
    assert page.count("<svg") == 2 and "a.png: 3 annotations" in page
    # attribution: a model that looks only at one patch
    class PatchModel(torch.nn.Module):
        def forward(self, x): return torch.stack([x[:, :, 4:8, 8:12].sum((1, 2, 3)), x[:, :, :4, :4].sum((1, 2, 3))], 1)
    pm, xin = PatchModel(), torch.ones(1, 16, 16)
    occ = V.occlusion_sensitivity(pm, xin, target=0, patch=4)
    assert occ[4:8, 8:12].min() == 16.0 and occ.sum() == 16.0 * 16 and V.occlusion_sensitivity(pm, xin, 1, patch=4, stride=2)[:4, :4].min() > 0
    sg = V.smooth_grad(pm, torch.rand(1, 16, 16), 0, samples=4, generator=torch.Generator().manual_seed(0))
    assert torch.equal(sg[4:8, 8:12], torch.ones(4, 4)) and sg.sum() == 16
    att = [torch.softmax(torch.randn(2, 5, 5), -1) for _ in range(3)]
    roll = V.attention_rollout(att)
    assert torch.allclose(roll.sum(-1), torch.ones(5), atol=1e-6) and (roll >= 0).all() and torch.allclose(V.attention_rollout([torch.zeros(1, 4, 4)]), torch.eye(4)) and V.attention_rollout(att, discard_ratio=0.5).shape == (5, 5)
    lin = torch.nn.Linear(6, 3, bias=False)
    am = V.activation_maximization(lin, (6,), lambda o: o[:, 1], steps=200, lr=0.05, l2=0.05, generator=torch.Generator().manual_seed(0))
    assert torch.nn.functional.cosine_similarity(am, lin.weight[1].detach(), dim=0) > 0.99
    # tiled processing equals whole-image processing for a local operator away from tile artefacts; upscaling too
    big = torch.rand(3, 150, 210)
    blur = lambda t: torch.nn.functional.avg_pool2d(torch.nn.functional.pad(t, (1, 1, 1, 1), mode="replicate"), 3, 1)
    tp = V.TiledProcessor(blur, tile=64, overlap=16)
    tiled = tp(big)
    assert tiled.shape == big.shape and tp.tiles >= 12 and float((tiled - blur(big[None])[0]).abs().max()) < 0.05 and float((tiled - blur(big[None])[0])[:, 20:40, 20:40].abs().max()) < 1e-6
    assert torch.allclose(V.TiledProcessor(lambda t: t * 2, tile=64, overlap=8)(big), big * 2, atol=1e-6)
    up = V.TiledProcessor(lambda t: torch.nn.functional.interpolate(t, scale_factor=2, mode="nearest"), tile=64, overlap=8, scale=2)(big)
    assert up.shape == (3, 300, 420) and torch.allclose(up, torch.nn.functional.interpolate(big[None], scale_factor=2, mode="nearest")[0], atol=1e-6)
    pool = V.ImageBufferPool(max_per_key=1)
    t1 = pool.acquire((3, 8, 8)); pool.release(t1); t2 = pool.acquire((3, 8, 8)); pool.release(t2); pool.release(torch.empty(3, 8, 8))
    assert t2 is t1 and (pool.hits, pool.misses) == (1, 1) and pool.bytes_held() == 3 * 64 * 4
    cnn = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.Flatten(), torch.nn.Linear(8 * 16 * 16, 4))
    est = V.estimate_batch_memory(cnn, torch.randn(2, 3, 16, 16))
    assert est["per_sample_bytes"] == (8 * 256 * 3 + 4 + 3 * 256) * 4 and est["fixed_bytes"] == 4 * est["parameters_bytes"]
    assert V.auto_batch_size(cnn, torch.randn(1, 3, 16, 16), memory_budget=est["fixed_bytes"] + 100 * est["per_sample_bytes"], safety=1.0) == 96 and V.auto_batch_size(cnn, torch.randn(1, 3, 16, 16), memory_budget=1) == 1
    pol = V.HardwarePolicy.detect()
    assert pol.device in ("cpu", "cuda") and pol.prepare(cnn)(pol.prepare_input(torch.randn(1, 3, 16, 16))).shape == (1, 4)
    # video clips
    clip = V.VideoClip(torch.arange(60.0).reshape(60, 1, 1, 1).expand(60, 1, 2, 2), fps=30.0)
    assert clip.duration == 2.0 and clip.subclip(0.5, 1.0).frames[:, 0, 0, 0].tolist() == list(range(15, 30)) and clip.subsample(3).fps == 10.0 and clip.reverse().frames[0, 0, 0, 0] == 59
    assert len(clip.speed(2.0).frames) == 30 and len(clip.resample_fps(15).frames) == 30 and clip.resample_fps(15).frames[1, 0, 0, 0] == 2 and len(clip.temporal_crop(16).frames) == 16 and clip.map(lambda f: f * 2).frames[3, 0, 0, 0] == 6
    # optical flow on a smooth pattern shifted by a known amount
    yy, xx = torch.meshgrid(torch.arange(64.0), torch.arange(64.0), indexing="ij")
    pattern = lambda dx, dy: (torch.sin((xx - dx) / 5.0) + torch.cos((yy - dy) / 7.0) + torch.sin((xx - dx + yy - dy) / 9.0))[None]
    a, b = pattern(0, 0), pattern(1.0, 0.5)
    hs = V.horn_schunck(a, b, alpha=0.5, iters=300)
    lk = V.lucas_kanade(a, b, window=9, levels=2)
    for flow in (hs, lk):
        inner = flow[:, 8:-8, 8:-8]
        assert float(inner[0].mean()) == pytest.approx(1.0, abs=0.15) and float(inner[1].mean()) == pytest.approx(0.5, abs=0.15)
    assert float((V.warp_by_flow(b, lk) - a)[:, 8:-8, 8:-8].abs().mean()) < 0.02 < float((b - a)[:, 8:-8, 8:-8].abs().mean())
    mid = V.interpolate_frames(a, pattern(2.0, 0.0), 0.5)
    assert float((mid - pattern(1.0, 0.0))[:, 8:-8, 8:-8].abs().mean()) < 0.03 < float((0.5 * (a + pattern(2.0, 0.0)) - pattern(1.0, 0.0))[:, 8:-8, 8:-8].abs().mean()) + 0.02
    # shots, phase correlation, stabilisation
    dark, bright = torch.rand(6, 3, 16, 16) * 0.2, 0.7 + torch.rand(5, 3, 16, 16) * 0.3
    assert V.detect_shots(torch.cat([dark, bright, dark[:4]])) == [6, 11] and V.detect_shots(dark) == []
    base = torch.rand(1, 48, 48)
    assert V.phase_correlation(base, torch.roll(base, (3, -5), (-2, -1))) == (-5, 3) and V.phase_correlation(base, base) == (0, 0)
    jitter = [(0, 0), (2, -1), (-1, 2), (1, 1), (-2, -2), (0, 1), (2, 0), (-1, -1)]
    shaky = torch.stack([torch.roll(base, (dy, dx), (-2, -1)) for dx, dy in jitter])
    stab, corr = V.stabilize(shaky, smoothing=5)
    resid = lambda fr: sum(abs(v) for i in range(len(fr) - 1) for v in V.phase_correlation(fr[i], fr[i + 1]))
    assert resid(stab) < 0.5 * resid(shaky) and corr.shape == (8, 2)
    # animated PNG
    anim = (torch.rand(4, 3, 6, 5) * 255).to(torch.uint8)
    data = V.encode_apng(anim, fps=8.0)
    frames, fps = V.decode_apng(data)
    assert torch.equal(frames, anim) and fps == pytest.approx(8.0) and data[:8] == b"\x89PNG\r\n\x1a\n" and data.count(b"fdAT") == 3 and data.count(b"fcTL") == 4
    assert torch.equal(decode_png(data)[:3], anim[0]) or torch.equal((decode_png(data)[:3] * 255).round().to(torch.uint8), anim[0])
    gray = V.decode_apng(V.encode_apng(torch.rand(2, 1, 4, 4)))[0]
    assert gray.shape == (2, 1, 4, 4)
    with pytest.raises(ValueError):
        V.decode_apng(data[:40] + bytes([data[40] ^ 1]) + data[41:])
    bt = V.benchmark_transforms({"flip": lambda t: t.flip(-1), "half": lambda t: t[:, ::2, ::2]}, torch.rand(3, 64, 64), iterations=3)
    assert bt["half"]["output_shape"] == (3, 32, 32) and bt["flip"]["images_per_s"] > 0


def test_quantization_adaptive_patterns_fused_blocks_engine_codec_autoconfig_and_annealing():
    from torsh_b200 import quantization_adaptive as A
    torch.manual_seed(0)
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c1, self.b1, self.r1 = torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.BatchNorm2d(8), torch.nn.ReLU()
            self.c2, self.b2 = torch.nn.Conv2d(8, 8, 3, padding=1), torch.nn.BatchNorm2d(8)
            self.r2, self.pool, self.fc, self.act, self.out = torch.nn.ReLU(), torch.nn.AdaptiveAvgPool2d(1), torch.nn.Linear(8, 16), torch.nn.GELU(), torch.nn.Linear(16, 4)
        def forward(self, x):
            h = self.r1(self.b1(self.c1(x)))
            h = self.r2(self.b2(self.c2(h)) + h)
            return self.out(self.act(self.fc(torch.flatten(self.pool(h), 1))))
    net = Net().eval()
    with torch.no_grad():
        for bn in (net.b1, net.b2):
            bn.running_mean.normal_(0, 0.2); bn.running_var.uniform_(0.5, 1.5); bn.weight.uniform_(0.5, 1.5); bn.bias.normal_(0, 0.2)
    gm = torch.fx.symbolic_trace(net)
    pm = A.PatternMatcher()
    found = {m["pattern"]: m["nodes"] for m in pm.match(gm)}
    assert found == {"conv_bn_relu": ["c1", "b1", "r1"], "conv_bn": ["c2", "b2"], "add_relu": ["add", "r2"], "linear_relu": ["fc", "act"], "linear": ["out"]}
    cov = pm.coverage(gm)
    assert cov["unmatched"] == ["pool", "flatten"] and cov["fraction"] == pytest.approx(10 / 12)
    only_wide = A.PatternMatcher([A.GraphPattern("wide_linear", ("Linear",), constraints=[lambda chain, mods: mods[chain[0].target].out_features >= 16])])
    assert [m["nodes"] for m in only_wide.match(gm)] == [["fc"]]
    # rewriting: fused int8 blocks stay close to the float model
    x = torch.randn(4, 3, 12, 12)
    qgm, done = A.fuse_and_quantize(net)
    assert {d["pattern"] for d in done} == {"conv_bn_relu", "conv_bn", "linear_relu", "linear"} and not any(isinstance(m, torch.nn.BatchNorm2d) for m in qgm.modules()) and sum(isinstance(m, A.FusedQuantBlock) for m in qgm.modules()) == 4
    ref, got = net(x).detach(), qgm(x).detach()
    assert float((got - ref).norm() / ref.norm()) < 0.05 and qgm.fused_c1.qweight.dtype == torch.int8 and qgm.fused_c1.act is not None and qgm.fused_c2.act is None
    q4, _ = A.fuse_and_quantize(net, bits=4)
    assert float((q4(x).detach() - ref).norm() / ref.norm()) > float((got - ref).norm() / ref.norm())
    # run-time engine
    feats = A.tensor_features(torch.tensor([0.0, 0.0, 1.0, -1.0, 8.0]))
    assert feats["sparsity"] == pytest.approx(0.4) and feats["abs_max"] == 8.0 and feats["numel"] == 5 and feats["dynamic_range_db"] == pytest.approx(20 * math.log10(8))
    eng = A.AdaptiveQuantizationEngine(A.AdaptiveQuantConfig(candidate_bits=(4, 6, 8), min_sqnr_db=28.0, target_mean_bits=8.0))
    g = torch.Generator().manual_seed(0)
    r = eng.quantize(torch.randn(4096, generator=g))
    assert r["bits"] in (6, 8) and r["sqnr_db"] > 25 and abs(r["sqnr_db"] - r["predicted_db"]) < 6 and r["q"].dtype == torch.int8
    lax = A.AdaptiveQuantizationEngine(A.AdaptiveQuantConfig(min_sqnr_db=12.0, target_mean_bits=4.0))
    assert lax.quantize(torch.randn(4096, generator=g))["bits"] == 4
    heavy = torch.randn(4096, generator=g); heavy[::512] *= 40
    clipped, plain = A.AdaptiveQuantizationEngine(A.AdaptiveQuantConfig(candidate_bits=(8,))), A.AdaptiveQuantizationEngine(A.AdaptiveQuantConfig(candidate_bits=(8,), clip_outliers=False))
    core = heavy.abs() < 4
    e_clip, e_plain = (clipped.quantize(heavy)["dequantized"] - heavy)[core].pow(2).mean(), (plain.quantize(heavy)["dequantized"] - heavy)[core].pow(2).mean()
    assert e_clip < e_plain / 4
    ctl = A.AdaptiveQuantizationEngine(A.AdaptiveQuantConfig(candidate_bits=(4, 6, 8), min_sqnr_db=45.0, target_mean_bits=5.0))
    for _ in range(60):
        ctl.quantize(torch.randn(2048, generator=g))
    s = ctl.summary()
    assert s["floor_db"] < 45.0 and s["mean_bits"] < 8.0 and len(s["bits_histogram"]) >= 2
    det = A.AdaptiveQuantizationEngine(A.AdaptiveQuantConfig(candidate_bits=(8,), degradation_window=10, degradation_drop_db=5.0))
    for i in range(40):
        t = torch.randn(2048, generator=g)
        if i >= 20:
            t[0] = 2000.0                                                             # an outlier the fixed 8 bits now have to cover
            det.cfg.clip_outliers = False
        det.quantize(t)
    assert det.summary()["alerts"] >= 1 and det.alerts[0]["drop_db"] > 5
    # learned codec
    weights = [torch.randn(64, 64, generator=g) * 0.1, torch.randn(32, 48, generator=g) * 0.1]
    codec = A.NeuralCodec(block=8, latent=4, codebook=256, hidden=32)
    hist = codec.fit(weights, steps=400, generator=g)
    c = codec.compress(weights[0])
    back = codec.decompress(c)
    rel = float((back - weights[0]).norm() / weights[0].norm())
    assert hist[-1] < hist[0] and back.shape == weights[0].shape and c["ratio"] == 32.0 and c["payload_bits"] == 8 * 512 and rel < 0.85
    structured = [torch.outer(torch.randn(64, generator=g), torch.ones(64)) * 0.1]
    codec2 = A.NeuralCodec(block=8, latent=2, codebook=64, hidden=32)
    codec2.fit(structured, steps=400, generator=g)
    assert float((codec2.decompress(codec2.compress(structured[0])) - structured[0]).norm() / structured[0].norm()) < 0.2
    odd = torch.randn(5, 7, generator=g) * 0.1
    assert codec.decompress(codec.compress(odd)).shape == (5, 7) and codec.compress(odd)["pad"] == 5
    # automatic configuration
    model = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 128), torch.nn.ReLU(), torch.nn.Linear(128, 10))
    auto = A.AutoConfigurator(A.HardwareConstraints(supported_bits=(4, 8, 16), max_error_db=30.0))
    cfg = auto.configure(model)
    assert set(cfg["bits"].values()) == {8} and cfg["fits"] and cfg["min_sqnr_db"] >= 30 and cfg["estimated_speedup"] == pytest.approx(2.0) and cfg["table"]["0.weight"][4]["sqnr_db"] < 30 < cfg["table"]["0.weight"][8]["sqnr_db"] < cfg["table"]["0.weight"][16]["sqnr_db"]
    tight = A.AutoConfigurator(A.HardwareConstraints(memory_bytes=0.7 * cfg["bytes"], supported_bits=(4, 8, 16), max_error_db=30.0)).configure(model)
    assert tight["fits"] and 4 in tight["bits"].values() and tight["relaxed_layers"] and tight["bytes"] <= 0.7 * cfg["bytes"] and tight["estimated_speedup"] > 2.0
    assert not A.AutoConfigurator(A.HardwareConstraints(memory_bytes=100.0, supported_bits=(4, 8))).configure(model)["fits"]
    front = auto.pareto_front(model)
    assert [c["name"] for c in front][0] == "uniform-4" and front[-1]["name"] == "uniform-16" and all(a["bytes"] < b["bytes"] and a["min_sqnr_db"] < b["min_sqnr_db"] for a, b in zip(front, front[1:]))
    # annealing: sensitive layers get more bits, the budget holds, and the result beats a uniform split
    sizes, sens = [1000, 1000, 1000, 1000], [100.0, 1.0, 0.01, 10.0]
    res = A.anneal_bit_allocation(sizes, sens, budget_bits=4 * 1000 * 4.5, choices=(2, 4, 8))
    uniform4 = sum(s * 4.0 ** -4 for s in sens)
    assert res["feasible"] and res["bits"][0] == 8 and res["bits"][2] == 2 and res["cost"] < uniform4 and res["used_bits"] <= 18000
    assert A.anneal_bit_allocation(sizes, sens, budget_bits=8000, choices=(2, 4, 8), schedule="linear")["bits"] == [2, 2, 2, 2] and A.anneal_bit_allocation(sizes, sens, budget_bits=1e9, schedule="logarithmic", steps=6000)["bits"] == [8, 8, 8, 8]


def test_fx_deploy_torchscript_custom_ops_types_cloud_manifests_accelerators_spiking_and_quantum_layer():
    import yaml
    from torsh_b200 import fx_deploy as D
    torch.manual_seed(0)
    # TorchScript round trip
    net = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.ReLU(), torch.nn.Linear(8, 3))
    gm = torch.fx.symbolic_trace(net)
    x = torch.randn(4, 6)
    sm = D.to_torchscript(gm, [x])
    desc = D.describe_torchscript(sm)
    assert torch.allclose(sm(x), net(x)) and desc["operators"]["aten::linear"] == 2 and desc["operators"]["aten::relu"] == 1 and len(desc["inputs"]) == 1
    back = D.from_torchscript(sm, [x])
    assert torch.allclose(back(x), net(x)) and [n.op for n in back.graph.nodes] == ["placeholder", "call_module", "output"]
    # custom operations
    reg = D.CustomOperationRegistry()
    swish2 = reg.register("swish2", lambda t: t * torch.sigmoid(2 * t), infer_shape=lambda s: s, cost=lambda s: 4.0 * math.prod(s), doc="x sigmoid(2x)")
    clipped = reg.register("clipped_identity", lambda t: t.clamp(-1, 1), backward=lambda g, t: g)       # straight-through gradient
    with pytest.raises(ValueError):
        reg.register("swish2", lambda t: t)
    def fn(a): return clipped(swish2(a) + 1.0)
    cg = torch.fx.symbolic_trace(fn)
    assert reg.nodes_in(cg) == ["swish2", "clipped_identity"] and torch.allclose(cg(x), (x * torch.sigmoid(2 * x) + 1).clamp(-1, 1))
    assert reg.infer_shapes(cg, [(4, 6)])["clipped_identity"] == (4, 6) and reg.total_cost(cg, [(4, 6)]) == 96.0
    xr = (torch.randn(5) * 3).requires_grad_(True)
    clipped(xr).sum().backward()
    assert torch.equal(xr.grad, torch.ones(5))
    reg.unregister("swish2")
    assert "swish2" not in reg.ops
    # custom types
    types = D.CustomTypeRegistry().with_defaults()
    t = torch.randn(1000)
    assert types.roundtrip_error("fixed<16,8>", t) < types.roundtrip_error("fixed<8,4>", t) < 0.05 and types.roundtrip_error("log8", t) < 0.05 and types.roundtrip_error("bfp16x8", t) < 0.02 and types.types["bfp16x8"].bits == 8.5
    assert types.types["fixed<8,4>"].validate(types.types["fixed<8,4>"].pack(t * 100)) and float(types.types["fixed<8,4>"].unpack(types.types["fixed<8,4>"].pack(torch.tensor([100.0])))) == pytest.approx(127 / 16)
    ann = {"_0": ("float32", "fixed<8,4>"), "_1": ("fixed<8,4>", "fixed<8,4>"), "_2": ("float32", "float32")}
    issues = types.check_graph(gm, ann)
    assert issues == [{"edge": ("_1", "_2"), "producer": "fixed<8,4>", "consumer": "float32"}]
    types.register_conversion("fixed<8,4>", "float32", types.types["fixed<8,4>"].unpack)
    assert types.check_graph(gm, ann) == []
    # cloud deployment
    spec = D.ServingSpec("llm", "registry.local/llm:1", "/models/llm.safetensors", gpus_per_replica=2, max_batch=16, max_replicas=12)
    docs = list(yaml.safe_load_all(D.kubernetes_manifests(spec)))
    assert [d["kind"] for d in docs] == ["Deployment", "Service", "HorizontalPodAutoscaler"] and docs[0]["spec"]["template"]["spec"]["containers"][0]["resources"]["limits"]["nvidia.com/gpu"] == 2 and docs[2]["spec"]["maxReplicas"] == 12 and docs[1]["spec"]["ports"][0]["targetPort"] == 8080
    df = D.dockerfile(spec, extra_packages=["einops"])
    assert df.startswith("FROM nvcr.io") and "pip install --no-cache-dir einops" in df and "EXPOSE 8080" in df and "HEALTHCHECK" in df
    plan = D.plan_capacity(400.0, {1: 12.0, 4: 20.0, 8: 30.0, 16: 60.0, 32: 110.0}, slo_ms=50.0, spec=spec)
    assert plan["batch"] == 8 and plan["replica_qps"] == pytest.approx(8 / 0.03) and plan["replicas"] == 2 and plan["instances"] == 1 and plan["feasible"] and plan["monthly_cost"] == pytest.approx(98.0 * 730) and 0.7 < plan["utilisation"] < 0.8
    assert not D.plan_capacity(10.0, {1: 80.0}, slo_ms=50.0, spec=spec)["feasible"] and not D.plan_capacity(50000.0, {8: 30.0}, slo_ms=50.0, spec=spec)["feasible"]
    # accelerators
    cnn = torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.Flatten(), torch.nn.Linear(8 * 8 * 8, 10)).eval()
    cgm = torch.fx.symbolic_trace(cnn)
    img = torch.randn(2, 3, 8, 8)
    mp = D.map_to_accelerator(cgm, img, D.ACCELERATORS["analog_in_memory"])
    assert mp["on_accelerator"] == ["_0", "_3"] and mp["on_host"] == ["_1", "_2"] and mp["macs_on"] == 2 * 8 * 64 * 27 + 2 * 10 * 512 and mp["boundary_bytes"] == 2 * 512 * 2 and mp["energy_saving"] > 0.8
    npu = D.map_to_accelerator(cgm, img, D.ACCELERATORS["digital_npu"])
    assert "_1" in npu["on_accelerator"] and npu["boundary_bytes"] < mp["boundary_bytes"] + 1 and D.map_to_accelerator(cgm, img, D.ACCELERATORS["photonic"])["on_accelerator"] == ["_3"]
    g = torch.Generator().manual_seed(0)
    clean = D.evaluate_with_device_noise(cnn, img, D.AcceleratorModel("ideal", ("Linear", "Conv2d"), 16, 16, 0.0), trials=2, generator=g)
    noisy = D.evaluate_with_device_noise(cnn, img, D.ACCELERATORS["analog_in_memory"], trials=4, generator=g)
    assert clean["mean_deviation"] < 1e-3 < noisy["mean_deviation"] < 0.5 and noisy["worst_deviation"] >= noisy["mean_deviation"] and clean["argmax_agreement"] == 1.0
    # spiking conversion approaches the rectifier network as the number of steps grows
    mlp = torch.nn.Sequential(torch.nn.Linear(10, 32), torch.nn.ReLU(), torch.nn.Linear(32, 32), torch.nn.ReLU(), torch.nn.Linear(32, 5)).eval()
    data = torch.rand(64, 10)
    snn = D.SpikingNetwork(mlp, data, percentile=99.9)
    with torch.no_grad():
        ref = mlp(data)
        o16, s16 = snn(data, steps=16)
        o256, s256 = snn(data, steps=256)
    e16, e256 = float((o16 - ref).norm() / ref.norm()), float((o256 - ref).norm() / ref.norm())
    assert e256 < 0.05 < e16 and e256 < e16 / 3 and float((o256.argmax(1) == ref.argmax(1)).float().mean()) > 0.9 and 0 < s256["spikes_per_neuron_per_step"] < 1 and s256["neurons"] == 64 and len(snn.scales) == 2
    en = D.snn_energy_estimate(s16, synaptic_ops_per_spike=32, ann_macs=64 * (10 * 32 + 32 * 32 + 32 * 5))
    assert en["snn_energy_pj"] > 0 and en["ratio"] == pytest.approx(en["snn_energy_pj"] / en["ann_energy_pj"])
    # variational quantum layer: probabilities stay normalised, gradients flow, a small regression is learnable
    vq = D.VariationalQuantumLayer(n_qubits=3, depth=2)
    inp = torch.rand(16, 3) * math.pi
    out = vq(inp)
    assert out.shape == (16, 3) and float(out.detach().abs().max()) <= 1.0 + 1e-5 and vq.circuit_summary() == {"qubits": 3, "depth": 2, "parameters": 12, "two_qubit_gates": 6, "single_qubit_gates": 15}
    with torch.no_grad():
        vq0 = D.VariationalQuantumLayer(2, 1); vq0.theta.zero_()
        z = vq0(torch.tensor([[0.0, 0.0], [math.pi, 0.0], [math.pi / 2, math.pi]]))
    assert torch.allclose(z, torch.tensor([[1.0, 1.0], [1.0, -1.0], [-1.0, 0.0]]), atol=1e-5)     # CNOT ring: (q0 -> q1) then (q1 -> q0)
    th = vq.theta.detach().clone().requires_grad_(True)
    def f(theta):
        vq.theta.data = theta.data
        return vq(inp).sum()
    loss = vq(inp).sum(); loss.backward()
    shift = torch.zeros_like(vq.theta); shift[0, 1, 0] = math.pi / 2
    with torch.no_grad():
        base = vq.theta.detach().clone()
        vq.theta.copy_(base + shift); plus = vq(inp).sum()
        vq.theta.copy_(base - shift); minus = vq(inp).sum()
        vq.theta.copy_(base)
    assert float(vq.theta.grad[0, 1, 0]) == pytest.approx(float((plus - minus) / 2), abs=1e-4)
    target = torch.cos(inp[:, :1])
    model = torch.nn.Sequential(D.VariationalQuantumLayer(2, 2), torch.nn.Linear(2, 1))
    opt = torch.optim.Adam(model.parameters(), lr=0.1)
    first = None
    for _ in range(150):
        l = torch.nn.functional.mse_loss(model(inp[:, :2]), target)
        first = first if first is not None else float(l.detach())
        opt.zero_grad(); l.backward(); opt.step()
    assert float(l.detach()) < 0.05 * first
    with pytest.raises(ValueError):
        D.VariationalQuantumLayer(13)


def test_graph_learning_continuous_time_lottery_tickets_and_pretraining():
    from torsh_b200 import graph_learning as G
    from torsh_b200.graph import GCN, stochastic_block_model
    torch.manual_seed(0)
    # time encoding: inner products depend on the time difference only (zero phases)
    te = G.TimeEncoder(32)
    t = torch.tensor([0.0, 5.0, 100.0, 105.0])
    e = te(t)
    e = e.detach()
    assert e.shape == (4, 32) and float(e[0] @ e[0]) == pytest.approx(32.0) and float((e[0] * e[1]).sum() - (e[2] * e[3]).sum()) != 0 and float(e.abs().max()) <= 1.0
    w = te.w.detach()
    assert float((torch.cos(5.0 * w)).sum()) == pytest.approx(float(((torch.cos(100 * w) * torch.cos(105 * w)) + (torch.sin(100 * w) * torch.sin(105 * w))).sum()), rel=1e-4)
    store = G.TemporalNeighborStore(k=2)
    store.insert(0, 1, 1.0, 0); store.insert(0, 2, 2.0, 1); store.insert(0, 3, 3.0, 2)
    assert [u for u, _, _ in store.recent(0, 10.0)] == [2, 3] and store.recent(0, 2.5) == [(2, 2.0, 1)] and store.recent(3, 3.0) == []
    att = G.TemporalAttentionLayer(8, 4, 8, 16)
    hs, hn, en, dt = torch.randn(3, 8), torch.randn(3, 5, 8), torch.randn(3, 5, 4), torch.rand(3, 5)
    mask = torch.tensor([[True] * 5, [True, True, False, False, False], [False] * 5])
    out = att(hs, hn, en, dt, mask)
    hn2 = hn.clone(); hn2[1, 3] += 10                                               # a masked neighbour does not matter
    assert out.shape == (3, 16) and torch.allclose(att(hs, hn2, en, dt, mask), out, atol=1e-6) and torch.isfinite(out).all()
    # event stream with a repeating pattern: node i talks to node (i + 1) mod n; the model learns to rank the true partner
    n = 8
    g = torch.Generator().manual_seed(0)
    def stream(T):
        src = torch.randint(0, n, (T,), generator=g)
        return src, (src + 1) % n, torch.arange(T, dtype=torch.float32), torch.ones(T, 2)
    model = G.ContinuousTimeGraphNetwork(n, edge_dim=2, memory_dim=16, time_dim=8, embed_dim=16, neighbors=5)
    opt = torch.optim.Adam(model.parameters(), lr=5e-3)
    def run(train: bool, T=200, batch=20):
        model.reset_state()
        src, dst, tt, ef = stream(T)
        correct = total = 0
        for s in range(0, T, batch):
            sl = slice(s, s + batch)
            neg = (dst[sl] + torch.randint(1, n - 1, (len(src[sl]),), generator=g)) % n
            pos_s, neg_s = model.score(src[sl], dst[sl], tt[sl]), model.score(src[sl], neg, tt[sl])
            if train:
                loss = torch.nn.functional.binary_cross_entropy_with_logits(pos_s, torch.ones_like(pos_s)) + torch.nn.functional.binary_cross_entropy_with_logits(neg_s, torch.zeros_like(neg_s))
                opt.zero_grad(); loss.backward(); opt.step()
            if s >= T // 2:
                correct += int((pos_s > neg_s).sum()); total += len(pos_s)
            with torch.no_grad() if not train else torch.enable_grad():
                model.update(src[sl], dst[sl], tt[sl], ef[sl])
            model.detach_state()
        return correct / total
    before = run(False)
    for _ in range(6):
        run(True)
    after = run(False)
    assert after > 0.85 and after > before + 0.2 and model.memory.abs().sum() > 0 and len(model.edge_feats) == 200
    # graph ODE: heat diffusion matches the matrix exponential, conserves the degree-weighted mean, and smooths
    ei = torch.tensor([[0, 1, 2, 3, 4, 0], [1, 2, 3, 4, 5, 5]])
    h0 = torch.randn(6, 3, dtype=torch.float64)
    ode = G.GraphODE(mode="heat", steps=40)
    L = G.GraphODE.laplacian(ei, 6).double()
    assert torch.allclose(ode(h0, ei, t=1.5), torch.linalg.matrix_exp(-1.5 * L) @ h0, atol=1e-6)
    rough = lambda h: float((h.T @ L @ h).trace())
    assert rough(ode(h0, ei, 3.0)) < 0.2 * rough(h0) and torch.allclose(ode(h0, ei, 0.0), h0)
    learned = G.GraphODE(dim=3, mode="gcn", steps=8)
    y = learned(h0.float(), ei, t=1.0)
    y.sum().backward()
    assert y.shape == (6, 3) and learned.conv.lin.weight.grad.abs().sum() > 0 and learned.gate.grad is not None
    # lottery ticket on a two-block graph
    data = stochastic_block_model(sizes=(30, 30), p_in=0.3, p_out=0.02, feat=8, seed=1)
    net = GCN(8, 16, 2)
    lt = G.GraphLotteryTicket(net, data.edge_index, weight_rate=0.3, edge_rate=0.1)
    init = {k: v.clone() for k, v in net.state_dict().items()}
    def train(model, edges, reapply):
        opt = torch.optim.Adam(model.parameters(), lr=0.05)
        for _ in range(60):
            loss = torch.nn.functional.cross_entropy(model(data.x, edges), data.y)
            opt.zero_grad(); loss.backward(); opt.step(); reapply()
        return float((model(data.x, edges).argmax(1) == data.y).float().mean())
    def importance(model, edges):
        with torch.no_grad():
            z = model(data.x, edges)
        return (z[edges[0]] * z[edges[1]]).sum(1)                                   # edges inside a block agree, edges across disagree
    recs = [lt.round(train, importance) for _ in range(4)]
    assert recs[-1]["weight_sparsity"] == pytest.approx(1 - 0.7 ** 4, abs=0.02) and recs[-1]["edge_sparsity"] == pytest.approx(1 - 0.9 ** 4, abs=0.02) and recs[-1]["score"] > 0.9 and recs[0]["score"] > 0.9
    for name, p in net.named_parameters():
        if name in lt.masks:
            assert torch.equal(p.detach(), init[name] * lt.masks[name]) and float((p == 0).float().mean()) >= recs[-1]["weight_sparsity"] - 0.3
    cross = (data.y[data.edge_index[0]] != data.y[data.edge_index[1]])
    assert float(cross[lt.edge_mask].float().mean()) < float(cross.float().mean()) and lt.masked_edges().shape[1] == int(lt.edge_mask.sum())
    # augmentations
    x, edges = data.x, data.edge_index
    gen = torch.Generator().manual_seed(0)
    xd, ed = G.augment_graph(x, edges, "node_drop", 0.3, gen)
    assert 30 <= xd.shape[0] <= 52 and int(ed.max()) < xd.shape[0] and ed.shape[1] < edges.shape[1]
    xp, ep = G.augment_graph(x, edges, "edge_perturb", 0.2, gen)
    assert ep.shape == edges.shape and not torch.equal(ep, edges) and torch.equal(xp, x)
    xm, em = G.augment_graph(x, edges, "feature_mask", 0.5, gen)
    assert torch.equal(em, edges) and 1 <= int((xm.abs().sum(0) == 0).sum()) <= 7
    xs, es = G.augment_graph(x, edges, "subgraph", 0.5, gen)
    assert xs.shape[0] == 30 and int(es.max()) < 30
    with pytest.raises(ValueError):
        G.augment_graph(x, edges, "rotate")
    z = torch.randn(6, 4)
    assert float(G.nt_xent(z, z + 0.01 * torch.randn(6, 4), 0.1)) < float(G.nt_xent(z, torch.randn(6, 4), 0.1))
    # pre-training, then prompt tuning on the frozen encoder
    enc = G.GraphEncoder(8, 16)
    graphs = [(stochastic_block_model((15, 15), 0.4, 0.02, 8, seed=s).x, stochastic_block_model((15, 15), 0.4, 0.02, 8, seed=s).edge_index) for s in range(4)]
    hist = G.pretrain_contrastive(enc, graphs, steps=30, generator=gen)
    assert sum(hist[-5:]) / 5 < sum(hist[:5]) / 5
    smooth_x = torch.cat([torch.randn(1, 8).expand(30, 8), torch.randn(1, 8).expand(30, 8)]) + 0.05 * torch.randn(60, 8)
    mh = G.pretrain_masked_features(enc, smooth_x, data.edge_index, steps=150, generator=gen)
    assert sum(mh[-10:]) / 10 < 0.3 * sum(mh[:10]) / 10
    frozen = {k: v.clone() for k, v in enc.state_dict().items()}
    pt = G.GraphPromptTuning(enc, 8, 2)
    assert pt.trainable_parameters() == 8 + 16 * 2 + 2
    opt = torch.optim.Adam([p for p in pt.parameters() if p.requires_grad], lr=0.05)
    for _ in range(100):
        loss = torch.nn.functional.cross_entropy(pt(data.x, data.edge_index), data.y)
        opt.zero_grad(); loss.backward(); opt.step()
    assert float((pt(data.x, data.edge_index).argmax(1) == data.y).float().mean()) > 0.9 and all(torch.equal(frozen[k], v) for k, v in enc.state_dict().items()) and pt.prompt.abs().sum() > 0


def test_sparse_tools_kernels_profiler_memory_analysis_format_choice_and_locality():
    import json
    from torsh_b200 import sparse_tools as T
    from torsh_b200.sparse import CooTensor
    torch.manual_seed(0)
    dense = torch.randn(40, 30) * (torch.rand(40, 30) < 0.15)
    dense[7] = 0                                                                     # an empty row
    csr = CooTensor.from_dense(dense).to_csr()
    crow, col, val = csr.indptr, csr.indices, csr.values
    B = torch.randn(30, 6)
    # kernels against dense algebra
    assert torch.allclose(T.csr_spmm(crow, col, val, B), dense @ B, atol=1e-5) and torch.allclose(T.csr_spmm_blocked(crow, col, val, B, row_block=7), dense @ B, atol=1e-5) and torch.allclose(T.csr_spmm(crow, col, val, B[:, 0]), dense @ B[:, 0], atol=1e-5)
    Q, K = torch.randn(40, 8), torch.randn(30, 8)
    mask = dense != 0
    assert torch.allclose(T.sddmm(crow, col, Q, K), (Q @ K.T)[mask], atol=1e-5) and torch.allclose(T.sddmm(crow, col, Q, K, val), (Q @ K.T * dense)[mask], atol=1e-5)
    sm = T.csr_row_softmax(crow, val)
    ref = torch.where(mask, dense, torch.full_like(dense, -float("inf"))).softmax(1)
    assert torch.allclose(sm, ref[mask], atol=1e-6) and torch.allclose(T.csr_row_reduce(crow, sm), mask.any(1).float(), atol=1e-6)
    assert torch.allclose(T.csr_row_reduce(crow, val, "norm2"), dense.norm(dim=1), atol=1e-5) and torch.allclose(T.csr_row_reduce(crow, val, "max")[mask.any(1)], torch.where(mask, dense, torch.full_like(dense, -1e9)).max(1).values[mask.any(1)]) and T.csr_row_reduce(crow, val, "max")[7] == -float("inf")
    out, keep = T.apply_with_threshold(val, torch.tanh, 0.5)
    assert torch.equal(out, torch.tanh(val)) and torch.equal(keep, torch.tanh(val).abs() > 0.5)
    V = torch.randn(30, 5)
    scores = (Q @ K.T / 8 ** 0.5).masked_fill(~mask, -float("inf"))
    att_ref = torch.nan_to_num(scores.softmax(1), nan=0.0) @ V
    assert torch.allclose(T.sparse_attention(crow, col, Q, K, V), att_ref, atol=1e-5)
    # profiler with a fake clock
    now = [0.0]
    prof = T.SparseProfiler(clock=lambda: now[0])
    def work(cost): now[0] += cost; return cost
    for i in range(10):
        prof.track("spmm_csr", work, 0.010, nnz=1000)
        prof.track("spmm_coo", work, 0.020 + 0.002 * i, nnz=1000)
    s = prof.statistics("spmm_csr")
    assert s["count"] == 10 and s["mean"] == pytest.approx(0.010) and s["consistent"] and s["nnz_per_second"] == pytest.approx(1e5) and prof.statistics("none") == {"count": 0}
    assert prof.trend("spmm_coo")["direction"] == "degrading" and prof.trend("spmm_csr")["direction"] == "stable" and prof.fastest() == "spmm_csr" and prof.top_by_throughput(1) == ["spmm_csr"]
    base = T.SparseProfiler()
    for i in range(5):
        base.add(T.Measurement("spmm_coo", 0.015, 1000, step=i)); base.add(T.Measurement("spmm_csr", 0.010, 1000, step=i))
    reg = prof.detect_regressions(base)
    assert [r["operation"] for r in reg] == ["spmm_coo"] and reg[0]["slowdown"] == pytest.approx(0.029 / 0.015)
    assert prof.to_csv().splitlines()[0] == "operation,step,seconds,nnz,bytes" and len(prof.to_csv().splitlines()) == 21 and json.loads(prof.to_json())["summary"]["spmm_csr"]["count"] == 10 and "degrading" in prof.report() and prof.report().count("\n") == 2
    # memory per format
    assert T.format_bytes((100, 100), 500, "csr") == 500 * 12 + 101 * 8 and T.format_bytes((100, 100), 500, "coo") == 500 * 20 and T.format_bytes((100, 100), 500, "dense") == 40000 and T.format_bytes((100, 100), 500, "ell", max_row_nnz=9) == 100 * 9 * 12
    tri = torch.diag(torch.ones(64)) * 2 + torch.diag(torch.ones(63), 1) + torch.diag(torch.ones(63), -1)
    mt = T.analyze_memory(tri)
    assert mt["most_compact"] == "dia" and mt["profile"]["diagonals"] == 3 and mt["profile"]["bandwidth"] == 1 and mt["compression_vs_dense"] > 15 and any("DIA" in r for r in mt["recommendations"])
    blocky = torch.kron((torch.rand(16, 16) < 0.1).float(), torch.ones(4, 4)) * torch.randn(64, 64)
    mb = T.analyze_memory(blocky)
    assert mb["most_compact"] == "bsr" and mb["profile"]["block_fill"] > 0.95 and any("BSR" in r for r in mb["recommendations"])
    skew = torch.zeros(64, 64); skew[0] = 1.0; skew[torch.arange(1, 64), torch.arange(1, 64)] = 1.0
    ms = T.analyze_memory(skew)
    assert ms["bytes"]["ell"] > 2 * ms["bytes"]["csr"] and any("ELL" in r for r in ms["recommendations"]) and ms["profile"]["max_row_nnz"] == 64
    assert any("too dense" in r for r in T.analyze_memory(torch.randn(16, 16))["recommendations"])
    # format choice
    assert T.suggest_format(T.structure_profile(tri))["format"] == "dia" and T.suggest_format(T.structure_profile(blocky))["format"] == "bsr" and T.suggest_format(T.structure_profile(torch.randn(8, 8)))["format"] == "dense"
    assert T.suggest_format(T.structure_profile(skew))["format"] == "csr" and T.suggest_format(T.structure_profile(skew), "build")["format"] == "coo" and T.suggest_format(T.structure_profile(skew), "transpose_matmul")["format"] == "csc"
    regular = torch.zeros(64, 64)
    for r in range(64):
        regular[r, [(r * 7 + k * 13) % 64 for k in range(4)]] = 1.0
    assert T.suggest_format(T.structure_profile(regular))["format"] == "ell"
    cmp = T.compare_formats(dense[:, :28], torch.randn(28, 4), repeats=2)
    assert set(cmp["results"]) == {"dense", "coo", "csr", "ell", "bsr"} and all(v["max_error"] < 1e-4 for v in cmp["results"].values()) and cmp["fastest"] == cmp["ranking"][0]
    tuner = T.FormatAutoTuner()
    assert tuner.choose(tri) == "dia" and tuner.trials == 0
    first = tuner.choose(regular, torch.randn(64, 4), measure=True)
    assert tuner.trials == 1 and tuner.choose(regular.roll(1, 0)) == first and tuner.trials == 1
    tuner.learn(T.structure_profile(skew), "coo")
    assert tuner.choose(skew) == "coo"
    # locality
    acc = T.benchmark_access_patterns(n=1 << 16, repeats=2, generator=torch.Generator().manual_seed(0))
    assert acc["sequential"]["gb_per_s"] > 0 and acc["random_penalty"] > 0
    band = CooTensor.from_dense(tri).to_csr()
    scat = CooTensor.from_dense(regular).to_csr()
    lb, ls = T.column_locality(band.indptr, band.indices), T.column_locality(scat.indptr, scat.indices)
    assert lb["same_line_fraction"] == 1.0 and lb["mean_gap"] == 1.0 and ls["mean_gap"] > 10 and ls["same_line_fraction"] < lb["same_line_fraction"]


def test_dynamic_linear_model_filter_smoother_forecast_and_likelihood_fit():
    from torsh_b200.series_ext import DynamicLinearModel
    g = torch.Generator().manual_seed(0)
    # local level: with a huge signal-to-noise ratio the filter follows the data, with a tiny one it averages
    y = torch.cumsum(torch.randn(200, generator=g, dtype=torch.float64) * 0.5, 0) + torch.randn(200, generator=g, dtype=torch.float64)
    follow = DynamicLinearModel(1, obs_var=1e-6, level_var=1.0).filter(y)
    flat = DynamicLinearModel(1, obs_var=1.0, level_var=1e-10).filter(y)
    assert torch.allclose(follow["m"][:, 0], y, atol=1e-3) and float(flat["m"][-1, 0]) == pytest.approx(float(y.mean()), abs=1e-3)
    # steady-state gain of the local level model: K = (-r + sqrt(r^2 + 4 r)) / 2 with r = W / V
    dlm = DynamicLinearModel(1, obs_var=1.0, level_var=0.25)
    f = dlm.filter(y)
    r = 0.25
    gain = (-r + math.sqrt(r * r + 4 * r)) / 2
    assert float(f["C"][-1, 0, 0]) == pytest.approx(gain * 1.0, rel=1e-6)
    sm = dlm.smooth(f)
    assert float(sm["cov"][100, 0, 0]) < float(f["C"][100, 0, 0]) and torch.allclose(sm["state"][-1], f["m"][-1]) and float((sm["level"].diff() ** 2).mean()) < float((f["m"][:, 0].diff() ** 2).mean())
    # the likelihood matches the sum of Gaussian one-step densities
    ll = sum(-0.5 * (math.log(2 * math.pi * float(q)) + float(yy - p) ** 2 / float(q)) for yy, p, q in zip(y, f["pred"], f["pred_var"]))
    assert float(f["loglik"]) == pytest.approx(ll, rel=1e-9)
    # missing observations are skipped and the uncertainty grows over the gap
    yg = y.clone(); yg[50:60] = float("nan")
    fg = dlm.filter(yg)
    assert float(fg["C"][59, 0, 0]) > 5 * float(fg["C"][49, 0, 0]) and torch.isfinite(fg["m"]).all()
    # trend + seasonality: components are recovered and the forecast continues both
    t = torch.arange(120, dtype=torch.float64)
    season = torch.tensor([3.0, -1.0, -2.0, 0.0], dtype=torch.float64).repeat(30)
    ys = 0.5 * t + season + 0.1 * torch.randn(120, generator=g, dtype=torch.float64)
    m2 = DynamicLinearModel(2, seasonal_period=4, obs_var=0.01, level_var=1e-6, slope_var=1e-8, seasonal_var=1e-8)
    f2 = m2.filter(ys); s2 = m2.smooth(f2)
    assert m2.n == 5 and float(s2["slope"][60]) == pytest.approx(0.5, abs=0.01) and torch.allclose(s2["seasonal"][40:44], season[40:44], atol=0.15) and torch.allclose(s2["level"][20:100], 0.5 * t[20:100], atol=0.2)
    fc = m2.forecast(f2, 8)
    truth = 0.5 * torch.arange(120, 128, dtype=torch.float64) + season[:8]
    assert torch.allclose(fc["mean"], truth, atol=0.3) and (fc["upper"] > fc["mean"]).all() and float(fc["std"][-1]) >= float(fc["std"][0])
    # regression component with a time-invariant coefficient
    X = torch.randn(150, 1, generator=g, dtype=torch.float64)
    yr = 2.0 + 3.0 * X[:, 0] + 0.1 * torch.randn(150, generator=g, dtype=torch.float64)
    m3 = DynamicLinearModel(1, regressors=1, obs_var=0.01, level_var=1e-8)
    f3 = m3.filter(yr, X)
    assert float(f3["m"][-1, 1]) == pytest.approx(3.0, abs=0.05) and float(f3["m"][-1, 0]) == pytest.approx(2.0, abs=0.05) and float(m3.forecast(f3, 1, torch.tensor([[2.0]]))["mean"][0]) == pytest.approx(8.0, abs=0.2)
    # maximum likelihood recovers the variances of a simulated local level model
    lvl = torch.cumsum(torch.randn(400, generator=g, dtype=torch.float64) * math.sqrt(0.3), 0)
    obs = lvl + torch.randn(400, generator=g, dtype=torch.float64) * math.sqrt(2.0)
    est = DynamicLinearModel(1, obs_var=1.0, level_var=1.0)
    start_nll = -float(est.filter(obs)["loglik"])
    res = est.fit(obs)
    assert res["variances"]["obs"] == pytest.approx(2.0, rel=0.35) and res["variances"]["level"] == pytest.approx(0.3, rel=0.6) and res["neg_loglik"] < start_nll and res["signal_to_noise"] == pytest.approx(0.15, rel=0.8)


def test_ensembles_voting_fitted_weights_stacking_bagging_snapshots_online_selection_and_model_file_ops(tmp_path):
    import numpy as np
    from torsh_b200.models import ensembles as E
    from torsh_b200.models.tooling import write_safetensors
    torch.manual_seed(0)
    # combining
    p = torch.tensor([[[0.9, 0.1], [0.4, 0.6]], [[0.6, 0.4], [0.45, 0.55]], [[0.2, 0.8], [0.9, 0.1]]])
    assert torch.allclose(E.combine_predictions(p, "soft"), p.mean(0)) and E.combine_predictions(p, "hard").tolist() == [[pytest.approx(2 / 3), pytest.approx(1 / 3)], [pytest.approx(1 / 3), pytest.approx(2 / 3)]]
    w = torch.tensor([0.0, 0.0, 1.0])
    assert torch.allclose(E.combine_predictions(p, "weighted", w), p[2]) and E.combine_predictions(p, "hard", torch.tensor([1.0, 1.0, 5.0])).argmax(1).tolist() == [1, 0] and torch.allclose(E.combine_predictions(p, "max"), torch.tensor([[0.9, 0.1], [0.9, 0.1]]))
    geo = E.combine_predictions(p, "geometric")
    assert torch.allclose(geo.sum(1), torch.ones(2)) and geo[0, 0] == pytest.approx((0.9 * 0.6 * 0.2) ** (1 / 3) / ((0.9 * 0.6 * 0.2) ** (1 / 3) + (0.1 * 0.4 * 0.8) ** (1 / 3)))
    # data: three informative views of a 3-class problem
    g = torch.Generator().manual_seed(0)
    n, k = 600, 3
    y = torch.randint(0, k, (n,), generator=g)
    centers = torch.randn(k, 6, generator=g) * 1.5
    x = centers[y] + torch.randn(n, 6, generator=g) * 1.6
    xtr, ytr, xva, yva = x[:400], y[:400], x[400:], y[400:]
    def fit(m, a, b, steps=150):
        opt = torch.optim.Adam(m.parameters(), lr=0.05)
        for _ in range(steps):
            opt.zero_grad(); torch.nn.functional.cross_entropy(m(a), b).backward(); opt.step()
    class View(torch.nn.Module):
        def __init__(self, cols): super().__init__(); self.cols, self.lin = cols, torch.nn.Linear(len(cols), k)
        def forward(self, t): return self.lin(t[:, self.cols])
    views = [[0, 1], [2, 3], [4, 5], [0]]
    base = []
    for c in views:
        m = View(c); fit(m, xtr, ytr); base.append(m.eval())
    with torch.no_grad():
        probs = torch.stack([m(xva).softmax(-1) for m in base])
    acc = lambda pr: float((pr.argmax(-1) == yva).float().mean())
    singles = [acc(q) for q in probs]
    assert acc(E.combine_predictions(probs, "soft")) > max(singles)
    wfit = E.fit_ensemble_weights(probs, yva)
    nll = lambda pr: float(torch.nn.functional.nll_loss(pr.clamp_min(1e-12).log(), yva))
    assert float(wfit.sum()) == pytest.approx(1.0, abs=1e-5) and wfit[3] < 0.1 and nll(E.combine_predictions(probs, "weighted", wfit)) <= nll(E.combine_predictions(probs, "soft")) + 1e-6
    # stacking beats every base model's out-of-fold accuracy
    st = E.StackingEnsemble([lambda c=c: View(c) for c in views[:3]], lambda m, a, b: fit(m, a, b, 80), folds=3).fit(xtr, ytr)
    assert acc(st.predict_proba(xva)) > max(st.oof_accuracy) and len(st.models) == 3 and st.predict_proba(xva).sum(1).allclose(torch.ones(200))
    # bagging
    models, oob = E.bagging(lambda: View([0, 1, 2, 3, 4, 5]), lambda m, a, b: fit(m, a, b, 60), xtr, ytr, n_models=4)
    oob_acc = E.out_of_bag_accuracy(models, oob, xtr, ytr)
    with torch.no_grad():
        bag_val = acc(torch.stack([m(xva).softmax(-1) for m in models]).mean(0))
    assert all(0.3 * 400 < len(o) < 0.45 * 400 for o in oob) and abs(oob_acc - bag_val) < 0.08 and bag_val > 0.6
    # snapshots
    snap = E.SnapshotEnsemble(View([0, 1, 2, 3, 4, 5]), cycles=3, steps_per_cycle=40, max_lr=0.2)
    hist = snap.fit(lambda m: torch.nn.functional.cross_entropy(m(xtr), ytr))
    assert len(snap.snapshots) == 3 and snap.lr_at(0) == 0.2 and snap.lr_at(39) < 0.01 and snap.lr_at(40) == 0.2 and hist[-1] < hist[0] and acc(snap.predict_proba(xva)) > 0.6 and snap.predict_proba(xva, last=1).shape == (200, 3)
    # online adaptive weights follow the better model, and a drift
    on = E.OnlineAdaptiveEnsemble(2, eta=0.5, forget=0.02)
    good, bad = torch.tensor([0.9, 0.1]), torch.tensor([0.3, 0.7])
    for _ in range(30):
        on.update(torch.stack([good, bad]), 0)
    assert on.w[0] > 0.9 and on.predict(torch.stack([good, bad]))[0] > 0.8
    for _ in range(60):
        on.update(torch.stack([good, bad]), 1)
    assert on.w[1] > 0.9 and on.cum_loss[0] > 0
    # diversity
    t = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1])
    same = torch.stack([torch.tensor([0, 0, 0, 1, 1, 1, 1, 0])] * 2)
    comp = torch.stack([torch.tensor([0, 0, 0, 1, 1, 1, 1, 0]), torch.tensor([1, 0, 0, 0, 0, 1, 1, 1])])
    ds, dc = E.diversity_measures(same, t), E.diversity_measures(comp, t)
    assert ds["disagreement"] == 0 and ds["q_statistic"] == 1.0 and ds["correlation"] == pytest.approx(1.0) and dc["disagreement"] == 0.5 and dc["q_statistic"] == -1.0 and dc["double_fault"] == 0.0 and ds["double_fault"] == 0.25
    # greedy selection
    sel = E.greedy_ensemble_selection(probs, yva)
    assert sel["validation_loss"] <= sel["best_single_loss"] and sel["improvement"] > 0 and sel["weights"].sum() == pytest.approx(1.0) and sel["trace"] == sorted(sel["trace"], reverse=True) and sel["members"][0] == int(torch.tensor([nll(q) for q in probs]).argmin())
    assert len(E.greedy_ensemble_selection(probs, yva, max_size=2, with_replacement=False)["members"]) <= 2
    assert E.estimate_ensemble_gain(0.7, 0.0, 11) == pytest.approx(sum(math.comb(11, j) * 0.7 ** j * 0.3 ** (11 - j) for j in range(6, 12))) and E.estimate_ensemble_gain(0.7, 1.0, 11) == pytest.approx(0.7) and E.estimate_ensemble_gain(0.7, 0.0, 11) > E.estimate_ensemble_gain(0.7, 0.5, 11)
    assert E.optimal_ensemble_size(0.7, 0.0) > E.optimal_ensemble_size(0.7, 0.6) >= 1 and E.optimal_ensemble_size(0.7, 1.0) == 1
    # model file operations
    a = {"w": torch.randn(4, 4), "b": torch.zeros(4), "old": torch.ones(2), "emb": torch.randn(10, 4)}
    b = {"w": a["w"] + 0.1 * torch.eye(4), "b": torch.zeros(4), "new": torch.ones(3), "emb": torch.randn(12, 4)}
    diff = E.compare_state_dicts(a, b)
    assert diff["only_in_a"] == ["old"] and diff["only_in_b"] == ["new"] and diff["shape_differences"] == [{"name": "emb", "a": (10, 4), "b": (12, 4)}] and diff["identical_tensors"] == 1 and diff["changed_tensors"] == 1
    assert diff["value_differences"][0]["name"] == "w" and diff["value_differences"][0]["max_abs"] == pytest.approx(0.1, rel=1e-4) and diff["value_differences"][0]["changed_fraction"] == 0.25 and not diff["same_architecture"] and E.compare_state_dicts(a, a)["identical"]
    sd = {"w": torch.randn(3, 3), "b": torch.arange(3.0)}
    torch.save(sd, tmp_path / "m.pt"); write_safetensors(sd, tmp_path / "m.safetensors"); np.savez(tmp_path / "m.npz", **{k_: v.numpy() for k_, v in sd.items()})
    for name in ("m.pt", "m.safetensors", "m.npz"):
        assert E.compare_state_dicts(E.load_model_auto(tmp_path / name), sd)["identical"], name
    with pytest.raises(ValueError, match="supported: .pt"):
        E.load_model_auto(tmp_path / "m.xyz")
    big = {"lin.weight": torch.randn(64, 64), "lin.bias": torch.randn(64), "spiky.weight": torch.cat([torch.randn(63, 64) * 0.01, torch.full((1, 64), 5.0)])}
    qs = E.quantization_stats(big)
    assert qs["tensors"] == 2 and qs["worst"][0]["name"] == "spiky.weight" and qs["worst"][0]["relative_error"] > qs["worst"][1]["relative_error"] and 3.5 < qs["compression"] < 4.0


def test_tensor_tuning_algorithms_blocking_tuner_bottlenecks_validation_plan_bf16_and_operation_log(tmp_path):
    from torsh_b200 import tensor_tuning as T
    torch.manual_seed(0)
    # Strassen
    a, b = torch.randn(150, 131, dtype=torch.float64), torch.randn(131, 97, dtype=torch.float64)
    assert torch.allclose(T.strassen_matmul(a, b, leaf=16), a @ b, atol=1e-9) and torch.allclose(T.strassen_matmul(a[:8, :8], b[:8, :8]), a[:8, :8] @ b[:8, :8])
    # Winograd and FFT convolution against the library
    x, w = torch.randn(2, 5, 13, 10, dtype=torch.float64), torch.randn(4, 5, 3, 3, dtype=torch.float64)
    ref = torch.nn.functional.conv2d(x, w)
    assert torch.allclose(T.winograd_conv2d(x, w), ref, atol=1e-10) and torch.allclose(T.fft_conv2d(x, w), ref, atol=1e-10)
    w7 = torch.randn(3, 5, 7, 5, dtype=torch.float64)
    assert torch.allclose(T.fft_conv2d(x, w7), torch.nn.functional.conv2d(x, w7), atol=1e-10)
    assert T.choose_conv_algorithm(3, 64, 56) == "winograd" and T.choose_conv_algorithm(3, 3, 224) == "implicit_gemm" and T.choose_conv_algorithm(11, 3, 224) == "fft" and T.choose_conv_algorithm(3, 64, 56, stride=2) == "implicit_gemm"
    # summation accuracy: one large value followed by many small ones
    v = torch.cat([torch.tensor([1e8]), torch.full((100000,), 0.01)]).float()
    exact = 1e8 + 1000.0
    import numpy as np
    naive = float(np.cumsum(v.numpy())[-1])                                          # strictly sequential float32 accumulation
    assert abs(float(T.kahan_sum(v)) - exact) <= 8 and abs(float(T.pairwise_sum(v)) - exact) <= 64 < abs(naive - exact)
    r = torch.randn(10007, dtype=torch.float64)
    assert float(T.pairwise_sum(r)) == pytest.approx(float(r.sum()), abs=1e-9) and float(T.kahan_sum(r)) == pytest.approx(float(r.sum()), abs=1e-9)
    # cache blocking
    tm, tn, tk = T.tile_sizes(4096, 4096, 4096, 4, cache_bytes=1 << 20)
    assert tm == tn == tk and tm % 16 == 0 and 3 * tm * tm * 4 <= 1 << 20 < 3 * (tm + 16) ** 2 * 4 and T.tile_sizes(8, 8, 8) == (8, 8, 8)
    assert torch.allclose(T.blocked_matmul(a, b, (32, 48, 64)), a @ b, atol=1e-9)
    small_t, big_t = T.memory_traffic_model(1024, 1024, 1024, (32, 32, 32)), T.memory_traffic_model(1024, 1024, 1024, (256, 256, 256))
    assert small_t["bytes"] > 4 * big_t["bytes"] and big_t["arithmetic_intensity"] > 4 * small_t["arithmetic_intensity"] and T.memory_traffic_model(64, 64, 64, (64, 64, 64))["reuse_factor"] == pytest.approx(4 / 3)
    # tuner
    now, calls = [0.0], []
    tuner = T.AdaptiveTuner(repeats=2, clock=lambda: now[0])
    mk = lambda name, cost: (lambda: (calls.append(name), now.__setitem__(0, now[0] + cost)))
    cands = {"direct": mk("direct", 0.3), "blocked": mk("blocked", 0.1), "strassen": mk("strassen", 0.2)}
    assert tuner.select("matmul", (1000, 1000, 1000), cands) == "blocked" and tuner.measurements == 3
    n_calls = len(calls)
    assert tuner.select("matmul", (1100, 900, 1024), cands) == "blocked" and len(calls) == n_calls and T.AdaptiveTuner.problem_class("matmul", (1000, 1000), torch.bfloat16) == "matmul|10,10|bfloat16"
    assert tuner.select("matmul", (16, 16, 16), {"direct": mk("direct", 0.01), "blocked": mk("blocked", 0.05)}) == "direct"
    tuner.save(tmp_path / "tune.json")
    assert T.AdaptiveTuner().load(tmp_path / "tune.json").select("matmul", (1000, 1000, 1000), {}) == "blocked"
    # bottleneck classification with a stated machine
    bp = T.BottleneckProfiler(calibrate=False, bandwidth=100e9, flops=1e12, overhead=5e-6)
    bp.record("copy", 2e-3, flops=0, nbytes=1e8); bp.record("gemm", 4e-3, flops=2e9, nbytes=1e7); bp.record("tiny_add", 6e-6, flops=100, nbytes=1200); bp.record("slow_gemm", 20e-3, flops=2e9, nbytes=1e7)
    an = {r["name"]: r for r in bp.analyze()}
    assert an["copy"]["bound"] == "memory" and an["copy"]["efficiency"] == pytest.approx(0.5) and an["gemm"]["bound"] == "compute" and an["gemm"]["efficiency"] == pytest.approx(0.5) and an["tiny_add"]["bound"] == "overhead" and bp.analyze()[0]["name"] == "slow_gemm"
    assert "100.0 GB/s" in bp.report() and "slow_gemm" in bp.report().splitlines()[2]
    live = T.BottleneckProfiler()
    live.measure("mm", lambda: a.float() @ b.float(), flops=2 * 150 * 131 * 97, nbytes=4 * (150 * 131 + 131 * 97 + 150 * 97))
    assert live.bandwidth > 0 and live.flops > 0 and live.overhead > 0 and live.analyze()[0]["bound"] in ("memory", "compute", "overhead")
    # validation across dtypes and layouts; a kernel that assumes contiguity is caught
    ok = T.validate_across_configurations(lambda p, q: p @ q, lambda g: [torch.randn(12, 9, generator=g), torch.randn(9, 7, generator=g)], devices=["cpu"])
    assert ok["passed"] and ok["checked"] == 12
    def assumes_contiguous(p, q):
        flat = torch.as_strided(p, (p.numel(),), (1,))                              # wrong for any non-contiguous input
        return flat.view(p.shape) @ q
    bad = T.validate_across_configurations(assumes_contiguous, lambda g: [torch.randn(12, 9, generator=g), torch.randn(9, 7, generator=g)], dtypes=(torch.float32,), devices=["cpu"])
    assert not bad["passed"] and {f["layout"] for f in bad["failures"]} == {"transposed", "strided"} and all(r["ok"] for r in bad["rows"] if r["layout"] == "contiguous")
    # plan for a workload
    plan = T.optimize_workload({"matmuls": [(4096, 4096, 4096), (64, 64, 64)], "convs": [(3, 64, 56), (11, 3, 224), (1, 256, 14)], "reductions": [1000, 1 << 20, 1 << 26], "dtype": torch.bfloat16, "allow_fast_algorithms": True})
    assert [m["algorithm"] for m in plan["matmul"]] == ["strassen", "direct"] and [c["algorithm"] for c in plan["conv"]] == ["winograd", "fft", "implicit_gemm"] and [r["method"] for r in plan["reduction"]] == ["direct", "pairwise", "kahan"] and any("float32" in n for n in plan["notes"])
    # bfloat16 rounding
    t = torch.randn(10000)
    assert torch.equal(T.bf16_round(t), t.to(torch.bfloat16)) and (T.bf16_round(t, "truncate").float().abs() <= t.abs()).all()
    vals = torch.full((200000,), 1.0 + 2.0 ** -10)
    st = T.bf16_round(vals, "stochastic", torch.Generator().manual_seed(0)).float()
    assert set(st.unique().tolist()) == {1.0, 1.0078125} and float(st.mean()) == pytest.approx(1.0 + 2.0 ** -10, abs=2e-5) and float(T.bf16_round(vals).float().mean()) == 1.0
    assert torch.isinf(T.bf16_round(torch.tensor([float("inf")]))).all() and torch.isnan(T.bf16_round(torch.tensor([float("nan")]))).all() and T.bf16_error_bound(1024) == pytest.approx(2 ** -7 + 1024 * 2 ** -24)
    # operation log
    with T.OperationLog() as log:
        y = torch.relu(torch.ones(4, 3) @ torch.ones(3, 2)) + 1
    ops = [e["op"] for e in log.entries]
    assert "matmul" in ops and "relu" in ops and log.summary()["matmul"]["count"] == 1 and [e for e in log.entries if e["op"] == "matmul"][0]["shapes"] == [(4, 3), (3, 2)] and len(log.to_jsonl().splitlines()) == len(log.entries)
    with T.OperationLog(only=["relu"]) as log2:
        torch.relu(torch.ones(2)); torch.exp(torch.ones(2))
    assert [e["op"] for e in log2.entries] == ["relu"]


def test_nn_blocks_factories_positions_attention_conv_blocks_backbones_pooling_and_cells():
    import torsh_b200.nn as tnn
    from torsh_b200.nn import blocks as B
    torch.manual_seed(0)
    # factories
    assert isinstance(B.ActivationFactory.create("GELU"), torch.nn.GELU) and B.ActivationFactory.create("leaky-relu", negative_slope=0.3).negative_slope == 0.3 and "geglu" in B.ActivationFactory.available() and tnn.ActivationFactory is B.ActivationFactory
    with pytest.raises(ValueError, match="unknown activation"):
        B.ActivationFactory.create("nope")
    act = B.ActivationBuilder("leaky_relu").negative_slope(0.2).inplace().build()
    assert act.negative_slope == 0.2 and act.inplace
    x = torch.randn(4, 7, 16)
    ln = B.AdvancedLayerNorm(16)
    assert torch.allclose(ln(x), torch.nn.functional.layer_norm(x, (16,)), atol=1e-6)
    rms = B.AdvancedLayerNorm(16, rms=True, eps=1e-6)
    assert rms.bias is None and torch.allclose(rms(x), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-6)
    r = torch.randn_like(x)
    assert torch.allclose(ln(x, residual=r), torch.nn.functional.layer_norm(x + r, (16,)), atol=1e-6) and ln(x.bfloat16()).dtype == torch.bfloat16
    NF = B.NormalizationFactory
    assert isinstance(NF.create("batch", 8, dims=1), torch.nn.BatchNorm1d) and isinstance(NF.create(B.NormalizationPresets.resnet(), 8), torch.nn.BatchNorm2d) and NF.create("group", 48).num_groups == 16 and isinstance(NF.create("none", 3), torch.nn.Identity)
    assert NF.create(B.NormalizationPresets.llama(), 16).rms and isinstance(NF.create(B.NormalizationPresets.style_transfer(), 4), torch.nn.InstanceNorm2d) and B.NormalizationPresets.diffusion_unet().groups == 32
    bn = NF.create("batch", 16, dims=1)
    stats = B.NormalizationStats(bn)
    bn(torch.randn(64, 16) * 3 + 5)
    s = stats.summary()
    assert abs(s["in_mean"] - 5) < 0.5 and abs(s["out_mean"]) < 1e-5 and abs(s["out_var"] - 1) < 0.05
    stats.remove()
    # positions
    pe = B.PositionalEncoding(16)
    out = pe(torch.zeros(2, 10, 16))
    assert out[0, 0, 0::2].abs().sum() == 0 and torch.allclose(out[0, 0, 1::2], torch.ones(8)) and out[0, 3, 0] == pytest.approx(math.sin(3.0))
    te = B.SinusoidalPositionEmbedding(8)(torch.tensor([0.0, 10.0]))
    assert te.shape == (2, 8) and te[0].tolist() == [0, 0, 0, 0, 1, 1, 1, 1] and te[1, 0] == pytest.approx(math.sin(10.0))
    rel = B.RelativePositionalEncoding(4, max_distance=3)
    rb = rel(5, 5)
    assert rb.shape == (4, 5, 5) and torch.equal(rb[:, 0, 1], rb[:, 2, 3]) and torch.equal(rb[:, 0, 3], rb[:, 0, 4]) and not torch.equal(rb[:, 0, 1], rb[:, 1, 0])
    ali = B.AlibiPositionalBias(8)
    ab = ali(4, 4)
    assert ali.slopes.tolist() == pytest.approx([2 ** -(i + 1) for i in range(8)]) and ab[0, 3, 1] == pytest.approx(-0.5 * 2) and torch.isinf(ab[0, 1, 2]) and ab[:, 2, 2].abs().sum() == 0 and len(B.AlibiPositionalBias(12).slopes) == 12
    assert not torch.isinf(B.AlibiPositionalBias(4, causal=False)(3, 3)).any() and B.AlibiPositionalBias(4)(1, 5)[0, 0].tolist() == pytest.approx([-1.0, -0.75, -0.5, -0.25, 0.0])
    # attention equals the library layer given the same weights
    mha, ref = B.MultiHeadAttention(16, 4), torch.nn.MultiheadAttention(16, 4, batch_first=True)
    with torch.no_grad():
        ref.in_proj_weight.copy_(torch.cat([mha.q_proj.weight, mha.k_proj.weight, mha.v_proj.weight])); ref.in_proj_bias.copy_(torch.cat([mha.q_proj.bias, mha.k_proj.bias, mha.v_proj.bias]))
        ref.out_proj.weight.copy_(mha.out_proj.weight); ref.out_proj.bias.copy_(mha.out_proj.bias)
    pad = torch.zeros(4, 7, dtype=torch.bool); pad[1, 5:] = True
    o1, w1 = mha(x, key_padding_mask=pad, need_weights=True)
    o2, w2 = ref(x, x, x, key_padding_mask=pad)
    assert torch.allclose(o1, o2, atol=1e-5) and torch.allclose(w1, w2, atol=1e-5) and torch.allclose(mha(x, key_padding_mask=pad), o1, atol=1e-5)
    cm = torch.nn.Transformer.generate_square_subsequent_mask(7)
    assert torch.allclose(mha(x, causal=True), ref(x, x, x, attn_mask=cm)[0], atol=1e-5) and mha(x, attn_bias=B.AlibiPositionalBias(4)(7, 7)).shape == x.shape
    mem = torch.randn(4, 3, 16)
    assert mha(x, mem).shape == (4, 7, 16)
    with pytest.raises(ValueError):
        B.MultiHeadAttention(10, 3)
    gg = B.GEGLU(16, 32)
    assert gg(x).shape == (4, 7, 32) and torch.allclose(B.GEGLU()(x), torch.nn.functional.gelu(x[..., :8]) * x[..., 8:])
    # convolutional blocks
    img = torch.randn(2, 16, 8, 8)
    assert B.BasicBlock(16, 16)(img).shape == img.shape and B.BasicBlock(16, 32, 2)(img).shape == (2, 32, 4, 4) and B.BasicBlock(16, 16).short is None and B.BottleneckBlock(16, 8, 2)(img).shape == (2, 32, 4, 4) and B.BottleneckBlock.expansion == 4
    assert B.BasicBlock(16, 16, cfg=B.BlockConfig(norm="group", activation="silu"))(img).shape == img.shape
    assert B.DenseLayer(16, growth_rate=12)(img).shape == (2, 28, 8, 8) and B.TransitionLayer(28)(torch.randn(2, 28, 8, 8)).shape == (2, 14, 4, 4)
    ds = B.DepthwiseSeparableConv(16, 32, 3, 2)
    full = torch.nn.Conv2d(16, 32, 3, 2, 1)
    assert ds(img).shape == (2, 32, 4, 4) and ds.multiply_adds(8, 8) == 16 * (16 * 9 + 16 * 32) and sum(p.numel() for p in ds.parameters() if p.dim() == 4) < 0.2 * full.weight.numel() and B.MobileNetV1Block is B.DepthwiseSeparableConv
    ir = B.InvertedResidual(16, 16)
    assert ir.use_res and ir(img).shape == img.shape and not B.InvertedResidual(16, 24, 2).use_res and B.InvertedResidual(16, 24, 2)(img).shape == (2, 24, 4, 4) and len(B.InvertedResidual(16, 16, expand_ratio=1).body) == 2
    mb = B.MBConvWithStochasticDepth(16, 16, drop_rate=0.5).eval()
    base = mb(img)
    mb.train()
    torch.manual_seed(1)
    dropped = [bool(torch.allclose(mb(img)[i], img[i])) for _ in range(20) for i in range(2)]
    assert 5 < sum(dropped) < 35 and base.shape == img.shape
    # backbones
    mn = B.MobileNetV1(num_classes=10, width_multiplier=0.25)
    assert mn(torch.randn(2, 3, 64, 64)).shape == (2, 10) and 150_000 < sum(p.numel() for p in mn.parameters()) < 300_000
    cfg = B.EfficientNetConfig(width_coefficient=1.1, depth_coefficient=1.2)
    assert cfg.round_channels(32) == 32 and cfg.round_channels(40) == 48 and cfg.round_repeats(3) == 4
    eff = B.EfficientNetBackbone(B.EfficientNetConfig(width_coefficient=0.25, depth_coefficient=0.35, num_classes=7))
    assert eff(torch.randn(2, 3, 64, 64)).shape == (2, 7) and eff.forward_features(torch.randn(1, 3, 64, 64)).shape == (1, eff.out_channels, 2, 2)
    b0 = sum(p.numel() for p in B.EfficientNetBackbone().parameters())
    assert 5.0e6 < b0 < 5.6e6                                                       # EfficientNet-B0 has 5.3 M parameters
    # pooling and cells
    v = torch.arange(24.0).reshape(1, 2, 3, 4)
    assert B.GlobalPool("avg")(v).tolist() == [[5.5, 17.5]] and B.GlobalPool("max")(v).tolist() == [[11.0, 23.0]] and B.GlobalPool("avgmax")(v).tolist() == [[8.25, 20.25]] and B.GlobalPool("catavgmax")(v).shape == (1, 4)
    fp = B.FractionalMaxPool1d(2, 0.7).eval()
    seq = torch.arange(20.0).reshape(1, 1, 20)
    po = fp(seq)
    assert po.shape == (1, 1, 14) and (po.diff() >= 0).all() and po[0, 0, -1] == 19 and po[0, 0, 0] == 1
    cell = B.CustomRNNCell(5, 8, activation="relu", layer_norm=True, learn_initial_state=True)
    hs, last = cell.unroll(torch.randn(3, 6, 5))
    assert hs.shape == (3, 6, 8) and torch.equal(hs[:, -1], last) and (hs >= 0).all() and cell.initial_state(3).shape == (3, 8)
    last.sum().backward()
    assert cell.h0.grad is not None and cell.hh.weight.grad.abs().sum() > 0


def test_optim_more_adam_variants_population_methods_gp_benchmarks_stress_wrappers_and_builders():
    import torsh_b200.optim as O
    from scipy.optimize import rosen
    torch.manual_seed(0)
    assert O.AdaDelta is torch.optim.Adadelta and O.AdaGrad is torch.optim.Adagrad and O.AdaMax is torch.optim.Adamax
    # AdvancedAdam with the switches off is AdamW; the switches do what they say
    w1, w2 = torch.nn.Parameter(torch.randn(4, 3)), None
    w2 = torch.nn.Parameter(w1.detach().clone())
    a, b = O.AdvancedAdam([w1], lr=0.01, weight_decay=0.1), torch.optim.AdamW([w2], lr=0.01, weight_decay=0.1)
    for _ in range(5):
        for w, o in ((w1, a), (w2, b)):
            o.zero_grad(); (w ** 2).sum().backward(); o.step()
    assert torch.allclose(w1, w2, atol=1e-6)
    w3 = torch.nn.Parameter(torch.ones(2, 3)); w3.grad = torch.ones(2, 3)
    before = w3.detach().clone()
    O.AdvancedAdam([w3], centralize=True).step()
    assert torch.allclose(w3, before)                                               # a constant gradient per row is centred away
    w4 = torch.nn.Parameter(torch.zeros(3)); w4.grad = torch.tensor([1.0, -1.0, 1e-9])
    O.AdvancedAdam([w4], lr=1.0, max_update=0.1).step()
    assert w4.abs().max() <= 0.1 + 1e-6
    ams = O.AdvancedAdam([torch.nn.Parameter(torch.ones(1))], amsgrad=True)
    p = ams.param_groups[0]["params"][0]
    for gval in (10.0, 0.1, 0.1):
        p.grad = torch.tensor([gval]); ams.step()
    assert float(ams.state[p]["vmax"]) >= float(ams.state[p]["v"])
    # schedule-free AdamW: trains without a schedule; the averaged weights are at least as good
    X = torch.randn(200, 5); yt = X @ torch.tensor([1.0, -2.0, 0.5, 0.0, 3.0]) + 0.05 * torch.randn(200)
    lin = torch.nn.Linear(5, 1)
    sf = O.ScheduleFreeAdamW(lin.parameters(), lr=0.05, warmup_steps=10)
    for i in range(300):
        idx = torch.randint(0, 200, (32,))
        sf.zero_grad(); torch.nn.functional.mse_loss(lin(X[idx]).squeeze(-1), yt[idx]).backward(); sf.step()
    train_loss = float(torch.nn.functional.mse_loss(lin(X).squeeze(-1), yt).detach())
    sf.eval_mode(); eval_loss = float(torch.nn.functional.mse_loss(lin(X).squeeze(-1), yt).detach()); y_params = lin.weight.detach().clone()
    sf.train_mode()
    assert eval_loss < 0.05 and eval_loss <= train_loss * 1.5 and not torch.equal(y_params, lin.weight.detach()) and type(O.Sophia(lin.parameters())).__name__ == "SophiaG"
    # population methods on standard functions
    ros, sph, ras = O.Rosenbrock(), O.Sphere(), O.Rastrigin()
    xr = torch.tensor([-1.2, 1.0, 0.5], dtype=torch.float64)
    assert float(ros(xr)) == pytest.approx(rosen(xr.numpy())) and float(ras(torch.zeros(3))) == 0.0 and float(O.Branin()(O.Branin().optimum())) == pytest.approx(O.Branin.minimum, abs=1e-6)
    cma = O.CMAES(torch.tensor([-1.5, 1.5, -0.5, 0.8]), sigma=0.5, seed=1).minimize(ros, generations=400)
    assert cma["value"] < 1e-8 and torch.allclose(cma["x"], torch.ones(4, dtype=torch.float64), atol=1e-3)
    es = O.OpenAIES(torch.full((5,), 2.0), sigma=0.1, population=40, lr=0.1, seed=0).minimize(sph, iterations=150)
    assert es["value"] < 0.05 and es["history"][-1] < es["history"][0]
    pso = O.ParticleSwarmOptimizer(3, particles=40, bounds=ras.bounds, seed=0).minimize(ras, iterations=150)
    assert pso["value"] < 1.5 and pso["x"].abs().max() <= 5.12
    # Gaussian process: interpolates, is uncertain away from data, EI prefers the promising gap
    xs = torch.tensor([[0.0], [1.0], [2.0], [4.0]]); ys = torch.sin(xs[:, 0])
    gp = O.GaussianProcess(length_scale=1.0, noise_var=1e-8).fit(xs, ys)
    mu, var = gp.predict(xs)
    assert torch.allclose(mu, ys.double(), atol=1e-5) and var.max() < 1e-6
    mu2, var2 = gp.predict(torch.tensor([[3.0], [10.0]]))
    assert var2[1] > 0.99 and var2[0] < var2[1] and abs(float(mu2[1]) - float(ys.mean())) < 1e-6
    from sklearn.gaussian_process import GaussianProcessRegressor
    from sklearn.gaussian_process.kernels import RBF
    sk = GaussianProcessRegressor(RBF(1.0), alpha=1e-8, optimizer=None, normalize_y=False).fit(xs.numpy(), (ys - ys.mean()).numpy())
    assert float(mu2[0]) == pytest.approx(float(sk.predict([[3.0]])[0] + ys.mean()), abs=1e-5) and gp.log_marginal_likelihood() == pytest.approx(sk.log_marginal_likelihood_value_, rel=1e-5)
    ei = gp.expected_improvement(torch.tensor([[1.0], [3.0], [5.0]]))
    assert ei[0] < 1e-6 and ei[2] > ei[0]
    # convergence tracker
    ct = O.ConvergenceTracker(patience=3, min_delta=1e-3)
    assert [ct.update(v) for v in (1.0, 0.5, 0.4999, 0.4999, 0.4999)] == [None, None, None, None, "stalled"] and O.ConvergenceTracker().update(float("nan")) == "diverged" and O.ConvergenceTracker(grad_tol=1e-3).update(1.0, 1e-5) == "gradient_tolerance"
    ct2 = O.ConvergenceTracker()
    for i in range(10):
        ct2.update(math.exp(-0.5 * i))
    assert ct2.rate() == pytest.approx(0.5) and ct2.update(1e9) == "diverged"
    # benchmarks and stress tests
    res = O.OptimizerBenchmarks(dim=3, steps=300, tol=1e-3).run({"sgd": lambda p: torch.optim.SGD(p, lr=1e-3), "lbfgs": lambda p: torch.optim.LBFGS(p, lr=1.0, max_iter=5, line_search_fn="strong_wolfe")})
    assert res["rosenbrock"]["winner"] == "lbfgs" and res["rosenbrock"]["lbfgs"]["steps_to_tolerance"] is not None and res["sphere"]["lbfgs"]["final"] < 1e-6
    st_adam = O.OptimizerStressTester(lambda p: torch.optim.Adam(p, lr=0.05)).run()
    st_sgd = O.OptimizerStressTester(lambda p: torch.optim.SGD(p, lr=0.05)).run()
    assert st_adam["ill_conditioned"]["finite"] and st_adam["spike"]["finite"] and not st_sgd["ill_conditioned"]["finite"] and not st_adam["non_finite"]["finite"] and "ill_conditioned" in st_adam["passed"]
    # wrappers
    ci = [500.0]
    wp = torch.nn.Parameter(torch.zeros(1))
    cc = O.CarbonConsciousOptimizer(torch.optim.SGD([wp], lr=1.0), lambda: ci[0], threshold=400, defer_factor=4)
    for _ in range(8):
        wp.grad = (wp.grad if wp.grad is not None else 0) + torch.ones(1)
        cc.step()
    assert cc.report()["applied"] == 2 and float(wp.detach()) == -8.0                      # accumulated gradients are applied later: nothing is lost
    ci[0] = 100.0
    wp.grad = torch.ones(1)
    assert cc.step() and cc.report()["grams_co2"] > 0
    pauses, watts = [], [900.0]
    pc = O.PowerCappedOptimizer(torch.optim.SGD([wp], lr=0.0), lambda: watts[0], cap_watts=700.0, sleep=pauses.append)
    wp.grad = torch.zeros(1)
    pc.step(); watts[0] = 500.0
    for _ in range(10):
        pc.step()
    assert pauses and pauses[0] == pytest.approx(0.01 * 200 / 700) and pc.avg < 700 and len(pauses) < 5
    wq = torch.nn.Parameter(torch.tensor([5.0]))
    ck = O.CheckpointingOptimizer(torch.optim.SGD([wq], lr=0.1, momentum=0.9), every=5, keep=2)
    for i in range(12):
        ck.zero_grad(); (wq ** 2).sum().backward(); ck.step()
        if i == 9:
            good = wq.detach().clone()
    wq.data.fill_(1e9)
    assert ck.rollback() == 10 and torch.equal(wq.detach(), good) and len(ck.snapshots) == 2 and ck.n == 10
    wt = torch.nn.Parameter(torch.zeros(2))
    tc = O.TemporalCreditOptimizer([wt], lr=1.0, trace_decay=0.5)
    for gr in ([1.0, 0.0], [0.0, 1.0]):
        wt.grad = torch.tensor(gr); tc.accumulate()
    tc.step(reward=2.0)
    assert wt.tolist() == [1.0, 2.0] and type(O.LowPrecisionOptimizer([torch.nn.Parameter(torch.zeros(2))])).__name__ == "LowPrecisionAdam"
    # builders and task matching
    model = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.LayerNorm(4))
    groups = O.ParamGroupBuilder().no_decay_for(model, 0.1).build()
    assert len(groups[0]["params"]) == 1 and len(groups[1]["params"]) == 3 and groups[1]["weight_decay"] == 0.0
    opt = O.OptimizerBuilder("adamw").lr(3e-4).weight_decay(0.1).betas((0.9, 0.95)).build(model.parameters())
    assert isinstance(opt, torch.optim.AdamW) and opt.defaults["betas"] == (0.9, 0.95) and type(O.OptimizerBuilder("lion").lr(1e-4).build(model.parameters())).__name__ == "Lion"
    with pytest.raises(ValueError):
        O.OptimizerBuilder("nope").build(model.parameters())
    tm = O.TaskMatcher().with_defaults()
    assert tm.suggest({"parameters": 7e9, "samples": 1e10, "gradient_noise": 0.3})["optimizer"] == "adamw" and tm.suggest({"parameters": 1.1e7, "samples": 1e6})["optimizer"] == "sgd" and tm.suggest({"parameters": 5e5, "samples": 1e5, "gradient_sparsity": 0.9})["optimizer"] == "adagrad"
    assert tm.suggest({"parameters": 5e3, "samples": 500}, k=2)["optimizer"] == "lbfgs" and len(tm.suggest({"parameters": 5e3, "samples": 500}, k=2)["alternatives"]) == 2


def test_series_models_var_vecm_x11_mice_wavelets_and_purged_validation():
    import itertools
    import numpy as np
    from scipy import signal as sps
    from torsh_b200 import series_models as sm

    g = torch.Generator().manual_seed(0)
    # ---- VAR: recover known matrices, stability, forecasts converge to the mean, FEVD rows sum to one, causality
    A1 = torch.tensor([[0.5, 0.2], [0.0, 0.4]], dtype=torch.float64)
    A2 = torch.tensor([[0.1, 0.0], [0.0, -0.2]], dtype=torch.float64)
    c = torch.tensor([1.0, -0.5], dtype=torch.float64)
    y = [torch.zeros(2, dtype=torch.float64)] * 2
    for _ in range(6000):
        y.append(c + A1 @ y[-1] + A2 @ y[-2] + 0.5 * torch.randn(2, generator=g, dtype=torch.float64))
    y = torch.stack(y[200:])
    var = sm.VAR(2).fit(y)
    assert torch.allclose(var.coefs[0], A1, atol=0.05) and torch.allclose(var.coefs[1], A2, atol=0.05)
    assert torch.allclose(var.intercept, c, atol=0.1) and var.is_stable()
    assert torch.allclose(var.sigma_u, 0.25 * torch.eye(2, dtype=torch.float64), atol=0.03)
    mean = torch.linalg.solve(torch.eye(2, dtype=torch.float64) - A1 - A2, c)
    assert torch.allclose(var.forecast(200)[-1], mean, atol=0.15)
    assert sm.VAR.select_order(y, 5, "bic") == 2
    irf = var.impulse_response(8, orthogonal=False)
    assert torch.allclose(irf[0], torch.eye(2, dtype=torch.float64)) and torch.allclose(irf[1], var.coefs[0])
    assert torch.allclose(irf[2], var.coefs[0] @ var.coefs[0] + var.coefs[1])
    fe = var.fevd(6)
    assert torch.allclose(fe.sum(2), torch.ones(6, 2, dtype=torch.float64))
    assert var.test_causality(y, caused=0, causing=1)["p_value"] < 1e-6           # y1 drives y0 through A1[0, 1]
    assert var.test_causality(y, caused=1, causing=0)["p_value"] > 0.001

    # ---- Johansen / VECM: two series sharing one random walk have rank one with vector proportional to (1, -2)
    w = torch.randn(1500, generator=g, dtype=torch.float64).cumsum(0)
    yy = torch.stack([2 * w + torch.randn(1500, generator=g, dtype=torch.float64), w + torch.randn(1500, generator=g, dtype=torch.float64)], 1)
    jo = sm.johansen_test(yy, 1)
    assert jo.rank == 1 and float(jo.trace_stat[0]) > jo.trace_crit_95[0] and float(jo.trace_stat[1]) < jo.trace_crit_95[1]
    b = jo.eigenvectors[:, 0]
    assert abs(float(b[1] / b[0]) + 2.0) < 0.1
    indep = torch.randn(1500, 2, generator=g, dtype=torch.float64).cumsum(0)
    assert sm.johansen_test(indep, 1).rank == 0
    ve = sm.VECM(1).fit(yy)
    assert ve.rank == 1 and abs(float(ve.beta[1, 0]) + 2.0) < 0.1 and float(ve.beta[0, 0]) == pytest.approx(1.0)
    assert float(ve.alpha[0, 0]) < 0 or float(ve.alpha[1, 0]) > 0                 # error correction pulls back to equilibrium
    fc = ve.forecast(50)
    assert abs(float(fc[-1, 0] - 2 * fc[-1, 1])) < abs(float(yy[-1, 0] - 2 * yy[-1, 1])) + 0.5
    Avar = ve.to_var()
    lvl = Avar[0] @ yy[-1] + Avar[1] @ yy[-2] + ve.const                          # level form reproduces the one-step forecast
    assert torch.allclose(lvl, fc[0], atol=1e-8)
    eg = sm.engle_granger(yy[:, 0], yy[:, 1])
    assert eg.cointegrated and abs(float(eg.beta[1]) - 2.0) < 0.1
    assert not sm.engle_granger(indep[:, 0], indep[:, 1]).cointegrated
    assert sm.phillips_perron(torch.randn(800, generator=g, dtype=torch.float64)).stationary
    assert not sm.phillips_perron(w).stationary

    # ---- Henderson and X-11
    for L in (5, 9, 13, 23):
        hw = sm.henderson_weights(L)
        j = torch.arange(-(L // 2), L // 2 + 1, dtype=torch.float64)
        assert float(hw.sum()) == pytest.approx(1.0, abs=1e-12) and abs(float((hw * j ** 2).sum())) < 1e-12
    assert float(sm.henderson_weights(13)[6]) == pytest.approx(0.24006, abs=1e-5)
    t = torch.arange(240, dtype=torch.float64)
    season = torch.tensor([3.0, 1, -2, -4, -1, 2, 5, 3, -1, -3, -2, -1], dtype=torch.float64)
    season = season - season.mean()
    trend = 50 + 0.3 * t + 0.001 * t ** 2
    x = trend + season.repeat(20) + 0.2 * torch.randn(240, generator=g, dtype=torch.float64)
    d = sm.X11Decomposition(12).decompose(x)
    assert float((d["seasonal"][24:-24] - season.repeat(20)[24:-24]).abs().max()) < 0.5
    assert float((d["trend"][24:-24] - trend[24:-24]).abs().max()) < 0.6
    assert torch.allclose(d["trend"] + d["seasonal"] + d["irregular"], x, atol=1e-9)
    xm = trend * (1 + season.repeat(20) / 20)
    dm = sm.X11Decomposition(12, "multiplicative").decompose(xm)
    assert torch.allclose(dm["trend"] * dm["seasonal"] * dm["irregular"], xm, rtol=1e-9)
    assert float((dm["seasonal"][24:-24] - (1 + season.repeat(20) / 20)[24:-24]).abs().max()) < 0.02
    md = sm.MultiplicativeDecomposition(12).decompose(xm)
    assert torch.allclose(md["trend"] * md["seasonal"] * md["residual"], xm, rtol=1e-9)
    assert set(sm.STLDecomposition(12).decompose(x)) >= {"trend", "seasonal", "remainder"}
    ms = sm.MSTLDecomposition([12, 4]).decompose(x)
    assert set(ms["seasonal"]) == {4, 12}

    # ---- SSA: a sine plus trend is captured by a few components and forecast by the recurrence
    xs = 0.02 * t[:200] + torch.sin(2 * math.pi * t[:200] / 20)
    ssa = sm.SSA(40).fit(xs)
    assert float(ssa.explained()[:4].sum()) > 0.999
    assert torch.allclose(ssa.reconstruct(range(len(ssa.S))), xs, atol=1e-8)
    truth = 0.02 * t[200:210] + torch.sin(2 * math.pi * t[200:210] / 20)
    assert float((ssa.forecast(10, rank=4) - truth).abs().max()) < 0.05

    # ---- MICE: a column that is a linear function of the others is recovered
    X = torch.randn(300, 3, generator=g, dtype=torch.float64)
    full = torch.cat([X, (X @ torch.tensor([1.0, -2.0, 0.5], dtype=torch.float64) + 3)[:, None]], 1)
    holes = full.clone()
    holes[::7, 3] = float("nan")
    holes[5::14, 0] = float("nan")
    filled = sm.MICEImputer(iters=15).fit_transform(holes)
    assert not torch.isnan(filled).any() and float((filled - full).abs().max()) < 1e-3
    assert torch.equal(filled[~torch.isnan(holes)], full[~torch.isnan(holes)])
    col = torch.arange(10, dtype=torch.float64).clone()
    col[4] = float("nan")
    assert float(sm.TimeSeriesImputer("linear").fit_transform(torch.stack([col, col], 1))[4, 1]) == pytest.approx(4.0)

    # ---- smoothing classes
    hw_x = 20 + 0.5 * t[:120] + season.repeat(10)
    hw = sm.HoltWinters(12).fit(hw_x, optimize=True)
    want = 20 + 0.5 * t[120:132] + season
    assert float((hw.forecast(12) - want).abs().max()) < 0.5
    hm = sm.HoltWinters(12, seasonal="multiplicative").fit((20 + 0.5 * t[:120]) * (1 + season.repeat(10) / 20))
    assert float((hm.forecast(12) / ((20 + 0.5 * t[120:132]) * (1 + season / 20)) - 1).abs().max()) < 0.05
    ses = sm.SimpleExpSmoothing().fit(torch.cat([torch.zeros(30), torch.ones(30) * 5]).double() + 0.01 * torch.randn(60, generator=g, dtype=torch.float64))
    assert ses.alpha > 0.8 and float(ses.forecast(3)[0]) == pytest.approx(5.0, abs=0.1)
    des = sm.DoubleExpSmoothing(0.8, 0.5).fit(3 + 2 * t[:50])
    assert torch.allclose(des.forecast(3), 3 + 2 * t[50:53], atol=1e-6)
    damped = sm.DoubleExpSmoothing(0.8, 0.5, phi=0.8).fit(3 + 2 * t[:50]).forecast(40)
    assert float(damped[-1] - damped[-2]) < 0.01
    ar = torch.zeros(600, dtype=torch.float64)
    e = torch.randn(600, generator=g, dtype=torch.float64)
    for i in range(1, 600):
        ar[i] = 0.7 * ar[i - 1] + e[i]
    arima = sm.ARIMA(1, 0, 0).fit(ar)
    assert arima.forecast(5).shape == (5,) and abs(float(arima.forecast(1)[0]) - 0.7 * float(ar[-1])) < 0.3
    assert sm.AutoARIMA(max_p=2, max_q=1).fit(ar).order[1] == 0

    # ---- change points
    steps = torch.cat([torch.zeros(80), torch.ones(70) * 4, torch.ones(90) * -1]).double() + 0.3 * torch.randn(240, generator=g, dtype=torch.float64)
    for method in ("pelt", "binseg"):
        r = sm.ChangePointDetector(method).detect(steps)
        assert len(r["change_points"]) == 2 and abs(r["change_points"][0] - 80) <= 2 and abs(r["change_points"][1] - 150) <= 2
        assert r["segment_means"][1] == pytest.approx(4.0, abs=0.2)

    # ---- spectra against scipy
    fs = 100.0
    tt = torch.arange(4096, dtype=torch.float64) / fs
    sig = torch.sin(2 * math.pi * 12 * tt) + 0.5 * torch.randn(4096, generator=g, dtype=torch.float64)
    f, p = sm.PSDEstimator(fs, 512).estimate(sig)
    f_ref, p_ref = sps.welch(sig.numpy(), fs, nperseg=512)
    assert np.allclose(f.numpy(), f_ref) and np.allclose(p.numpy(), p_ref, rtol=1e-9)
    other = torch.sin(2 * math.pi * 12 * tt + 0.7) + 0.5 * torch.randn(4096, generator=g, dtype=torch.float64)
    co = sm.CoherenceAnalyzer(fs, 512).analyze(sig, other)
    _, c_ref = sps.coherence(sig.numpy(), other.numpy(), fs, nperseg=512)
    assert np.allclose(co["coherence"].numpy(), c_ref, rtol=1e-8)
    k12 = int(torch.argmin((co["freqs"] - 12).abs()))
    assert float(co["coherence"][k12]) > 0.9 and float(co["phase"][k12]) == pytest.approx(0.7, abs=0.1)
    fa = sm.FFTAnalyzer(fs).analyze(3 * torch.sin(2 * math.pi * 12.5 * tt[:4000]))
    assert fa["dominant_frequency"] == pytest.approx(12.5, abs=0.03) and fa["dominant_amplitude"] == pytest.approx(3.0, rel=0.02)
    assert sm.PeriodogramAnalyzer().analyze(torch.sin(2 * math.pi * t / 24))["dominant_period"] == pytest.approx(24, rel=0.05)

    # ---- CWT: a chirp's ridge follows its instantaneous frequency
    cw = sm.CWTAnalyzer(6.0, fs)
    freqs = torch.linspace(4, 30, 40, dtype=torch.float64)
    scales = cw.frequency_to_scale(freqs)
    assert torch.allclose(cw.scale_to_frequency(scales), freqs)
    res = cw.analyze(torch.sin(2 * math.pi * 12 * tt), scales)
    assert res["dominant_frequency"] == pytest.approx(12, abs=0.7)
    chirp = torch.sin(2 * math.pi * (5 * tt + 0.25 * tt ** 2))                      # 5 Hz rising 0.5 Hz/s
    P = cw.transform(chirp, scales).abs() / scales.sqrt()[:, None]
    for sample in (1000, 2000, 3000):
        assert float(freqs[int(P[:, sample].argmax())]) == pytest.approx(5 + 0.5 * sample / fs, abs=1.0)

    # ---- wavelets: perfect reconstruction, energy conservation, polynomial cancellation, denoising, packets
    for name in ("haar", "db2", "db4"):
        wd = sm.WaveletDecomposer(name, 3)
        z = torch.randn(256, generator=g, dtype=torch.float64)
        cs = wd.decompose(z)
        assert [len(v) for v in cs] == [32, 32, 64, 128]
        assert torch.allclose(wd.reconstruct(cs), z, atol=1e-10)
        assert float(sum((v ** 2).sum() for v in cs)) == pytest.approx(float((z ** 2).sum()), rel=1e-10)
    lin = sm.WaveletDecomposer("db2", 1).decompose(torch.arange(64, dtype=torch.float64))[1]
    assert float(lin[:-1].abs().max()) < 1e-10                                     # two vanishing moments (wrap-around aside)
    clean = torch.sin(2 * math.pi * torch.arange(512, dtype=torch.float64) / 128)
    noisy = clean + 0.3 * torch.randn(512, generator=g, dtype=torch.float64)
    den = sm.WaveletDecomposer("db4", 4).denoise(noisy)
    assert float((den - clean).pow(2).mean()) < 0.35 * float((noisy - clean).pow(2).mean())
    assert float(sm.WaveletDecomposer("db4", 4).energy_by_level(clean)[0]) > 0.9
    wp = sm.WaveletPacketDecomposer("db2", 3)
    leaves = wp.decompose(noisy)
    assert len(leaves) == 8 and torch.allclose(wp.reconstruct(leaves), noisy, atol=1e-10)
    bb = wp.best_basis(clean)
    assert torch.allclose(wp.reconstruct(bb), clean, atol=1e-10) and len(bb) <= 8

    # ---- transfer entropy with a common driver
    n = 4000
    z = torch.randn(n, generator=g, dtype=torch.float64)
    xa = torch.roll(z, 1) + 0.3 * torch.randn(n, generator=g, dtype=torch.float64)
    yb = torch.roll(z, 2) + 0.3 * torch.randn(n, generator=g, dtype=torch.float64)  # both driven by z; x leads y only through z
    te = sm.TransferEntropyEstimator(3).estimate(xa, yb)
    cte = sm.ConditionalTransferEntropy(3).estimate(xa, yb, torch.roll(z, 1))
    assert te > 0.1 and cte < 0.5 * te
    assert sm.TransferEntropyEstimator(3).net_flow(xa, yb) > 0
    assert sm.GrangerCausality(2).test(yb, xa)["p_value"] < 1e-6
    assert "pp" in sm.StationarityTestSuite().run(z[:500]) and "ljung_box" in sm.ResidualDiagnostics().run(z[:500])
    rs = sm.RollingStatistics(5)
    assert float(rs.mean(t[:10])[-1]) == pytest.approx(7.0) and torch.isnan(rs.zscore(t[:10])[0])

    # ---- detectors
    base = torch.sin(2 * math.pi * t / 24) + 0.05 * torch.randn(240, generator=g, dtype=torch.float64)
    spiked = base.clone()
    spiked[100] += 4.0
    assert bool(sm.OutlierDetector("hampel").detect(spiked)[100]) and int(sm.OutlierDetector("hampel").detect(spiked).sum()) <= 3
    assert abs(float(sm.OutlierDetector("hampel").treat(spiked)[100] - base[100])) < 0.3
    for m in ("zscore", "mad", "iqr"):
        assert bool(sm.StatisticalDetector(m, 3.0).detect(spiked)[100])
    wdet = sm.WindowDetector(24, 3.5).detect(spiked)
    assert bool(wdet[100]) and int(wdet.sum()) <= 3
    torch.manual_seed(0)
    la = sm.LSTMAnomaly(12, 16).fit(base, epochs=80)
    sc = la.scores(spiked)
    assert int(sc.argmax()) in (100, 101) and bool(la.detect(spiked)[int(sc.argmax())])
    assert int(la.detect(base).sum()) <= 6

    # ---- container and validation splitters
    ts = sm.TimeSeries(torch.arange(10.0), torch.arange(10.0) * 30, frequency=1 / 30)
    r = ts.resample(60, "mean")
    assert len(r) == 5 and torch.allclose(r.values, torch.tensor([0.5, 2.5, 4.5, 6.5, 8.5], dtype=torch.float64))
    xi, yo = ts.windows(4, 2)
    assert xi.shape == (5, 4) and yo.shape == (5, 2) and float(yo[0, 0]) == 4
    assert torch.isnan(ts.lag(2).values[:2]).all() and float(ts.lag(2).values[2]) == 0 and len(ts.diff(2)) == 8
    a, b2 = ts.split(0.7)
    assert len(a) == 7 and len(b2) == 3
    for tr, te_ in sm.BlockedTimeSeriesCV(4, 0.25, gap=1).split(100):
        assert max(tr) + 1 < min(te_) and min(tr) // 25 == max(te_) // 25
    pcv = sm.PurgedTimeSeriesCV(5, label_horizon=3, embargo=4)
    for tr, te_ in pcv.split(100):
        lo, hi = te_[0], te_[-1] + 1
        assert not set(tr) & set(range(lo - 3, hi + 4)) and set(tr) | set(range(max(0, lo - 3), min(100, hi + 4))) == set(range(100))
    ccv = sm.CombinatorialPurgedCV(6, 2, label_horizon=1, embargo=1)
    splits = list(ccv.split(60))
    assert len(splits) == 15 and ccv.num_paths() == 5
    assert all(len(te_) == 20 and not set(tr) & set(te_) for tr, te_ in splits)
    ff = lambda tr, h, alpha: sm.SimpleExpSmoothing(alpha).fit(tr).forecast(h)
    walk = torch.randn(300, generator=g, dtype=torch.float64).cumsum(0)
    ramp = 0.5 * torch.arange(300, dtype=torch.float64) + 0.1 * torch.randn(300, generator=g, dtype=torch.float64)
    nested = sm.NestedTimeSeriesCV(3, 3).run(ramp, [0.05, 0.95], ff)
    assert nested["chosen"] == [0.95] * 3 and len(nested["scores"]) == 3         # a ramp wants the most recent level
    sc = sm.ScoredTimeSeriesCV(4).score(walk, lambda tr, h: tr[-1].repeat(h))
    assert len(sc["scores"]) == 4 and sc["std"] >= 0
    fm = sm.ForecastMetrics.compute(torch.tensor([1.0, 2, 3]), torch.tensor([1.0, 2, 4]))
    assert fm["mae"] == pytest.approx(1 / 3)


def test_cluster_estimators_match_sklearn_and_hdbscan_finds_varied_density_groups():
    import numpy as np
    from sklearn import cluster as skc
    from sklearn.metrics import adjusted_rand_score
    from torsh_b200 import cluster_models as cm

    g = torch.Generator().manual_seed(0)
    centres = torch.tensor([[0.0, 0], [6, 0], [0, 6], [6, 6]])
    x = torch.cat([c + 0.5 * torch.randn(80, 2, generator=g) for c in centres])
    truth = torch.arange(4).repeat_interleave(80)

    km = cm.KMeans(4, n_init=3, seed=0).fit(x)
    ref = skc.KMeans(4, n_init=3, random_state=0).fit(x.numpy())
    assert km.inertia_ == pytest.approx(ref.inertia_, rel=1e-4) and adjusted_rand_score(truth, km.labels_) == 1.0
    assert km.result.converged and km.result.n_iter < 30
    assert torch.equal(km.predict(x), km.labels_) and km.transform(x).shape == (320, 4)
    for init in ("forgy", "random_partition"):
        assert adjusted_rand_score(truth, cm.KMeans(4, init=init, n_init=6, seed=1).fit_predict(x)) == 1.0
    assert adjusted_rand_score(truth, cm.KMeans(4, distance="manhattan", seed=0).fit_predict(x)) == 1.0
    mb = cm.KMeans(4, batch_size=64, max_iter=200, n_init=2, seed=0).fit(x)
    assert adjusted_rand_score(truth, mb.labels_) > 0.95 and mb.inertia_ < 1.2 * ref.inertia_
    dirs = torch.nn.functional.normalize(torch.tensor([[1.0, 0, 0], [0, 1, 0], [0, 0, 1]]), dim=1)
    xs = torch.cat([(d + 0.1 * torch.randn(50, 3, generator=g)) * (1 + 5 * torch.rand(50, 1, generator=g)) for d in dirs])
    cos = cm.KMeans(3, distance="cosine", n_init=3, seed=0).fit(xs)
    assert adjusted_rand_score(torch.arange(3).repeat_interleave(50), cos.labels_) == 1.0            # scale does not matter
    assert torch.allclose(cos.cluster_centers_.norm(dim=1), torch.ones(3), atol=1e-5)
    one_chunk = cm.ChunkedDataProcessor(10 ** 6).assign(x, km.cluster_centers_)
    small = cm.ChunkedDataProcessor(37).assign(x, km.cluster_centers_)
    assert torch.equal(one_chunk[0], small[0]) and torch.allclose(one_chunk[1], small[1])
    sums, cnt = cm.ChunkedDataProcessor(37).reduce(x, km.labels_, 4)
    assert torch.allclose(sums / cnt[:, None], km.cluster_centers_, atol=1e-4)
    empty_seed = cm.KMeans(4, init="forgy", n_init=1, seed=0)
    empty_seed.fit(torch.cat([x, x[:1] + 100]))                                                        # an outlier cannot leave a cluster empty
    assert len(torch.unique(empty_seed.labels_)) == 4

    inc = cm.IncrementalCentroidUpdater(centres + 1.0)
    for lo in range(0, 320, 40):
        perm = torch.randperm(320, generator=g)[:40]
        inc.update(x[perm], truth[perm])
    assert float((inc.centres - centres).abs().max()) < 0.4 and float(inc.counts.sum()) == 320
    drift = cm.IncrementalCentroidUpdater(torch.zeros(1, 2), decay=0.5)
    for step in range(20):
        drift.update(torch.full((10, 2), float(step)), torch.zeros(10, dtype=torch.long))
    assert float(drift.centres[0, 0]) > 17.5                                                           # follows the stream

    # ---- DBSCAN: identical partition and noise set as scikit-learn
    moons_t = torch.linspace(0, math.pi, 150)
    moons = torch.cat([torch.stack([moons_t.cos(), moons_t.sin()], 1), torch.stack([1 - moons_t.cos(), 0.4 - moons_t.sin()], 1)]) + 0.04 * torch.randn(300, 2, generator=g)
    moons = torch.cat([moons, torch.tensor([[3.0, 3.0], [-2.0, -2.0]])])
    db = cm.DBSCAN(0.2, 5).fit(moons)
    sk = skc.DBSCAN(eps=0.2, min_samples=5).fit(moons.numpy())
    assert db.n_clusters_ == 2 and adjusted_rand_score(sk.labels_, db.labels_) == 1.0
    assert np.array_equal(db.labels_.numpy() == -1, sk.labels_ == -1) and np.array_equal(db.core_sample_indices_.numpy(), sk.core_sample_indices_)

    # ---- HDBSCAN: clusters of different density plus background noise
    dense = 0.15 * torch.randn(100, 2, generator=g)
    loose = torch.tensor([8.0, 0]) + 1.0 * torch.randn(100, 2, generator=g)
    mid = torch.tensor([0.0, 8]) + 0.4 * torch.randn(100, 2, generator=g)
    noise = torch.rand(20, 2, generator=g) * 30 - 10
    data = torch.cat([dense, loose, mid, noise])
    lab_true = torch.cat([torch.arange(3).repeat_interleave(100), torch.full((20,), -1)])
    hd = cm.HDBSCAN(min_cluster_size=15, min_samples=5).fit(data)
    assert hd.result.n_clusters == 3
    core_pts = hd.labels_[:300]
    assert adjusted_rand_score(lab_true[:300][core_pts >= 0], core_pts[core_pts >= 0]) == 1.0 and float((core_pts >= 0).float().mean()) > 0.9
    assert float((hd.labels_[300:] == -1).float().mean()) >= 0.6
    ref_h = skc.HDBSCAN(min_cluster_size=15, min_samples=5, copy=True).fit(data.numpy())
    assert adjusted_rand_score(ref_h.labels_, hd.labels_) > 0.95
    p = hd.probabilities_
    assert float(p.min()) >= 0 and float(p.max()) == 1.0 and float(p[hd.labels_ < 0].max()) == 0.0
    assert float(hd.result.outlier_scores[hd.labels_ < 0].min()) == 1.0 and len(hd.result.cluster_persistence) == 3
    blob = cm.HDBSCAN(10).fit(dense)
    assert blob.result.n_clusters == 0 and cm.HDBSCAN(10, allow_single_cluster=True).fit(dense).result.n_clusters == 1

    # ---- spectral clustering separates concentric rings that k-means cannot
    ang = torch.rand(300, generator=g) * 2 * math.pi
    rad = torch.cat([torch.full((150,), 1.0), torch.full((150,), 4.0)]) + 0.08 * torch.randn(300, generator=g)
    rings = torch.stack([rad * ang.cos(), rad * ang.sin()], 1)
    ring_truth = torch.arange(2).repeat_interleave(150)
    sp = cm.SpectralClustering(2, affinity="knn", n_neighbors=8).fit(rings)
    assert adjusted_rand_score(ring_truth, sp.labels_) == 1.0 and float(sp.eigenvalues_[1]) < 1e-10 < float(sp.eigenvalues_[2])
    assert adjusted_rand_score(ring_truth, cm.KMeans(2, seed=0).fit_predict(rings)) < 0.2
    blobs_sp = cm.SpectralClustering(4, "rbf", gamma=0.5).fit(x)
    assert adjusted_rand_score(truth, blobs_sp.labels_) == 1.0 and blobs_sp.eigengap(8) == 4

    gs = cm.GapStatistic(7, 6).fit(x)
    assert gs.optimal_k_ == 4 and len(gs.gaps_) == 7
    ev = cm.evaluate_clustering(data, hd.labels_, lab_true)
    assert ev.n_clusters == 3 and ev.silhouette > 0.6 and 0 < ev.noise_fraction < 0.15 and ev.external["ari"] > 0.9
    ph = cm.PageHinkleyTest()
    assert hasattr(ph, "update") or hasattr(ph, "add")


def test_advanced_graph_models_generative_quantum_spiking_operators_and_matching():
    from torch import nn
    from torsh_b200 import graph_advanced as ga
    from torsh_b200.graph import erdos_renyi, grid_graph, stochastic_block_model

    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)

    # ---- graph-level prediction: rings versus cliques; regression of edge count
    def ring(n): return torch.stack([torch.arange(n), (torch.arange(n) + 1) % n]).repeat(1, 1)
    def clique(n): return torch.tensor([[i, j] for i in range(n) for j in range(n) if i != j]).T
    def batchify(graphs):
        xs, eis, bs, off = [], [], [], 0
        for b, (n, ei) in enumerate(graphs):
            und = torch.cat([ei, ei.flip(0)], 1)
            deg = torch.bincount(und[0], minlength=n).float()
            xs.append(torch.stack([torch.ones(n), deg / 10], 1)); eis.append(und + off); bs.append(torch.full((n,), b)); off += n
        return torch.cat(xs), torch.cat(eis, 1), torch.cat(bs)
    graphs = [(n, ring(n)) for n in range(5, 11)] + [(n, clique(n)) for n in range(5, 11)]
    x, ei, batch = batchify(graphs)
    y = torch.tensor([0] * 6 + [1] * 6)
    for model in (ga.GraphClassificationGCN(2, 16, 2), ga.GraphClassificationGAT(2, 16, 2), ga.HierarchicalGraphClassifier(2, 16, 2)):
        opt = torch.optim.Adam(model.parameters(), 0.02)
        for _ in range(80):
            opt.zero_grad(); loss = nn.functional.cross_entropy(model(x, ei, batch), y); loss.backward(); opt.step()
        assert (model(x, ei, batch).argmax(1) == y).all(), type(model).__name__
    hier = ga.HierarchicalGraphClassifier(2, 8, 2, levels=2, ratio=0.5)
    hier(x, ei, batch)
    assert len(hier.kept[0]) == sum(math.ceil(n / 2) for n, _ in graphs) and len(hier.kept[1]) < len(hier.kept[0])
    reg = ga.GraphRegressor(2, 16)
    target = torch.tensor([[float(e.shape[1])] for _, e in graphs]) / 10
    opt = torch.optim.Adam(reg.parameters(), 0.01)
    for _ in range(300):
        opt.zero_grad(); loss = ((reg(x, ei, batch) - target) ** 2).mean(); loss.backward(); opt.step()
    assert float(loss) < 0.15 * float(target.var())
    mt = ga.MultiTaskGraphNetwork(2, 8, {"node_cls": ("node", 3), "graph_reg": ("graph", 1)})
    out = mt(x, ei, batch)
    assert out["node_cls"].shape == (len(x), 3) and out["graph_reg"].shape == (12, 1)
    total = mt.loss({"node_cls": torch.tensor(2.0), "graph_reg": torch.tensor(0.5)})
    assert float(total) == pytest.approx(2.5) and {n for n, _ in mt.named_parameters() if "log_vars" in n} == {"log_vars.node_cls", "log_vars.graph_reg"}

    # ---- VGAE recovers community structure; GAN statistics are permutation invariant
    sbm = stochastic_block_model((20, 20), 0.5, 0.02, feat=8, seed=0)
    vae = ga.GraphVAE(8, 16, 8)
    opt = torch.optim.Adam(vae.parameters(), 0.02)
    first = None
    for _ in range(150):
        opt.zero_grad(); loss = vae.loss(sbm.x, sbm.edge_index); loss.backward(); opt.step()
        first = first if first is not None else float(loss)
    vae.eval()
    logits, mu, _ = vae(sbm.x, sbm.edge_index)
    adj = ga.dense_adjacency(sbm.edge_index, 40)
    iu = torch.triu_indices(40, 40, 1)
    from torsh_b200.utils.metrics import roc_auc
    assert float(loss) < first and roc_auc(logits[iu[0], iu[1]].detach(), adj[iu[0], iu[1]]) > 0.85
    assert vae.sample(10).shape == (10, 10) and float(vae.sample(10).diagonal().sum()) == 0
    gan = ga.GraphGAN(8)
    fake = gan.generate(5)
    assert fake.shape == (5, 8, 8) and torch.allclose(fake, fake.transpose(1, 2)) and float(fake.diagonal(dim1=1, dim2=2).abs().sum()) == 0
    perm = torch.randperm(8, generator=g)
    assert torch.allclose(gan.statistics(fake), gan.statistics(fake[:, perm][:, :, perm]), atol=1e-6)
    tri = ga.dense_adjacency(clique(8), 8)[None]
    assert gan.statistics(tri)[0, 3] == pytest.approx(1.0) and gan.statistics(tri)[0, 4] == pytest.approx(1.0)
    d_loss, g_loss = gan.losses(torch.stack([ga.dense_adjacency(ring(8), 8)] * 4))
    d_loss.backward(); assert gan.disc[0].weight.grad is not None and float(g_loss) > 0
    cg = ga.ConditionalGraphGenerator(6, cond_dim=2)
    assert cg.generate_conditioned(torch.rand(3, 2)).shape == (3, 6, 6)

    # ---- discrete diffusion: marginals, posterior consistency, training signal
    diff = ga.DiscreteGraphDiffusion(steps=20, hidden=16, rho=0.2)
    a0 = ga.dense_adjacency(ring(12), 12)
    assert torch.allclose(diff.q_prob(a0, 19), torch.full_like(a0, 0.2), atol=0.1) and float(diff.q_prob(a0, 0)[0, 1]) > 0.99
    emp = torch.stack([diff.q_sample(a0, 10, g) for _ in range(300)]).mean(0)
    assert float((emp - diff.q_prob(a0, 10))[iu[0][:66] % 12, iu[1][:66] % 12].abs().mean()) < 0.06
    samp = diff.q_sample(a0, 5, g)
    assert torch.equal(samp, samp.T) and float(samp.diagonal().sum()) == 0
    # posterior marginalised over a_t must give back q(a_{t-1} | a_0)
    t = 7
    for a0v in (0.0, 1.0):
        p_t = diff.abar[t] * a0v + (1 - diff.abar[t]) * 0.2
        marg = p_t * diff.posterior(torch.ones(1), torch.tensor([a0v]), t) + (1 - p_t) * diff.posterior(torch.zeros(1), torch.tensor([a0v]), t)
        assert float(marg) == pytest.approx(float(diff.abar[t - 1] * a0v + (1 - diff.abar[t - 1]) * 0.2), abs=1e-6)
    opt = torch.optim.Adam(diff.parameters(), 0.01)
    losses = []
    for _ in range(60):
        opt.zero_grad(); l = diff.loss(a0, g); l.backward(); opt.step(); losses.append(float(l))
    assert sum(losses[-10:]) < sum(losses[:10])
    gen = diff.sample(12, g)
    assert gen.shape == (12, 12) and torch.equal(gen, gen.T) and set(gen.unique().tolist()) <= {0.0, 1.0}

    # ---- LRP conserves relevance; gradients identify the informative neighbour
    adj = ga.dense_adjacency(torch.tensor([[0, 1, 2], [1, 2, 3]]), 4, dtype=torch.float64)
    w = [torch.rand(3, 5, generator=g, dtype=torch.float64), torch.rand(5, 2, generator=g, dtype=torch.float64)]
    xin = torch.rand(4, 3, generator=g, dtype=torch.float64)
    lrp = ga.GraphLRP(w).explain(xin, adj, node=1, target=0)
    assert float(lrp["feature_relevance"].sum()) == pytest.approx(lrp["output"], rel=1e-6)
    assert float(lrp["node_relevance"][3]) > 0 and float(lrp["node_relevance"][1]) > float(lrp["node_relevance"][3])      # two hops reach node 3
    one_layer = ga.GraphLRP(w[:1]).explain(xin, adj, node=0, target=0)
    assert float(one_layer["node_relevance"][2].abs()) < 1e-15                                                         # one hop does not reach node 2
    lin = nn.Linear(3, 2).double()
    model = lambda xx, ee: ga.GraphLRP.a_hat(ga.dense_adjacency(ee, 4, dtype=torch.float64)) @ lin(xx)
    attr = ga.GraphGradientAttribution(model)
    e4 = torch.tensor([[0, 1, 2], [1, 2, 3]])
    ig = attr.integrated_gradients(xin, e4, 1, 0)
    assert float(ig.sum()) == pytest.approx(float(model(xin, e4)[1, 0] - model(torch.zeros_like(xin), e4)[1, 0]), abs=1e-9)
    assert float(attr.saliency(xin, e4, 0, 0)[3].sum()) == 0 and torch.allclose(attr.gradient_x_input(xin, e4, 1, 0), ig)
    dense_model = lambda xx, aa: ga.GraphLRP.a_hat(aa) @ lin(xx)
    imp = attr.edge_importance(dense_model, xin, adj, 0, 0)
    assert float(imp[0, 1]) > 0 and float(imp[2, 3]) == 0

    # ---- quantum walk and QAOA
    c4 = ga.dense_adjacency(ring(4), 4, dtype=torch.float64)
    qw = ga.QuantumWalk(c4)
    for tt in (0.3, 1.7):
        p = qw.probabilities(0, tt)
        assert float(p.sum()) == pytest.approx(1.0) and float(p[1]) == pytest.approx(float(p[3]))
    assert float(qw.probabilities(0, math.pi / 2)[2]) == pytest.approx(1.0, abs=1e-9)                                   # perfect transfer on the 4-cycle
    from scipy.linalg import expm
    assert torch.allclose(qw.evolve(0, 0.9), torch.from_numpy(expm(-1j * c4.numpy() * 0.9))[:, 0])
    assert qw.node_features([0.5, 1.0]).shape == (4, 2) and float(qw.average_distribution(0, 20.0).sum()) == pytest.approx(1.0)
    qaoa = ga.QuantumQAOA(ring(4), 4, depth=2)
    assert qaoa.max_cut() == 4.0 and float(qaoa.state().abs().pow(2).sum()) == pytest.approx(1.0)
    before = float(qaoa())
    after = qaoa.optimize(120, 0.05)
    bits, cut = qaoa.best_assignment()
    assert after > before and after > 3.5 and cut == 4.0 and bits.tolist() in ([0, 1, 0, 1], [1, 0, 1, 0])
    p1 = ga.QuantumQAOA(torch.tensor([[0], [1]]), 2, depth=1)
    with torch.no_grad():
        p1.gamma.fill_(math.pi / 2); p1.beta.fill_(math.pi / 8)
    assert float(p1()) == pytest.approx(1.0, abs=1e-9)                                                                  # single edge: depth one reaches the optimum
    with pytest.raises(ValueError):
        ga.QuantumQAOA(ring(17), 17)
    ql = ga.QuantumGraphLayer(3, 5)
    out = ql(torch.rand(4, 3), c4.float())
    out.sum().backward()
    assert out.shape == (4, 5) and ql.times.grad is not None

    # ---- spiking network trains; liquid state machine remembers
    sbm2 = stochastic_block_model((15, 15), 0.5, 0.03, feat=6, seed=1)
    adj2 = ga.dense_adjacency(sbm2.edge_index, 30)
    snn = ga.SpikingGraphNetwork(6, 16, 2, steps=10)
    opt = torch.optim.Adam(snn.parameters(), 0.02)
    for _ in range(60):
        opt.zero_grad(); loss = nn.functional.cross_entropy(snn(sbm2.x, adj2), sbm2.y); loss.backward(); opt.step()
    assert float((snn(sbm2.x, adj2).argmax(1) == sbm2.y).float().mean()) > 0.9
    assert 0 <= float(snn.spike_rate.min()) and float(snn.spike_rate.max()) <= 1 and 0 < float(snn.spike_rate.mean()) < 1
    res_adj = (torch.rand(60, 60, generator=g) < 0.1).double()
    lsm = ga.LiquidStateMachine(res_adj, 1, spectral_radius=0.9, leak=0.5)
    u = torch.rand(600, 1, generator=g) - 0.5
    delayed = torch.roll(u, 2, 0)
    lsm.fit(u[:400], delayed[:400])
    pred = lsm.predict(u)[420:]
    assert float(((pred - delayed[420:]) ** 2).mean()) < 0.3 * float(delayed.var())
    assert float(torch.linalg.eigvals(lsm.w).abs().max()) == pytest.approx(0.9, rel=1e-6)

    # ---- operators
    grid = grid_graph(8, 8)
    gadj = ga.dense_adjacency(grid, 64)
    lap = ga.normalized_laplacian(gadj)
    fno = ga.GraphFNO(1, 16, 1, modes=12, layers=2)
    basis = fno.basis(gadj)
    assert torch.allclose(basis.T @ basis, torch.eye(12), atol=1e-4)
    heat = torch.matrix_exp(-2.0 * lap)
    u0 = torch.randn(40, 64, generator=g) @ basis @ basis.T
    opt = torch.optim.Adam(fno.parameters(), 0.01)
    for _ in range(150):
        opt.zero_grad(); loss = sum(((fno(v[:, None], gadj, basis)[:, 0] - heat @ v) ** 2).mean() for v in u0[:8]) / 8; loss.backward(); opt.step()
    test_err = float(((fno(u0[20][:, None], gadj, basis)[:, 0] - heat @ u0[20]) ** 2).mean() / (heat @ u0[20]).pow(2).mean())
    assert test_err < 0.2
    coords = torch.stack(torch.meshgrid(torch.linspace(0, 1, 8), torch.linspace(0, 1, 8), indexing="ij"), -1).reshape(64, 2)
    don = ga.GraphDeepONet(64, 2, 32, 16)
    assert don(u0[:5], coords).shape == (5, 64)
    opt = torch.optim.Adam(don.parameters(), 0.01)
    start = None
    for _ in range(100):
        opt.zero_grad(); loss = ((don(u0[:30], coords) - u0[:30] @ heat.T) ** 2).mean(); loss.backward(); opt.step()
        start = start if start is not None else float(loss)
    assert float(loss) < 0.5 * start
    pinn = ga.PhysicsInformedGNN(16, dt=0.1)
    u_now = torch.randn(64, generator=g)
    u_next = u_now - 0.1 * 1.5 * (lap @ u_now)                                                                       # explicit Euler with kappa = 1.5
    assert float(pinn.residual(u_now, u_next, lap).abs().max()) > 1e-3
    with torch.no_grad():
        pinn.log_kappa.fill_(math.log(1.5))
    assert float(pinn.residual(u_now, u_next, lap).abs().max()) < 1e-5
    pinn.loss(u_now, u_next, grid, lap).backward()
    assert pinn.log_kappa.grad is not None

    # ---- barycentre and matching
    def sp(adj):
        d = torch.where(adj > 0, torch.ones_like(adj), torch.full_like(adj, 99.0)).fill_diagonal_(0)
        for k in range(len(adj)):
            d = torch.minimum(d, d[:, k:k + 1] + d[k:k + 1])
        return d.double()
    r6 = sp(ga.dense_adjacency(ring(6), 6))
    bary = ga.GraphBarycenter(6, iters=8, reg=0.05).fit([r6, r6[torch.randperm(6, generator=g)][:, torch.randperm(6, generator=g)] * 0 + r6])
    assert bary.shape == (6, 6) and torch.allclose(bary, bary.T, atol=1e-8)
    assert sorted(round(v, 1) for v in torch.linalg.eigvalsh(bary).tolist())[-1] == pytest.approx(sorted(torch.linalg.eigvalsh(r6).tolist())[-1], rel=0.15)
    sia = ga.SiameseGraphNetwork(2, 8)
    xr, eir, _ = batchify([(6, ring(6))]); xc, eic, _ = batchify([(6, clique(6))])
    permn = torch.randperm(6, generator=g)
    inv = torch.argsort(permn)
    assert float(sia((xr, eir), (xr[permn], inv[eir]))) == pytest.approx(1.0, abs=1e-5)                                 # isomorphic copies embed identically
    assert float(sia.contrastive_loss((xr, eir), (xr, eir), True)) < 1e-8
    gmn = ga.GraphMatchingNetwork(2, 8, 2)
    same = gmn((xr, eir), (xr, eir)); diff_ = gmn((xr, eir), (xc, eic))
    assert float(same) == pytest.approx(0.0, abs=1e-8) and float(diff_) < float(same) and gmn.attention.shape == (6, 6)

    # ---- foundation model and modalities
    fm = ga.GraphFoundationModel(8, 16, 2).add_head("cls", "node", 2).add_head("link", "link").add_head("prop", "regression", 1)
    pl = fm.pretrain_loss(sbm.x, sbm.edge_index, 0.2, g)
    assert set(pl) == {"masked_features", "structure", "total"} and float(pl["total"]) == pytest.approx(float(pl["masked_features"] + pl["structure"]))
    pl["total"].backward()
    assert fm.mask_token.grad is not None
    assert fm("cls", sbm.x, sbm.edge_index).shape == (40, 2) and fm("link", sbm.x, sbm.edge_index, pairs=sbm.edge_index[:, :7]).shape == (7,)
    assert fm("prop", sbm.x, sbm.edge_index).shape == (1, 1)
    fm.freeze_encoder()
    assert not any(p.requires_grad for p in fm.encoder.parameters()) and all(p.requires_grad for p in fm.heads.parameters())
    feats = {"text": torch.randn(5, 12), "image": torch.randn(5, 20), "audio": torch.randn(5, 6)}
    path = ga.dense_adjacency(torch.tensor([[0, 1, 2, 3], [1, 2, 3, 4]]), 5)
    cma = ga.CrossModalGraphAttention({"text": 12, "image": 20, "audio": 6}, 16, 4)
    o1 = cma(feats, path)
    feats2 = {k: v.clone() for k, v in feats.items()}
    feats2["image"][4] += 10.0                                                                                        # node 4 is not adjacent to node 0
    o2 = cma(feats2, path)
    assert o1["text"].shape == (5, 16) and torch.allclose(o1["text"][0], o2["text"][0], atol=1e-6) and not torch.allclose(o1["text"][3], o2["text"][3])
    for mode in ("gated", "concat", "bilinear"):
        assert ga.MultiModalFusion({"text": 12, "image": 20, "audio": 6}, 10, mode)(feats).shape == (5, 10)
    fus = ga.MultiModalFusion({"text": 12, "image": 20, "audio": 6}, 10, "gated")
    fus({"text": feats["text"], "image": None, "audio": feats["audio"]})
    assert set(fus.last_gates) == {"text", "audio"} and torch.allclose(fus.last_gates["text"] + fus.last_gates["audio"], torch.ones(5))


def test_vision_geometry_hough_binary_features_alignment_pose_and_efficientnet_v2():
    from torch import nn
    from torsh_b200.vision import geometry as vg
    from torsh_b200.vision import ops as V

    g = torch.Generator().manual_seed(0)
    # ---- Hough lines: a horizontal and a diagonal line
    img = torch.zeros(100, 120)
    img[30, 10:110] = 1
    for i in range(80):
        img[10 + i, 20 + i] = 1
    lines = vg.hough_lines(img, max_lines=2)
    assert len(lines) == 2
    horiz = min(lines, key=lambda l: abs(l.theta - math.pi / 2))
    diag = min(lines, key=lambda l: abs(l.theta - 3 * math.pi / 4))
    assert horiz.rho == pytest.approx(30, abs=1.5) and horiz.theta == pytest.approx(math.pi / 2, abs=0.02) and horiz.votes >= 95
    assert diag.theta == pytest.approx(3 * math.pi / 4, abs=0.02) and abs(diag.rho - (20 * math.cos(diag.theta) + 10 * math.sin(diag.theta))) < 1.5
    # ---- Hough circles
    yy, xx = torch.meshgrid(torch.arange(100.0), torch.arange(120.0), indexing="ij")
    ring = lambda cx, cy, r: ((torch.hypot(xx - cx, yy - cy) - r).abs() < 0.6).float()
    edges = torch.maximum(ring(40, 50, 20), ring(85, 40, 12))
    circles = vg.hough_circles(edges, radii=range(10, 24, 2), max_circles=2)
    found = sorted((c.cx, c.cy, c.radius) for c in circles)
    assert len(found) == 2 and abs(found[0][0] - 40) <= 1 and abs(found[0][1] - 50) <= 1 and found[0][2] == 20 and abs(found[1][0] - 85) <= 1 and found[1][2] == 12

    # ---- binary descriptors: match a translated copy; orientation makes them survive a rotation
    base = V.gaussian_blur(torch.rand(1, 160, 160, generator=g), 1.5)[0]
    kps = torch.stack([torch.randint(40, 120, (40,), generator=g), torch.randint(40, 120, (40,), generator=g)], 1)
    shifted = torch.roll(base, (7, -5), (0, 1))
    d1 = vg.brief_descriptors(base, kps)
    d2 = vg.brief_descriptors(shifted, kps + torch.tensor([-5, 7]))
    assert d1.shape == (40, 32) and d1.dtype == torch.uint8
    hd = vg.hamming_distance(d1, d2)
    assert hd.shape == (40, 40) and int(hd.diagonal().max()) == 0 and float(hd[~torch.eye(40, dtype=torch.bool)].float().mean()) > 90
    ref_pop = sum(bin(int(a) ^ int(b)).count("1") for a, b in zip(d1[0].tolist(), d1[1].tolist()))
    assert int(vg.hamming_distance(d1[:1], d1[1:2])) == ref_pop
    noisy = shifted + 0.02 * torch.randn(160, 160, generator=g)
    matches = vg.BruteForceMatcher(0.8).match(d1, vg.brief_descriptors(noisy, kps + torch.tensor([-5, 7])))
    assert len(matches) >= 30 and all(m.query == m.train for m in matches)
    rot90 = torch.rot90(base, 1, (0, 1))                                                   # (x, y) -> (y, 159 - x)
    kps_r = torch.stack([kps[:, 1], 159 - kps[:, 0]], 1)
    plain = vg.hamming_distance(d1, vg.brief_descriptors(rot90, kps_r)).diagonal().float().mean()
    orient = vg.hamming_distance(vg.brief_descriptors(base, kps, oriented=True), vg.brief_descriptors(rot90, kps_r, oriented=True)).diagonal().float().mean()
    assert float(orient) < 0.35 * float(plain)
    fl = vg.BruteForceMatcher(0.9, cross_check=False).match(torch.tensor([[0.0, 0], [5, 5]]), torch.tensor([[5.1, 5], [0, 0.1], [9, 9]]))
    assert [(m.query, m.train) for m in fl] == [(0, 1), (1, 0)]

    # ---- Kabsch, ICP
    ang = 0.4
    R = torch.tensor([[math.cos(ang), -math.sin(ang), 0], [math.sin(ang), math.cos(ang), 0], [0, 0, 1]], dtype=torch.float64)
    pts = torch.randn(200, 3, generator=g, dtype=torch.float64)
    t = torch.tensor([0.5, -1.0, 2.0], dtype=torch.float64)
    Rk, tk, sk = vg.kabsch(pts, 1.7 * pts @ R.T + t, with_scale=True)
    assert torch.allclose(Rk, R, atol=1e-9) and torch.allclose(tk, t, atol=1e-9) and float(sk) == pytest.approx(1.7)
    mirrored = pts * torch.tensor([1.0, 1.0, -1.0], dtype=torch.float64)
    assert float(torch.linalg.det(vg.kabsch(pts, mirrored)[0])) == pytest.approx(1.0)         # never a reflection
    small = 0.15
    Rs = torch.tensor([[math.cos(small), -math.sin(small), 0], [math.sin(small), math.cos(small), 0], [0, 0, 1]], dtype=torch.float64)
    target = pts @ Rs.T + torch.tensor([0.1, 0.05, -0.1], dtype=torch.float64)
    Ri, ti, hist = vg.icp(pts, target[torch.randperm(200, generator=g)])
    assert torch.allclose(Ri, Rs, atol=1e-6) and hist[-1] < 1e-6 and hist[0] > hist[-1]
    Rp, tp, hp = vg.icp(pts[:150], target, trim=0.9)
    assert torch.allclose(Rp, Rs, atol=1e-3)

    # ---- intensity registration recovers a known affine warp
    smooth = V.gaussian_blur(torch.rand(1, 96, 96, generator=g), 4.0)[0].double()
    smooth = (smooth - smooth.min()) / (smooth.max() - smooth.min())
    p_true = torch.tensor([0.03, -0.02, 0.02, 0.01, 2.5, -1.5], dtype=torch.float64)
    fixed = vg.ImageRegistrar._warp(smooth, p_true)
    reg = vg.ImageRegistrar("affine", levels=3, iters=40).register(fixed, smooth)
    assert reg["rmse"] < 0.01 and reg["rmse"] < 0.2 * float((smooth - fixed).pow(2).mean().sqrt())
    assert torch.allclose(reg["matrix"], torch.tensor([[1.03, 0.02, 2.5], [-0.02, 1.01, -1.5]], dtype=torch.float64), atol=0.05)
    shift_only = vg.ImageRegistrar._warp(smooth, torch.tensor([0, 0, 0, 0, 3.0, -2.0], dtype=torch.float64))
    tr = vg.ImageRegistrar("translation", levels=2).register(shift_only, smooth)
    assert float(tr["matrix"][0, 2]) == pytest.approx(3.0, abs=0.3) and float(tr["matrix"][1, 2]) == pytest.approx(-2.0, abs=0.3)

    # ---- camera pose
    K = torch.tensor([[800.0, 0, 320], [0, 800, 240], [0, 0, 1]])
    pe = vg.PoseEstimator(K)
    world = torch.rand(30, 3, generator=g, dtype=torch.float64) * 2 - 1
    tc = torch.tensor([0.2, -0.1, 6.0], dtype=torch.float64)
    uv = pe.project(world, R, tc)
    est = pe.estimate(world, uv)
    assert torch.allclose(est["rotation"], R, atol=1e-6) and torch.allclose(est["translation"], tc, atol=1e-5) and est["reprojection_error"] < 1e-6
    noisy_est = pe.estimate(world, uv + 0.5 * torch.randn(30, 2, generator=g, dtype=torch.float64))
    assert noisy_est["reprojection_error"] < 2.0 and float((noisy_est["translation"] - tc).norm()) < 0.3

    # ---- EfficientNetV2
    net = vg.EfficientNetV2(10, "tiny", drop_path=0.1, head_dim=64)
    out = net(torch.randn(2, 3, 64, 64, generator=g))
    out.sum().backward()
    assert out.shape == (2, 10) and net.features[0].weight.grad is not None
    full = vg.EfficientNetV2(1000, "s")
    n_params = sum(p.numel() for p in full.parameters())
    assert 20.5e6 < n_params < 22.5e6
    fused, classic = vg.FusedMBConv(24, 24, 4, 1, True), vg.FusedMBConv(24, 24, 4, 1, False)
    assert not any(isinstance(m, nn.Conv2d) and m.groups > 1 for m in fused.modules()) and any(isinstance(m, nn.Conv2d) and m.groups > 1 for m in classic.modules())
    fused.eval()
    xin = torch.randn(1, 24, 8, 8, generator=g)
    assert fused.residual and fused(xin).shape == xin.shape and not vg.FusedMBConv(24, 48, 4, 2).residual

    # ---- transforms and registry
    rgb = torch.rand(3, 16, 16, generator=g)
    assert vg.Grayscale()(rgb).shape == (1, 16, 16) and vg.Grayscale(3)(rgb).shape == (3, 16, 16)
    assert torch.equal(vg.RandomGrayscale(0.0)(rgb), rgb) and torch.allclose(vg.RandomGrayscale(1.0)(rgb)[0], vg.RandomGrayscale(1.0)(rgb)[2])
    assert float(vg.GaussianBlur(2.0)(rgb).std()) < float(rgb.std()) and torch.equal(vg.GaussianBlur(2.0, p=0.0)(rgb), rgb)
    sol = vg.Solarize(0.5)(rgb)
    assert torch.equal(sol[rgb < 0.5], rgb[rgb < 0.5]) and torch.allclose(sol[rgb >= 0.5], 1 - rgb[rgb >= 0.5])
    assert vg.Pad(2)(rgb).shape == (3, 20, 20) and vg.Pad((1, 3))(rgb).shape == (3, 22, 18)
    assert torch.allclose(vg.Rotation(0.0)(rgb), rgb, atol=1e-5)
    rr = vg.RandomRotation(30, seed=0)
    rr(rgb)
    assert -30 <= rr.last_angle <= 30
    mu = vg.MixUp(0.4, 5, seed=0)
    xb, yb = torch.rand(8, 3, 4, 4, generator=g), torch.randint(0, 5, (8,), generator=g)
    xm, ym = mu(xb, yb)
    assert xm.shape == xb.shape and torch.allclose(ym.sum(1), torch.ones(8)) and 0 <= mu.last_lambda <= 1
    regy = vg.TransformRegistry()
    pipe = regy.build([{"name": "GaussianBlur", "sigma": 1.0}, "Grayscale", {"name": "Pad", "padding": 1}])
    assert pipe(rgb).shape == (1, 18, 18) and len(pipe.steps) == 3 and "Solarize" in regy.names()
    regy.register("Invert", lambda: (lambda v: 1 - v))
    assert torch.allclose(regy.create("Invert")(rgb), 1 - rgb)
    with pytest.raises(KeyError):
        regy.create("Nope")

    # ---- cache, prefetcher, batch loader
    loads = []
    def loader(k):
        loads.append(k)
        return torch.full((3, 8 + k % 2, 8), float(k))
    cache = vg.ImageCache(capacity_bytes=3 * 3 * 9 * 8 * 4)
    for k in (0, 1, 0, 2, 3, 0):
        cache.get(k, lambda k=k: loader(k))
    assert loads == [0, 1, 2, 3] and cache.hit_rate() == pytest.approx(2 / 6) and 1 not in cache.data and cache.used <= cache.cap
    order = [k for k, _ in vg.ImagePrefetcher(range(10), lambda k: torch.tensor(k), depth=3)]
    assert order == list(range(10))
    bl = vg.BatchImageLoader(range(7), loader, batch_size=3, size=(8, 8), cache=vg.ImageCache())
    batches = list(bl)
    assert [b.shape for b in batches] == [(3, 3, 8, 8), (3, 3, 8, 8), (1, 3, 8, 8)] and len(bl) == 3 and float(batches[1][0].mean()) == pytest.approx(3.0)
