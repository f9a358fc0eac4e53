"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6)).item()


def _rel_elem(a, b):
    """Element-wise criterion: the largest |a - b| / (|b| + rms(b)) over all elements, so a single wrong element in a
    small-magnitude position cannot hide behind the tensor's largest value."""
    a, b = a.float(), b.float()
    rms = b.pow(2).mean().sqrt().clamp(min=1e-6)
    return ((a - b).abs() / (b.abs() + rms)).max().item()


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("am,bm", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (384, 640, 320), (200, 328, 136), (1024, 1024, 512)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_majors(am, bm, shape, bn):
    from torsh_b200.ops.gemm import gemm
    M, N, K = shape
    torch.manual_seed(1)
    a = torch.randn((M, K) if am == 0 else (K, M), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((N, K) if bm == 0 else (K, N), device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, a_major=am, b_major=bm, bn=bn)
    A = a.float() if am == 0 else a.float().t()
    B = b.float() if bm == 0 else b.float().t()
    assert _rel_elem(out, A @ B.t()) < 1e-2


def test_gemm_dynamic_tile_scheduler():
    """The opt-in dynamic tile scheduler (work items drawn from a device counter) gives the same product as the static
    deal, launch after launch (the counters reset themselves)."""
    from torsh_b200 import _native as nv
    from torsh_b200.ops.gemm import gemm
    torch.manual_seed(3)
    M, N, K = 8192, 4096, 512          # 32 x 16 tiles of 256 x 256: more than one wave on 148 SMs
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    ref = gemm(a, b)
    was = nv.cuda().tb_gemm_set_dynamic(1)
    try:
        for _ in range(3):
            out = gemm(a, b)
            assert torch.equal(out, ref)
    finally:
        nv.cuda().tb_gemm_set_dynamic(was)
    assert _rel_elem(ref, a.float() @ b.float().t()) < 1e-2


def test_gemm_epilogues():
    from torsh_b200.ops.gemm import gemm
    torch.manual_seed(2)
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = gemm(a, b, bias=bias, gelu=True, residual=res, preact_out=pre)
    u = a.float() @ b.float().t() + bias.float()
    ref = torch.nn.functional.gelu(u, approximate="tanh") + res.float()
    assert _rel_elem(out, ref) < 1e-2 and _rel_elem(pre, u) < 1e-2
    out2 = gemm(a, b, dgelu_aux=pre)
    uu = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(uu, approximate="tanh").sum().backward()
    assert _rel_elem(out2, (a.float() @ b.float().t()) * uu.grad) < 1e-2
    # ragged N (scalar epilogue path) and fp32 accumulate
    b3 = torch.randn(100, K, device=DEV, dtype=torch.bfloat16)
    o3 = torch.ones(M, 100, device=DEV, dtype=torch.float32)
    gemm(a, b3, out=o3, accumulate=True)
    assert _rel_elem(o3, a.float() @ b3.float().t() + 1.0) < 1e-2


def test_gemm_splitk_atomic_wgrad():
    from torsh_b200.ops.gemm import gemm
    torch.manual_seed(3)
    T = 4096
    dy = torch.randn(T, 512, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(T, 384, device=DEV, dtype=torch.bfloat16)
    g = torch.zeros(512, 384, device=DEV, dtype=torch.float32)
    gemm(dy, x, a_major=1, b_major=1, out=g, atomic=True, split_k=8)
    gemm(dy, x, a_major=1, b_major=1, out=g, atomic=True, split_k=8)
    assert _rel_elem(g, 2 * dy.float().t() @ x.float()) < 1e-4


@pytest.mark.parametrize("shape", [(512, 384, 4096), (4096, 1024, 8192), (1024, 1024, 8192), (200, 72, 1000), (50304, 1024, 2048)])
@pytest.mark.parametrize("majors", [(1, 1), (0, 0)])
def test_gemm_stream_k_matches_fp32(shape, majors):
    """split_k=-1: equal K-block ranges per CTA, pieces of a tile meet through fp32 atomics (and a bias enters once)."""
    from torsh_b200.ops.gemm import gemm
    torch.manual_seed(7)
    M, N, K = shape
    am, bm = majors
    a = torch.randn((K, M) if am else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if bm else (N, K), device=DEV, dtype=torch.bfloat16)
    ref = (a.float().t() if am else a.float()) @ (b.float() if bm else b.float().t())
    g = torch.ones(M, N, device=DEV, dtype=torch.float32)
    gemm(a, b, a_major=am, b_major=bm, out=g, atomic=True, split_k=-1)
    assert _rel_elem(g, ref + 1.0) < 1e-4
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    g.zero_()
    gemm(a, b, a_major=am, b_major=bm, out=g, atomic=True, split_k=-1, bias=bias)
    assert _rel_elem(g, ref + bias.float()) < 1e-4


# ------------------------------------------------------------------ norms
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H", [256, 1024, 4096])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(dtype, H, rms):
    from torsh_b200.ops.norm import layer_norm, rms_norm
    torch.manual_seed(4)
    rows = 333
    x = torch.randn(rows, H, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(H, device=DEV) * 0.2 + 1).to(dtype).requires_grad_(True)
    b = None if rms else (torch.randn(H, device=DEV) * 0.1).to(dtype).requires_grad_(True)
    dy = torch.randn(rows, H, device=DEV, dtype=dtype)
    y = rms_norm(x, w, 1e-6) if rms else layer_norm(x, w, b, 1e-5)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    if rms:
        yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    else:
        bf = b.detach().float().requires_grad_(True)
        yr = torch.nn.functional.layer_norm(xf, (H,), wf, bf, 1e-5)
    yr.backward(dy.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel(y, yr) < tol and _rel(x.grad, xf.grad) < tol and _rel(w.grad, wf.grad) < tol
    if not rms:
        assert _rel(b.grad, bf.grad) < tol


# ------------------------------------------------------------------ softmax / cross-entropy
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("C", [1000, 4097, 50304])
def test_softmax_and_log_softmax(dtype, C):
    from torsh_b200.ops.softmax import log_softmax, softmax
    torch.manual_seed(5)
    x = (torch.randn(37, C, device=DEV) * 3).to(dtype).requires_grad_(True)
    dy = torch.randn(37, C, device=DEV, dtype=dtype)
    for fn, ref in ((softmax, torch.softmax), (log_softmax, torch.log_softmax)):
        x.grad = None
        y = fn(x, -1)
        y.backward(dy)
        xf = x.detach().float().requires_grad_(True)
        yr = ref(xf, -1)
        yr.backward(dy.float())
        tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
        assert _rel(y, yr) < tol and _rel(x.grad, xf.grad) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy_padded_vocab(dtype):
    from torsh_b200.ops.softmax import cross_entropy
    torch.manual_seed(6)
    rows, V, Vp = 256, 50257, 50304
    lg = (torch.randn(rows, Vp, device=DEV) * 2).to(dtype).requires_grad_(True)
    tg = torch.randint(0, V, (rows,), device=DEV)
    tg[5] = -100
    loss = cross_entropy(lg, tg, num_classes=V)
    loss.backward()
    lf = lg.detach().float()[:, :V].requires_grad_(True)
    lr = torch.nn.functional.cross_entropy(lf, tg, ignore_index=-100)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-3 * abs(lr.item())
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel(lg.grad[:, :V], lf.grad) < tol
    assert lg.grad[:, V:].abs().max().item() == 0.0
    # fused-backward contract
    lg2 = lg.detach().clone().requires_grad_(True)
    tg2 = tg.clone()
    tg2[5] = 7
    l2 = cross_entropy(lg2, tg2, num_classes=V, root_scale=0.5)
    l2.backward()
    lf2 = lg.detach().float()[:, :V].requires_grad_(True)
    (0.5 * torch.nn.functional.cross_entropy(lf2, tg2)).backward()
    assert _rel(lg2.grad[:, :V], lf2.grad) < tol


# ------------------------------------------------------------------ elementwise / reduce / embedding / rope
def test_unary_binary_reduce():
    from torsh_b200.ops import elementwise as ew
    torch.manual_seed(7)
    for dtype in (torch.bfloat16, torch.float32):
        x = torch.randn(1000, 77, device=DEV, dtype=dtype)
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        for op, ref in ew._TORCH_UNARY.items():
            xi = x.abs() + 0.1 if op in ("log", "sqrt", "rsqrt") else x
            assert _rel(ew.unary_raw(op, xi), ref(xi.float())) < tol, op
        y = torch.randn_like(x)
        for op, ref in ew._TORCH_BINARY.items():
            yi = y.abs() + 0.5 if op == "div" else y
            assert _rel(ew.binary_raw(op, x, yi), ref(x.float(), yi.float())) < tol, op
        assert _rel(ew.binary_raw("mul", x, 2.5), x.float() * 2.5) < tol
        x3 = torch.randn(6, 130, 50, device=DEV, dtype=dtype)
        for dim in (0, 1, 2):
            for op in ("sum", "max", "min", "mean"):
                r = getattr(x3.float(), op)(dim)
                r = r.values if op in ("max", "min") else r
                assert _rel(ew.reduce(op, x3, dim), r) < (3e-2 if dtype == torch.bfloat16 else 1e-4), (op, dim)


def test_activation_grads_swiglu_rope_embedding():
    from torsh_b200.ops import elementwise as ew
    torch.manual_seed(8)
    x = torch.randn(64, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(64, 512, device=DEV, dtype=torch.bfloat16)
    for fn, ref in ((ew.gelu, lambda t: torch.nn.functional.gelu(t, approximate="tanh")), (ew.silu, torch.nn.functional.silu),
                    (ew.relu, torch.relu), (ew.tanh, torch.tanh), (ew.sigmoid, torch.sigmoid)):
        x.grad = None
        fn(x).backward(dy)
        xf = x.detach().float().requires_grad_(True)
        ref(xf).backward(dy.float())
        assert _rel(x.grad, xf.grad) < 3e-2
    x.grad = None
    y = ew.swiglu(x)
    y.backward(dy[:, :256])
    xf = x.detach().float().requires_grad_(True)
    yr = xf[:, :256] * torch.nn.functional.silu(xf[:, 256:])
    yr.backward(dy[:, :256].float())
    assert _rel(y, yr) < 2e-2 and _rel(x.grad, xf.grad) < 3e-2
    q = torch.randn(2, 100, 4, 128, device=DEV, dtype=torch.float32, requires_grad=True)
    r = ew.rope(q, 10000.0)
    assert _rel(r, ew._rope_torch(q.detach(), 10000.0, 0, False)) < 1e-4
    r.backward(torch.ones_like(r))
    assert _rel(q.grad, ew._rope_torch(torch.ones_like(q), 10000.0, 0, True)) < 1e-4
    wte = torch.randn(500, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    wpe = torch.randn(32, 64, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 500, (4, 32), device=DEV)
    e = ew.embedding(ids, wte, wpe)
    ref = wte.detach().float()[ids] + wpe.detach().float()[None]
    assert _rel(e, ref) < 1e-2
    e.backward(torch.ones_like(e))
    cnt = torch.bincount(ids.reshape(-1), minlength=500).float()
    assert _rel(wte.grad[:, 0], cnt) < 1e-2 and _rel(wpe.grad, torch.full_like(wpe, 4.0)) < 1e-2


# ------------------------------------------------------------------ linear / MLP autograd
def test_linear_and_mlp_autograd():
    from torsh_b200.ops.linear import linear, mlp_gelu
    torch.manual_seed(9)
    x = torch.randn(4, 96, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    for layout in ("nk", "kn"):
        w = (torch.randn((384, 256) if layout == "nk" else (256, 384), device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
        b = torch.randn(384, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        x.grad = None
        y = linear(x, w, b, layout=layout)
        dy = torch.randn_like(y)
        y.backward(dy)
        xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
        yr = torch.nn.functional.linear(xf, wf if layout == "nk" else wf.t(), bf)
        yr.backward(dy.float())
        assert _rel(y, yr) < 1e-2 and _rel(x.grad, xf.grad) < 1e-2 and _rel(w.grad, wf.grad) < 1e-2 and _rel(b.grad, bf.grad) < 1e-2
    w1 = (torch.randn(1024, 256, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
    b1 = torch.randn(1024, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w2 = (torch.randn(256, 1024, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
    b2 = torch.randn(256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    x.grad = None
    y = mlp_gelu(x, w1, b1, w2, b2, residual=x)
    dy = torch.randn_like(y)
    y.backward(dy)
    fs = [t.detach().float().requires_grad_(True) for t in (x, w1, b1, w2, b2)]
    yr = torch.nn.functional.linear(torch.nn.functional.gelu(torch.nn.functional.linear(fs[0], fs[1], fs[2]), approximate="tanh"), fs[3], fs[4]) + fs[0]
    yr.backward(dy.float())
    assert _rel(y, yr) < 2e-2
    for got, ref in zip((x, w1, b1, w2, b2), fs):
        assert _rel(got.grad, ref.grad) < 3e-2
    # main_grad accumulation path
    w = (torch.randn(384, 256, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
    w.main_grad = torch.zeros(384, 256, device=DEV, dtype=torch.float32)
    y = linear(x, w, None)
    y.backward(torch.ones_like(y))
    assert w.grad is None
    ref = torch.ones(4 * 96, 384, device=DEV).t() @ x.detach().float().reshape(-1, 256)
    assert _rel(w.main_grad, ref) < 1e-3


# ------------------------------------------------------------------ attention
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("S", [128, 384, 200])
def test_flash_attention_fwd_bwd(D, causal, S):
    from torsh_b200.ops.attention import _sdpa_reference, flash_attention
    torch.manual_seed(10)
    B, H = 2, 3
    q, k, v = (torch.randn(B, S, H, D, device=DEV, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    o = flash_attention(q, k, v, causal=causal)
    do = torch.randn_like(o)
    o.backward(do)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    orf = _sdpa_reference(qf, kf, vf, causal, 1.0 / math.sqrt(D))
    orf.backward(do.float())
    assert _rel(o, orf) < 2e-2
    assert _rel(q.grad, qf.grad) < 3e-2 and _rel(k.grad, kf.grad) < 3e-2 and _rel(v.grad, vf.grad) < 3e-2


def test_flash_attention_qkvpacked():
    from torsh_b200.ops.attention import _sdpa_reference, flash_attention_qkvpacked
    torch.manual_seed(11)
    B, S, H, D = 2, 256, 4, 64
    E = H * D
    qkv = torch.randn(B * S, 3 * E, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    o = flash_attention_qkvpacked(qkv, B, S, H, D, causal=True)
    do = torch.randn_like(o)
    o.backward(do)
    f = qkv.detach().float().requires_grad_(True)
    q, k, v = (f[:, i * E:(i + 1) * E].reshape(B, S, H, D) for i in range(3))
    orf = _sdpa_reference(q, k, v, True, 1.0 / math.sqrt(D)).reshape(B * S, E)
    orf.backward(do.float())
    assert _rel(o, orf) < 2e-2 and _rel(qkv.grad, f.grad) < 3e-2


# ------------------------------------------------------------------ GNN gather-scale-scatter
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gnn_scatter_fwd_bwd(dtype):
    from torsh_b200.ops.elementwise import gnn_scatter
    torch.manual_seed(11)
    N, E, Fd = 300, 5000, 64
    x = torch.randn(N, Fd, device=DEV, dtype=dtype, requires_grad=True)
    src, dst = torch.randint(0, N, (E,), device=DEV), torch.randint(0, N, (E,), device=DEV)
    w = torch.rand(E, device=DEV, requires_grad=True)
    out = gnn_scatter(x, dst, N, src=src, weight=w)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().clone().requires_grad_()
    ref = torch.zeros(N, Fd, device=DEV).index_add_(0, dst, xr[src] * wr[:, None])
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert _rel(out, ref) < tol
    g = torch.randn_like(ref)
    out.backward(g.to(dtype))
    ref.backward(g.to(dtype).float())
    assert _rel(x.grad, xr.grad) < tol and _rel(w.grad, wr.grad) < tol
    # plain scatter-add (no gather, no weight) and a GCN layer against the dense normalised-adjacency formula
    m = torch.randn(E, Fd, device=DEV, dtype=dtype)
    assert _rel(gnn_scatter(m, dst, N), torch.zeros(N, Fd, device=DEV).index_add_(0, dst, m.float())) < tol
    from torsh_b200.graph import GCNConv
    conv = GCNConv(Fd, 32).to(DEV)
    xf = torch.randn(N, Fd, device=DEV)
    ei = torch.stack([src, dst])
    A = torch.zeros(N, N, device=DEV).index_put_((dst, src), torch.ones(E, device=DEV), accumulate=True) + torch.eye(N, device=DEV)
    dg = A.sum(1)
    want = (dg.rsqrt()[:, None] * A * dg.rsqrt()[None]) @ conv.lin(xf) + conv.bias
    assert _rel(conv(xf, ei), want) < 1e-4


# ------------------------------------------------------------------ conv / BatchNorm / pooling (channels-last)
@pytest.mark.parametrize("geom", [(3, 64, 7, 2, 3, 34), (64, 64, 1, 1, 0, 20), (64, 128, 3, 1, 1, 19), (128, 128, 3, 2, 1, 18),
                                  (256, 512, 1, 2, 0, 14), (128, 64, 3, 1, 1, 5), (256, 256, 3, 1, 1, 14), (64, 64, 3, 1, 1, 56),
                                  (64, 72, 3, 1, 1, 9)])
def test_conv2d_nhwc_fwd_bwd(geom):
    from torsh_b200.ops.conv import conv2d_nhwc
    ci, co, k, stride, pad, hw = geom
    torch.manual_seed(3)
    x = torch.randn(4, hw, hw + 3, ci, device=DEV, dtype=torch.bfloat16, requires_grad=ci != 3)
    w = (torch.randn(co, ci, k, k, device=DEV) * (2.0 / (ci * k * k)) ** 0.5).requires_grad_()
    y = conv2d_nhwc(x, w, stride, pad)
    xr = x.detach().float().permute(0, 3, 1, 2).requires_grad_()
    wr = w.detach().to(torch.bfloat16).float().requires_grad_()
    ref = torch.nn.functional.conv2d(xr, wr, None, stride, pad)
    assert y.shape == ref.permute(0, 2, 3, 1).shape and _rel(y, ref.permute(0, 2, 3, 1)) < 1.5e-2
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float().permute(0, 3, 1, 2))
    assert _rel(w.grad, wr.grad) < 1.5e-2
    if ci != 3:
        assert _rel(x.grad, xr.grad.permute(0, 2, 3, 1)) < 1.5e-2


@pytest.mark.parametrize("C", [136, 128])
@pytest.mark.parametrize("relu,res", [(False, False), (True, False), (True, True)])
def test_batch_norm_nhwc_fwd_bwd(relu, res, C):
    from torsh_b200.ops.conv import batch_norm_nhwc
    torch.manual_seed(4)
    N, H, W = 8, 13, 11
    x = (torch.randn(N, H, W, C, device=DEV) * 2 + 0.5).to(torch.bfloat16).requires_grad_()
    r = torch.randn(N, H, W, C, device=DEV, dtype=torch.bfloat16).requires_grad_() if res else None
    bn = torch.nn.BatchNorm2d(C).to(DEV)
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5); bn.bias.normal_()
    ref_bn = torch.nn.BatchNorm2d(C).to(DEV)
    ref_bn.load_state_dict(bn.state_dict())
    y = batch_norm_nhwc(x, bn, residual=r, relu=relu)
    xr = x.detach().float().permute(0, 3, 1, 2).requires_grad_()
    rr = r.detach().float().permute(0, 3, 1, 2).requires_grad_() if res else None
    z = ref_bn(xr) + (rr if res else 0)
    ref = torch.relu(z) if relu else z
    assert _rel(y, ref.permute(0, 2, 3, 1)) < 1e-2
    assert torch.allclose(bn.running_mean, ref_bn.running_mean, atol=2e-3) and torch.allclose(bn.running_var, ref_bn.running_var, rtol=2e-2)
    g = torch.randn_like(y)
    # mask the oracle's gradient with the kernel's own ReLU decision so rounding at the kink does not count
    y.backward(g)
    gm = g.float() * ((y.detach() > 0) if relu else 1)
    z.backward(gm.permute(0, 3, 1, 2))
    assert _rel(x.grad, xr.grad.permute(0, 2, 3, 1)) < 2e-2
    assert _rel(bn.weight.grad, ref_bn.weight.grad) < 2e-2 and _rel(bn.bias.grad, ref_bn.bias.grad) < 2e-2
    if res:
        assert _rel(r.grad, rr.grad.permute(0, 2, 3, 1)) < 1e-2
    bn.eval(); ref_bn.eval()
    assert _rel(batch_norm_nhwc(x.detach(), bn, relu=relu), (torch.relu(ref_bn(xr)) if relu else ref_bn(xr)).permute(0, 2, 3, 1)) < 1e-2


def test_pooling_nhwc():
    from torsh_b200.ops.conv import global_avg_pool_nhwc, max_pool_nhwc
    torch.manual_seed(5)
    x = torch.relu(torch.randn(4, 17, 15, 64, device=DEV)).to(torch.bfloat16).requires_grad_()   # many ties at zero
    y = max_pool_nhwc(x, 3, 2, 1)
    xr = x.detach().float().permute(0, 3, 1, 2).requires_grad_()
    ref = torch.nn.functional.max_pool2d(xr, 3, 2, 1)
    assert torch.equal(y.float(), ref.permute(0, 2, 3, 1))
    g = torch.randn_like(y)
    y.backward(g)
    ref.backward(g.float().permute(0, 3, 1, 2))
    assert _rel(x.grad, xr.grad.permute(0, 2, 3, 1)) < 1e-2
    x2 = torch.randn(6, 7, 7, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    a = global_avg_pool_nhwc(x2)
    assert _rel(a, x2.detach().float().mean((1, 2))) < 1e-2
    a.backward(torch.ones_like(a))
    assert _rel(x2.grad, torch.full_like(x2, 1 / 49)) < 1e-2


def test_resnet_kernel_path_matches_torch_layers():
    """Oracle: the fp32 PyTorch layers. A random-init BatchNorm network amplifies bf16 rounding, so the yardstick for
    "close enough" is PyTorch's own bf16 autocast run of the same model: the kernel path must track fp32 as well as
    that does (gradient direction per parameter), and exactly at the head."""
    from torsh_b200.models import ResNet, ResNetConfig
    torch.manual_seed(6)
    m = ResNet(ResNetConfig(layers=(1, 1, 1, 1), num_classes=16)).to(DEV)
    x = torch.randn(16, 3, 96, 96, device=DEV)
    tgt = torch.randint(0, 16, (16,), device=DEV)

    def run(mode):
        m.zero_grad()
        for b in m.modules():
            if isinstance(b, torch.nn.BatchNorm2d):
                b.reset_running_stats()
        m.use_kernels = mode == "kernel"
        if mode == "autocast":
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = torch.nn.functional.cross_entropy(m(x).float(), tgt)
        else:
            loss = torch.nn.functional.cross_entropy(m(x), tgt)
        loss.backward()
        return loss.item(), {n: p.grad.clone().float() for n, p in m.named_parameters()}

    cos = lambda a, b: torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    lk, gk = run("kernel")
    lf, gf = run("fp32")
    _, ga = run("autocast")
    assert abs(lk - lf) < 0.02 * abs(lf) + 0.02
    bad = {n: (round(cos(gk[n], gf[n]), 3), round(cos(ga[n], gf[n]), 3)) for n in gk if cos(gk[n], gf[n]) < cos(ga[n], gf[n]) - 0.04}
    assert not bad, bad
    assert cos(gk["fc.weight"], gf["fc.weight"]) > 0.999 and cos(gk["layer4.0.bn3.weight"], gf["layer4.0.bn3.weight"]) > 0.99


# ------------------------------------------------------------------ gradient compression + native profiler ranges
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_compression_kernels_match_cpu_arithmetic(dtype):
    from torsh_b200.parallel import compression as cp
    torch.manual_seed(12)
    g = torch.randn(100_003, device=DEV).to(dtype)
    q, sc = cp.Int8BlockQuantization().compress(g)
    qc, scc = cp.Int8BlockQuantization().compress(g.cpu())
    assert torch.allclose(sc.cpu(), scc, rtol=1e-6) and (q.cpu().int() - qc.int()).abs().max() <= 1
    back = cp.Int8BlockQuantization().decompress((q, sc), g.shape, dtype)
    assert (back.float() - g.float()).abs().max() <= sc.max() * 0.51 + 0.02
    bits, s, n = cp.PackedSignSGD().compress(g)
    bc, scpu, _ = cp.PackedSignSGD().compress(g.cpu())
    assert torch.equal(bits.cpu(), bc) and abs(s.item() - scpu.item()) < 1e-3 * scpu.item()
    sg = cp.PackedSignSGD().decompress((bits, s, n), g.shape, dtype)
    assert torch.equal(sg > 0, g >= 0)
    idx, vals = cp.threshold_sparsify(g, 2.5)
    want = (g.float().abs() > 2.5).nonzero().flatten()
    order = idx.long().argsort()
    assert torch.equal(idx.long()[order], want) and torch.equal(vals[order], g.float()[want])


def test_native_profiler_ranges():
    from torsh_b200.ops import elementwise as ew
    from torsh_b200.utils.profiler import DeviceRangeProfiler
    prof = DeviceRangeProfiler()
    x = torch.randn(1 << 22, device=DEV)
    with prof.range("step"):
        with prof.range("relu"):
            ew.unary_raw("relu", x)
        with prof.range("exp"):
            ew.unary_raw("exp", x)
    rec = prof.collect()
    by = {r["name"]: r for r in rec}
    assert set(by) == {"step", "relu", "exp"} and by["step"]["depth"] == 0 and by["relu"]["depth"] == 1
    assert by["step"]["device_us"] >= by["relu"]["device_us"] > 0 and "traceEvents" in prof.chrome_trace()


# ------------------------------------------------------------------ quantised / sparse
@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_int4_groupwise_kernels_match_reference(group, dtype):
    from torsh_b200 import quantization as Q
    torch.manual_seed(0)
    w = (torch.randn(96, 512, device=DEV) * 0.05).to(dtype)
    q, s = Q.quantize_groupwise(w, group, 4)
    q_ref, s_ref = Q.quantize_groupwise(w.float().cpu(), group, 4)       # the plain PyTorch formulation
    assert q.dtype == torch.int8 and q.shape == (96, 256) and s.shape == (96, 512 // group)
    assert torch.allclose(s.cpu(), s_ref, rtol=1e-6, atol=0)
    same = (q.cpu() == q_ref).float().mean().item()
    assert same > 0.99        # bytes hold two codes; values within rounding of a .5 tie may land on the neighbouring code
    d = Q.dequantize_groupwise(q, s, group, 4, dtype=torch.float32)
    d_ref = Q.dequantize_groupwise(q.cpu(), s.cpu(), group, 4)
    assert torch.equal(d.cpu(), d_ref)
    assert ((d - w.float()).abs() <= 0.505 * s.repeat_interleave(group, -1) + 1e-7).all()


@pytest.mark.parametrize("M", [1, 2, 3, 8])
def test_int4_linear_matches_dequantised_matmul(M):
    from torsh_b200 import quantization as Q
    torch.manual_seed(1)
    lin = torch.nn.Linear(1024, 384).to(DEV)
    ql = Q.Int4Linear(lin, group=128)
    x = torch.randn(M, 1024, device=DEV, dtype=torch.bfloat16)
    y = ql(x)
    ref = x.float() @ ql.dequantized_weight(torch.float32).t() + lin.bias.float()
    assert y.shape == (M, 384) and _rel_elem(y, ref) < 1e-2
    big = torch.randn(32, 1024, device=DEV, dtype=torch.bfloat16)        # the dequantise + GEMM route
    assert _rel_elem(ql(big), big.float() @ ql.dequantized_weight(torch.float32).t() + lin.bias.float()) < 2e-2


def test_int8_rowwise_kernels():
    from torsh_b200 import quantization as Q
    torch.manual_seed(2)
    x = torch.randn(300, 777, device=DEV, dtype=torch.bfloat16)
    q, s = Q.quantize_int8_rowwise(x)
    assert torch.allclose(s, x.float().abs().amax(-1) / 127, rtol=1e-6)
    ref = (x.float() / s[:, None]).round().clamp(-127, 127)
    assert ((q.float() - ref).abs() <= 1).all() and ((q.float() == ref).float().mean() > 0.99)
    d = Q.dequantize_int8_rowwise(q, s, torch.float32)
    assert torch.equal(d, q.float() * s[:, None])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 7, 128, 200])
def test_csr_spmm_matches_dense(dtype, n):
    from torsh_b200.sparse import CudaSparseTensor, prune_magnitude
    torch.manual_seed(3)
    a = prune_magnitude(torch.randn(333, 517, device=DEV), 0.93)
    a[5] = 0                                                               # an empty row
    sp = CudaSparseTensor.from_dense(a)
    b = torch.randn(517, n, device=DEV).to(dtype)
    out = sp @ b
    ref = a.double() @ b.double()
    assert out.dtype == dtype and _rel_elem(out, ref) < (1e-5 if dtype == torch.float32 else 1e-2)
    assert torch.equal(sp.to_dense(), a) and torch.equal(sp.transpose().to_dense(), a.t())
    v = torch.randn(517, device=DEV)
    assert _rel_elem(sp @ v, a.double() @ v.double()) < 1e-5


# ------------------------------------------------------------------ LSTM, depthwise / grouped convolution
@pytest.mark.parametrize("T,B,I,H", [(5, 4, 64, 128), (12, 16, 256, 256)])
def test_lstm_layer_matches_torch(T, B, I, H):
    from torsh_b200.ops.rnn import KernelLSTM
    torch.manual_seed(0)
    ref = torch.nn.LSTM(I, H, num_layers=2).to(DEV)
    mine = KernelLSTM(I, H, num_layers=2).to(DEV)
    mine.load_state_dict(ref.state_dict())
    mine = mine.to(torch.bfloat16)
    x = (torch.randn(T, B, I, device=DEV) * 0.5)
    xb = x.to(torch.bfloat16).requires_grad_(True)
    xr = x.to(torch.bfloat16).float().requires_grad_(True)
    for p in ref.parameters():
        p.data = p.data.to(torch.bfloat16).float()         # same rounded weights on both sides
    out, (hT, cT) = mine(xb)
    out_r, (hT_r, cT_r) = ref(xr)
    assert _rel(out, out_r) < 3e-2 and _rel(hT, hT_r) < 3e-2 and _rel(cT, cT_r) < 3e-2
    g = torch.randn_like(out_r)
    out.backward(g.to(torch.bfloat16))
    out_r.backward(g)
    assert _rel(xb.grad, xr.grad) < 5e-2
    for (n, p), (_, q) in zip(mine.named_parameters(), ref.named_parameters()):
        assert _rel(p.grad, q.grad) < 5e-2, n


@pytest.mark.parametrize("k,stride,pad", [(3, 1, 1), (3, 2, 1), (5, 1, 2), (7, 1, 3), (3, 2, 0)])
def test_depthwise_conv_matches_torch(k, stride, pad):
    from torsh_b200.ops.conv import depthwise_conv2d_nhwc
    torch.manual_seed(1)
    n, h, w, c = 3, 19, 23, 72
    x = torch.randn(n, h, w, c, device=DEV).to(torch.bfloat16).requires_grad_(True)
    wt = (torch.randn(c, 1, k, k, device=DEV) * 0.2).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(c, device=DEV).to(torch.bfloat16).requires_grad_(True)
    y = depthwise_conv2d_nhwc(x, wt, b, stride, pad)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, wt, b))
    yr = torch.nn.functional.conv2d(xf.permute(0, 3, 1, 2), wf, bf, stride, pad, groups=c).permute(0, 2, 3, 1)
    assert y.shape == yr.shape and _rel(y, yr) < 1e-2
    g = torch.randn_like(yr)
    y.backward(g.to(torch.bfloat16))
    yr.backward(g.to(torch.bfloat16).float())
    assert _rel(x.grad, xf.grad) < 1e-2 and _rel(wt.grad, wf.grad) < 1e-2 and _rel(b.grad, bf.grad) < 1e-2


def test_grouped_conv_matches_torch():
    from torsh_b200.ops.conv import grouped_conv2d_nhwc
    torch.manual_seed(2)
    x = torch.randn(2, 14, 14, 128, device=DEV).to(torch.bfloat16)
    wt = (torch.randn(256, 32, 3, 3, device=DEV) * 0.05).to(torch.bfloat16)
    y = grouped_conv2d_nhwc(x, wt, None, 1, 1, groups=4)
    yr = torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), wt.float(), None, 1, 1, groups=4).permute(0, 2, 3, 1)
    assert _rel(y, yr) < 1e-2


# ------------------------------------------------------------------ run-time generated kernels
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [8, 1000, 1 << 20, (1 << 20) + 13])
def test_generated_fused_elementwise_kernel(dtype, n, tmp_path_factory, monkeypatch):
    from torsh_b200.core import kernel_gen as kg
    monkeypatch.setenv("TORSH_JIT_DIR", str(tmp_path_factory.getbasetemp() / "jit"))     # one compile per dtype for all sizes
    f = kg.FusedElementwise(lambda a, b, c: kg.where(kg.greater(a, 0.0), a * kg.sigmoid(b) + 0.5,
                                                    kg.gelu_tanh(c) / (1.0 + kg.absolute(b))), 3)
    torch.manual_seed(n)
    a, b, c = (torch.randn(n, device=DEV).to(dtype) for _ in range(3))
    out = f(a, b, c)
    af, bf, cf = a.float(), b.float(), c.float()
    ref = torch.where(af > 0, af * torch.sigmoid(bf) + 0.5, torch.nn.functional.gelu(cf, approximate="tanh") / (1 + bf.abs()))
    assert out.dtype == dtype and out.shape == a.shape
    assert _rel_elem(out, ref) < (1e-2 if dtype == torch.bfloat16 else 1e-4)
    if n >= 1 << 20:
        table = kg.default_selector().tuner.table
        assert any(k.startswith(f.expr.key()) for k in table)          # a variant was measured and remembered


def test_deferred_expression_runs_as_one_generated_kernel(tmp_path_factory, monkeypatch):
    from torsh_b200 import tensor_ext as E
    monkeypatch.setenv("TORSH_JIT_DIR", str(tmp_path_factory.getbasetemp() / "jit_expr"))
    E.Expr._KERNELS.clear()
    torch.manual_seed(0)
    a, b = torch.randn(1 << 18, device=DEV), torch.randn(1 << 18, device=DEV)
    ex = (E.expr(a) * 2.0 + E.expr(b)).apply("relu") - 1 + (-E.expr(a)) / 4
    out = ex.eval()
    assert len(E.Expr._KERNELS) == 1 and _rel_elem(out, torch.relu(a * 2 + b) - 1 - a / 4) < 1e-4
    assert ex.eval().shape == a.shape and len(E.Expr._KERNELS) == 1                      # second call reuses the compiled kernel


def test_gemm_measured_tile_selection():
    """With autotuning on, every candidate tile / raster choice is timed once per shape, the winner is remembered and
    the product is unchanged."""
    from torsh_b200.ops import gemm as G
    torch.manual_seed(5)
    a = torch.randn(2048, 1024, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(3072, 1024, device=DEV, dtype=torch.bfloat16)
    ref = G.gemm(a, b)
    tuner = G.gemm_autotune(True)
    try:
        out = G.gemm(a, b)
        key = "gemm|2048x3072x1024|a0b0|f0"
        assert key in tuner.table and set(tuner.table[key].times_ms) == {"bn128_r0", "bn128_r1", "bn256_r0", "bn256_r1"}
        assert tuner.table[key].choice == min(tuner.table[key].times_ms, key=tuner.table[key].times_ms.get)
        assert _rel_elem(out, a.float() @ b.float().t()) < 1e-2 and _rel_elem(out, ref) < 1e-2
        n = len(tuner.table)
        G.gemm(a, b)
        assert len(tuner.table) == n                       # second call: table hit, no new measurement
    finally:
        G.gemm_autotune(False)


def test_jit_compiler_runs_fused_regions_as_generated_kernels(tmp_path_factory, monkeypatch):
    from torsh_b200 import jit_compiler as J
    monkeypatch.setenv("TORSH_JIT_DIR", str(tmp_path_factory.getbasetemp() / "jit"))
    torch.manual_seed(0)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = torch.nn.Linear(256, 256)

        def forward(self, x, y):
            h = self.fc(x)
            return (torch.tanh(h) * y + torch.nn.functional.silu(h) - 0.5).sum(-1)
    net = Net().to(DEV).to(torch.bfloat16)
    x, y = (torch.randn(512, 256, device=DEV, dtype=torch.bfloat16) for _ in range(2))
    jf = J.jit(net, hot_threshold=1)
    outs = [jf(x, y) for _ in range(3)]
    assert jf.stats.specializations == 1 and jf.stats.fused_regions == 1 and jf.stats.compiled_calls == 2
    exe = jf.cache[jf.signature((x, y))]
    assert any(k._libs for k in exe._kernels.values())                    # a generated library was loaded and launched
    ref = net(x, y).float()
    assert _rel(outs[-1], ref) < 2e-2
