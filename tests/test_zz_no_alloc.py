"""The allocation-free norm-backward entry point must agree with the regular one.

It is meant for callers that cannot allocate when they call (stream capture, serving loops, plain C hosts),
so the test drives it the way such a caller would: through the exported C symbol, with buffers that already
exist, twice in a row on the same stream (the second call reuses the scratch the first one dirtied).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup():
    from torsh_b200 import _native as nv
    lib = nv.require_cuda()
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.tb_norm_bwd_static.restype = I
    lib.tb_norm_bwd_static.argtypes = [P] * 9 + [I] * 4 + [P]
    lib.tb_norm_bwd_static_capacity.restype = ctypes.c_long
    lib.tb_norm_bwd.restype = I
    lib.tb_norm_bwd.argtypes = [P] * 10 + [I] * 4 + [P]
    lib.tb_norm_bwd_workspace.restype = ctypes.c_long
    lib.tb_norm_bwd_workspace.argtypes = [I, I]
    lib.tb_norm_fwd.restype = I
    lib.tb_norm_fwd.argtypes = [P] * 6 + [I, I, ctypes.c_float, I, I, P]
    return nv, lib


@pytest.mark.parametrize("dtype,rms", [(torch.bfloat16, False), (torch.float32, False), (torch.bfloat16, True)])
def test_static_scratch_entry_point_matches_regular_one(dtype, rms):
    nv, lib = _setup()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = nv.stream_ptr()
    code = 0 if dtype == torch.bfloat16 else 1
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    for call_no, (rows, H) in enumerate(((777, 1024), (2048, 512))):  # two calls in a row, different shapes
        torch.manual_seed(20 + call_no)
        x = torch.randn(rows, H, device=dev, dtype=dtype)
        dy = torch.randn(rows, H, device=dev, dtype=dtype)
        dres = torch.randn(rows, H, device=dev, dtype=dtype)
        gamma = (torch.randn(H, device=dev) * 0.2 + 1).to(dtype)
        beta = torch.zeros(H, device=dev, dtype=dtype)
        y = torch.empty_like(x)
        mean = torch.empty(rows, device=dev, dtype=torch.float32)
        rstd = torch.empty(rows, device=dev, dtype=torch.float32)
        assert lib.tb_norm_fwd(x.data_ptr(), gamma.data_ptr(), None if rms else beta.data_ptr(), y.data_ptr(),
                               mean.data_ptr(), rstd.data_ptr(), rows, H, 1e-5, int(rms), code, stream) == 0
        outs = []
        for static in (False, True):
            dx = torch.empty_like(x)
            dg = torch.zeros(H, device=dev, dtype=torch.float32)
            db = torch.zeros(H, device=dev, dtype=torch.float32)
            if static:
                assert lib.tb_norm_bwd_workspace(rows, H) <= lib.tb_norm_bwd_static_capacity()
                rc = lib.tb_norm_bwd_static(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                            rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), dg.data_ptr(),
                                            None if rms else db.data_ptr(), rows, H, int(rms), code, stream)
            else:
                ws = torch.empty(lib.tb_norm_bwd_workspace(rows, H), device=dev, dtype=torch.float32)
                rc = lib.tb_norm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                     dres.data_ptr(), dx.data_ptr(), dg.data_ptr(), None if rms else db.data_ptr(),
                                     ws.data_ptr(), rows, H, int(rms), code, stream)
            assert rc == 0, lib.tb_last_error()
            torch.cuda.synchronize()
            outs.append((dx.float(), dg, db))
        for a, b in zip(*outs):
            denom = b.abs().max().clamp(min=1e-6)
            assert ((a - b).abs().max() / denom).item() < tol
        # and against a plain fp32 PyTorch evaluation of the same backward
        xf = x.float().requires_grad_(True)
        gf = gamma.float().requires_grad_(True)
        bf = beta.float().requires_grad_(True)
        if rms:
            yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gf
        else:
            yf = torch.nn.functional.layer_norm(xf, (H,), gf, bf, 1e-5)
        yf.backward(dy.float())
        ref = (xf.grad + dres.float(), gf.grad, None if rms else bf.grad)
        for a, r in zip(outs[1], ref):
            if r is not None:
                assert ((a - r).abs().max() / r.abs().max().clamp(min=1e-6)).item() < tol


def test_static_scratch_rejects_oversized_requests():
    nv, lib = _setup()
    dev = torch.device("cuda", torch.cuda.current_device())
    rows, H = 4096, 4096  # needs far more than 8 MiB of partial sums
    assert lib.tb_norm_bwd_workspace(rows, H) > lib.tb_norm_bwd_static_capacity()
    t = torch.zeros(8, device=dev)
    rc = lib.tb_norm_bwd_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None,
                                t.data_ptr(), t.data_ptr(), None, rows, H, 0, 1, nv.stream_ptr())
    assert rc == -4 and b"scratch" in lib.tb_last_error()
