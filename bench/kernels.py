#!/usr/bin/env python
"""Kernel micro-benchmarks (device-timed with CUDA events) and the small cases used for ncu captures.

  python bench/kernels.py gemm --m 8192 --n 4096 --k 4096 [--a-major 0 --b-major 0 --bn 256]
  python bench/kernels.py attn_fwd | attn_bwd --batch 4 --seq 2048 --heads 16 --dim 64
  python bench/kernels.py layernorm | xent | adamw
  python bench/kernels.py bn --batch 64 --hw 56 --channels 256        # BatchNorm2d fwd and bwd, channels-last bf16
  python bench/kernels.py conv --batch 64 --hw 56 --channels 64 --ksize 3 # conv fwd (im2col + GEMM) and bwd
Each run prints achieved TFLOP/s or GB/s and the fraction of the measured peak in MEASURED_PEAKS.json
(fallback 6.65 TB/s, 1.59 PFLOP/s when that file is absent).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters, flush):
    for _ in range(3):
        fn()
    e = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    torch.cuda.synchronize()
    for a, b in e:
        flush.add_(1.0)  # 256 MB write: evicts the 126 MB L2 between timed iterations
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in e)
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--no-residual", action="store_true", help="bn: BatchNorm + ReLU without a residual input")
    ap.add_argument("what", choices=["gemm", "attn_fwd", "attn_bwd", "layernorm", "layernorm_bwd", "xent", "adamw", "bn", "conv", "fsdp_gather"])
    ap.add_argument("--hw", type=int, default=56); ap.add_argument("--channels", type=int, default=256)
    ap.add_argument("--cout", type=int, default=0); ap.add_argument("--ksize", type=int, default=3); ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--m", type=int, default=8192); ap.add_argument("--n", type=int, default=4096); ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--a-major", type=int, default=0); ap.add_argument("--b-major", type=int, default=0); ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--batch", type=int, default=4); ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16); ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--compare", action="store_true", help="gemm: also time torch.matmul on the same operands")
    ap.add_argument("--split-k", type=int, default=1, help="gemm: K splits, -1 = stream-K (implies fp32 atomic accumulation, the weight-gradient path)")
    a = ap.parse_args()
    from torsh_b200 import _native as nv
    dev = "cuda"
    hbm, tf, kind = peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    torch.manual_seed(0)
    if a.what == "gemm":
        from torsh_b200.ops.gemm import gemm
        A = torch.randn((a.m, a.k) if a.a_major == 0 else (a.k, a.m), device=dev, dtype=torch.bfloat16)
        B = torch.randn((a.n, a.k) if a.b_major == 0 else (a.k, a.n), device=dev, dtype=torch.bfloat16)
        if a.split_k != 1:
            out = torch.zeros(a.m, a.n, device=dev, dtype=torch.float32)
            ms = timeit(lambda: gemm(A, B, a_major=a.a_major, b_major=a.b_major, out=out, bn=a.bn, atomic=True, split_k=a.split_k), a.iters, flush)
        else:
            out = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
            ms = timeit(lambda: gemm(A, B, a_major=a.a_major, b_major=a.b_major, out=out, bn=a.bn), a.iters, flush)
        t = 2.0 * a.m * a.n * a.k / ms / 1e9
        if a.compare:
            Am = A if a.a_major == 0 else A.t()
            Bm = B.t() if a.b_major == 0 else B
            ref = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
            msl = timeit(lambda: torch.matmul(Am, Bm, out=ref), a.iters, flush)
            print(f"  torch.matmul (cuBLAS) same shape: {msl*1e3:.1f} us, {2.0*a.m*a.n*a.k/msl/1e9:.0f} TFLOP/s")
        print(f"gemm {a.m}x{a.n}x{a.k} majors {a.a_major}{a.b_major} bn {a.bn} split_k {a.split_k}: {ms*1e3:.1f} us, {t:.0f} TFLOP/s = {t/tf:.2f} of {kind} bf16 peak")
    elif a.what == "fsdp_gather":
        # One rank, no peer: the FSDP un-shard machinery on local memory (the NVLink share is measured by bench.py on
        # several GPUs). Times the stand-alone gather of one GPT-2-medium block (24 MB) for several copy-CTA counts, the
        # QKV GEMM alone, and the same GEMM with the gather fused in (copy CTAs + per-chunk ready words).
        import ctypes
        from torsh_b200.ops.gemm import _lib, gemm
        lib = _lib()
        P, I = ctypes.c_void_p, ctypes.c_int
        lib.tb_fsdp_unit_gather.restype = I
        lib.tb_fsdp_unit_gather.argtypes = [P] * 5 + [I] * 5 + [P] * 2
        chunk, cpr = 512 * 1024, 48
        shard = torch.randn(chunk * cpr // 2, device=dev, dtype=torch.bfloat16)
        unit = torch.zeros_like(shard)
        flags = torch.zeros(320 * 8, device=dev, dtype=torch.int32)
        epoch = torch.ones(1, device=dev, dtype=torch.int32)
        ready = torch.zeros(2 * cpr, device=dev, dtype=torch.int32)
        arr = lambda t: (ctypes.c_void_p * 8)(t.data_ptr(), *([0] * 7))
        shards, flag_tbl = arr(shard), arr(flags)
        st = nv.status_word(torch.device(dev))
        for ctas in (16, 32, 64, 96, 128):
            def run():
                rc = lib.tb_fsdp_unit_gather(shards, unit.data_ptr(), flag_tbl, epoch.data_ptr(), ready.data_ptr(), chunk, cpr, 0, 1,
                                             ctas, st.data_ptr(), nv.stream_ptr())
                assert rc == 0, lib.tb_last_error()
            ms = timeit(run, a.iters, flush)
            nv.check_status()
            assert torch.equal(unit, shard)
            gb = 2 * shard.numel() * 2 / ms / 1e6
            print(f"stand-alone gather, 24 MB unit, {ctas:3d} copy CTAs: {ms*1e3:.1f} us, {gb:.0f} GB/s read+write = {gb/hbm:.2f} of {kind} copy bandwidth")
        M, N, K = a.m, 3072, 1024
        A = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        Bw = unit[: N * K].view(N, K)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ms0 = timeit(lambda: gemm(A, Bw, out=out), a.iters, flush)
        print(f"QKV GEMM alone {M}x{N}x{K}: {ms0*1e3:.1f} us, {2.0*M*N*K/ms0/1e9:.0f} TFLOP/s")
        ref = out.clone()
        for ctas in (8, 16, 32):
            def run():
                rc = lib.tb_fsdp_ag_gemm(A.data_ptr(), Bw.data_ptr(), out.data_ptr(), M, N, K, 0, 0, K, K, N, None, None, 0, None, None, 0, 0,
                                         shards, unit.data_ptr(), flag_tbl, epoch.data_ptr(), ready.data_ptr(), chunk, cpr, 0, 0, 1, ctas,
                                         st.data_ptr(), nv.stream_ptr())
                assert rc == 0, lib.tb_last_error()
            unit.zero_()
            ms = timeit(run, a.iters, flush)
            nv.check_status()
            assert torch.equal(unit, shard) and torch.equal(out, ref)
            print(f"QKV GEMM with the 24 MB un-shard fused in, {ctas:2d} copy CTAs: {ms*1e3:.1f} us ({ms/ms0:.2f} x the GEMM alone)")
    elif a.what in ("attn_fwd", "attn_bwd"):
        from torsh_b200.ops.attention import flash_attention
        q, k, v = (torch.randn(a.batch, a.seq, a.heads, a.dim, device=dev, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
        fl = 4.0 * a.batch * a.heads * a.seq * a.seq * a.dim * 0.5
        if a.what == "attn_fwd":
            with torch.no_grad():
                ms = timeit(lambda: flash_attention(q, k, v, causal=True), a.iters, flush)
        else:
            o = flash_attention(q, k, v, causal=True)
            do = torch.randn_like(o)
            ms = timeit(lambda: o.backward(do, retain_graph=True), a.iters, flush)
            fl *= 2.5
        t = fl / ms / 1e9
        print(f"{a.what} B{a.batch} S{a.seq} H{a.heads} D{a.dim} causal: {ms*1e3:.1f} us, {t:.0f} TFLOP/s = {t/tf:.2f} of {kind} bf16 peak")
    elif a.what == "layernorm":
        from torsh_b200.ops.norm import layer_norm
        x = torch.randn(a.m, a.n, device=dev, dtype=torch.bfloat16)
        w, b = torch.ones(a.n, device=dev, dtype=torch.bfloat16), torch.zeros(a.n, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            ms = timeit(lambda: layer_norm(x, w, b), a.iters, flush)
        gb = 2.0 * x.numel() * 2 / ms / 1e6
        print(f"layernorm fwd {a.m}x{a.n}: {ms*1e3:.1f} us, {gb:.0f} GB/s = {gb/hbm:.2f} of {kind} copy bandwidth")
    elif a.what == "layernorm_bwd":
        from torsh_b200.ops.norm import layer_norm
        x = torch.randn(a.m, a.n, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(a.n, device=dev, dtype=torch.bfloat16, requires_grad=True)
        b = torch.zeros(a.n, device=dev, dtype=torch.bfloat16, requires_grad=True)
        y = layer_norm(x, w, b)
        dy = torch.randn_like(y)
        ms = timeit(lambda: torch.autograd.grad(y, (x, w, b), dy, retain_graph=True), a.iters, flush)
        gb = 3.0 * x.numel() * 2 / ms / 1e6          # dy and x in, dx out
        print(f"layernorm bwd {a.m}x{a.n} (incl. the weight-gradient reduction): {ms*1e3:.1f} us, {gb:.0f} GB/s = {gb/hbm:.2f} of {kind} copy bandwidth")
    elif a.what == "xent":
        from torsh_b200.ops.softmax import cross_entropy
        lg = torch.randn(a.m, 50304, device=dev, dtype=torch.bfloat16, requires_grad=True)
        tg = torch.randint(0, 50257, (a.m,), device=dev)
        ms = timeit(lambda: cross_entropy(lg, tg, num_classes=50257, inplace_grad=False, root_scale=1.0), a.iters, flush)
        gb = 2.0 * lg.numel() * 2 / ms / 1e6
        print(f"cross-entropy fwd+bwd {a.m}x50304: {ms*1e3:.1f} us, {gb:.0f} GB/s = {gb/hbm:.2f} of {kind} copy bandwidth")
    elif a.what == "bn":
        from torsh_b200.ops.conv import batch_norm_nhwc
        C = a.channels
        x = torch.randn(a.batch, a.hw, a.hw, C, device=dev, dtype=torch.bfloat16, requires_grad=True)
        r = None if a.no_residual else torch.randn_like(x)
        bn = torch.nn.BatchNorm2d(C).to(dev)
        nbytes = x.numel() * 2
        with torch.no_grad():
            ms = timeit(lambda: batch_norm_nhwc(x, bn, residual=r, relu=True), a.iters, flush)
        gb = (3.0 if r is None else 4.0) * nbytes / ms / 1e6      # statistics read x; apply reads x (and the residual), writes y
        print(f"batchnorm fwd (+residual, +relu) {a.batch}x{a.hw}x{a.hw}x{C}: {ms*1e3:.1f} us, {gb:.0f} GB/s = {gb/hbm:.2f} of {kind} copy bandwidth")
        y = batch_norm_nhwc(x, bn, residual=r, relu=True)
        dy = torch.randn_like(y)
        ms = timeit(lambda: y.backward(dy, retain_graph=True), a.iters, flush)
        # reduce reads dy, y, x; apply reads them again and writes dx and the residual gradient; without a residual the
        # mask is recomputed from x: dy, x twice and dx
        gb = (5.0 if r is None else 8.0) * nbytes / ms / 1e6
        print(f"batchnorm bwd {a.batch}x{a.hw}x{a.hw}x{C}: {ms*1e3:.1f} us, {gb:.0f} GB/s = {gb/hbm:.2f} of {kind} copy bandwidth")
    elif a.what == "conv":
        from torsh_b200.ops.conv import conv2d_nhwc
        C, Co, k = a.channels, (a.cout or a.channels), a.ksize
        x = torch.randn(a.batch, a.hw, a.hw, C, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = (torch.randn(Co, C, k, k, device=dev) * (2.0 / (C * k * k)) ** 0.5).requires_grad_()
        with torch.no_grad():
            ms = timeit(lambda: conv2d_nhwc(x, w, a.stride, k // 2), a.iters, flush)
        ho = (a.hw + 2 * (k // 2) - k) // a.stride + 1
        fl = 2.0 * a.batch * ho * ho * Co * C * k * k
        print(f"conv {k}x{k}/{a.stride} fwd {a.batch}x{a.hw}x{a.hw}x{C}->{Co}: {ms*1e3:.1f} us, {fl/ms/1e9:.0f} TFLOP/s = {fl/ms/1e9/tf:.2f} of {kind} bf16 peak")
        y = conv2d_nhwc(x, w, a.stride, k // 2)
        dy = torch.randn_like(y)
        ms = timeit(lambda: y.backward(dy, retain_graph=True), a.iters, flush)
        print(f"conv {k}x{k}/{a.stride} bwd (dgrad + wgrad): {ms*1e3:.1f} us, {2*fl/ms/1e9:.0f} TFLOP/s = {2*fl/ms/1e9/tf:.2f} of {kind} bf16 peak")
    else:
        from torsh_b200.optim import FlatAdamW, FlatParameters
        p = torch.nn.Parameter(torch.randn(a.m * a.n, device=dev))
        flat = FlatParameters([p])
        opt = FlatAdamW(flat)
        flat.grad.normal_()
        ms = timeit(lambda: opt.step(), a.iters, flush)
        gb = flat.total * 30.0 / ms / 1e6
        print(f"fused AdamW {flat.total/1e6:.0f}M params: {ms*1e3:.1f} us, {gb:.0f} GB/s = {gb/hbm:.2f} of {kind} copy bandwidth")
    torch.cuda.synchronize()
    nv.check_status()


if __name__ == "__main__":
    main()
