"""bf16 tensor-core GEMM (tcgen05 / TMEM / TMA) with fused epilogues.

``gemm(a, b, ...)`` computes ``D[M,N] = A · Bᵀ`` where each operand may be stored K-major
(contraction index contiguous) or MN-major (output index contiguous); that covers the three
products of a linear layer (forward ``x Wᵀ``, dgrad ``dy W``, wgrad ``dyᵀ x``) without a transpose
pass. Kernel: ``csrc/kernels/gemm_sm100.cu``. The reference's matmul is a 2-D naive triple loop
(``crates/torsh-tensor/src/advanced_ops.rs:1000-1042``).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv

EPI_BIAS = 1
EPI_GELU = 2
EPI_RESIDUAL = 4
EPI_OUT_F32 = 8
EPI_ATOMIC = 16
EPI_STORE_PREACT = 32
EPI_MUL_DGELU = 64
EPI_ACCUM = 128
EPI_RASTER_M = 256

_configured = False

# ---- measured tile selection --------------------------------------------------------------------------------------
# Off by default: the launcher's heuristic (BN 256 unless the grid would be short, rasterise along M for wide outputs)
# is what the benchmarks run. `gemm_autotune(True)` or TORSH_GEMM_AUTOTUNE=1 times the candidates (BN 128 / 256 x both
# raster orders) once per problem shape on the caller's tensors and remembers the winner; TORSH_GEMM_TUNE_FILE keeps
# the table across runs. Accumulating / atomic products and launches inside a CUDA-graph capture are never timed.
_autotune = None


def gemm_autotune(on: bool = True, path: str | None = None):
    """Switches measured tile selection on or off; returns the tuner (its ``table`` maps shape keys to choices)."""
    global _autotune
    if not on:
        _autotune = None
        return None
    import os
    from ..core.backend import Autotuner
    _autotune = Autotuner(path or os.environ.get("TORSH_GEMM_TUNE_FILE"), warmup=1, iters=3)
    return _autotune


def _env_autotune():
    import os
    if _autotune is None and os.environ.get("TORSH_GEMM_AUTOTUNE", "0") == "1":
        gemm_autotune(True)
    return _autotune


def _lib():
    global _configured
    lib = nv.require_cuda()
    if not _configured:
        lib.tb_gemm_bf16.restype = ctypes.c_int
        lib.tb_gemm_bf16.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 8 + [ctypes.c_void_p] * 2 + [
            ctypes.c_int] + [ctypes.c_void_p] * 2 + [ctypes.c_int] * 3 + [ctypes.c_void_p] * 2
        lib.tb_fsdp_ag_gemm.restype = ctypes.c_int
        lib.tb_fsdp_ag_gemm.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 8 + [ctypes.c_void_p] * 2 + [
            ctypes.c_int] + [ctypes.c_void_p] * 2 + [ctypes.c_int] * 2 + [ctypes.c_void_p] * 5 + [ctypes.c_int] * 2 + [
            ctypes.c_int64] + [ctypes.c_int] * 3 + [ctypes.c_void_p] * 2
        _configured = True
    return lib


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_major: int = 0, b_major: int = 0, out: torch.Tensor | None = None,
         bias: torch.Tensor | None = None, gelu: bool = False, residual: torch.Tensor | None = None,
         preact_out: torch.Tensor | None = None, dgelu_aux: torch.Tensor | None = None, out_dtype=torch.bfloat16,
         atomic: bool = False, accumulate: bool = False, split_k: int = 1, bn: int = 0,
         raster_m: bool | None = None) -> torch.Tensor:
    """``D = op(A) · op(B)ᵀ`` on the 5th-gen tensor cores.

    a_major=0: ``a`` is ``[M, K]``; a_major=1: ``a`` is ``[K, M]`` (i.e. Aᵀ stored row-major).
    b_major=0: ``b`` is ``[N, K]``; b_major=1: ``b`` is ``[K, N]``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda and b.is_cuda
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_major == 0:
        M, K = a.shape
    else:
        K, M = a.shape
    if b_major == 0:
        N, Kb = b.shape
    else:
        Kb, N = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    flags = 0
    if out is None:
        out = (torch.zeros if atomic else torch.empty)((M, N), dtype=out_dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    if out.dtype == torch.float32:
        flags |= EPI_OUT_F32
    else:
        assert out.dtype == torch.bfloat16
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.numel() == N
        flags |= EPI_BIAS
    if gelu:
        flags |= EPI_GELU
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.shape == (M, N) and residual.stride(1) == 1
        flags |= EPI_RESIDUAL
    if preact_out is not None:
        assert preact_out.dtype == torch.bfloat16 and preact_out.shape == (M, N) and preact_out.stride(0) == out.stride(0)
        flags |= EPI_STORE_PREACT
    if dgelu_aux is not None:
        assert dgelu_aux.dtype == torch.bfloat16 and dgelu_aux.shape == (M, N) and dgelu_aux.stride(0) == out.stride(0)
        flags |= EPI_MUL_DGELU
    if atomic:
        flags |= EPI_ATOMIC
    if accumulate:
        flags |= EPI_ACCUM
    tuner = _env_autotune()
    if (tuner is not None and bn == 0 and raster_m is None and not atomic and not accumulate and split_k == 1
            and getattr(b, "_tb_fsdp_unit", None) is None and not torch.cuda.is_current_stream_capturing()):
        key = f"gemm|{M}x{N}x{K}|a{a_major}b{b_major}|f{flags}"
        rec = tuner.table.get(key)
        if rec is None:
            kw = dict(a_major=a_major, b_major=b_major, out=out, bias=bias, gelu=gelu, residual=residual, preact_out=preact_out,
                      dgelu_aux=dgelu_aux)
            cands = {f"bn{tbn}_r{int(r)}": (lambda tbn=tbn, r=r: gemm(a, b, bn=tbn, raster_m=r, **kw))
                     for tbn in (128, 256) for r in (False, True)}
            choice = tuner.select(key, cands)
        else:
            choice = rec.choice
        bn, raster_m = int(choice[2:5]), choice.endswith("_r1")
    if raster_m is None:
        raster_m = N > 4 * M or (N >= 16384 and N > M)
    if raster_m:
        flags |= EPI_RASTER_M
    st = nv.status_word(a.device)
    # FSDP full shard: the first GEMM that reads a weight of a unit whose un-shard is pending performs that un-shard
    # itself (copy CTAs of the same launch pull the shards while the tiles are computed)
    unit = getattr(b, "_tb_fsdp_unit", None)
    if unit is not None:
        g = unit[0].take_pending_gather(unit[1], b, fusable=(a_major == 0 and not atomic and not accumulate and split_k == 1))
        if g is not None:
            rc = _lib().tb_fsdp_ag_gemm(
                a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a_major, b_major, a.stride(0), b.stride(0),
                out.stride(0), nv.ptr(bias), nv.ptr(residual), residual.stride(0) if residual is not None else 0,
                nv.ptr(preact_out), nv.ptr(dgelu_aux), flags, bn, *g, st.data_ptr(), nv.stream_ptr())
            nv.check(rc, "tb_fsdp_ag_gemm")
            nv.launch_count += 2
            return out
    rc = _lib().tb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a_major, b_major, a.stride(0), b.stride(0),
        out.stride(0), nv.ptr(bias), nv.ptr(residual), residual.stride(0) if residual is not None else 0,
        nv.ptr(preact_out), nv.ptr(dgelu_aux), flags, split_k, bn, st.data_ptr(), nv.stream_ptr())
    nv.check(rc, "tb_gemm_bf16")
    nv.launch_count += 1
    return out
