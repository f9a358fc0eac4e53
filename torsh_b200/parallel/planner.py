"""Python face of the native planner (``csrc/host/planner.cpp``): DDP buckets, FSDP shard ranges,
3-D rank mapping and pipeline schedules."""
from __future__ import annotations

import ctypes

from .. import _native as nv

_cfg = False


def _lib():
    global _cfg
    lib = nv.host()
    if not _cfg:
        i, i64 = ctypes.c_int, ctypes.c_int64
        lib.tsh_ddp_assign_buckets.argtypes = [ctypes.POINTER(i64), i, i64, ctypes.POINTER(ctypes.c_int32)]
        lib.tsh_fsdp_shard_range.argtypes = [i64, i, i, ctypes.POINTER(i64), ctypes.POINTER(i64)]
        lib.tsh_rank_of.argtypes = [i] * 7
        lib.tsh_coords_of.argtypes = [i] * 5 + [ctypes.POINTER(i)] * 3
        lib.tsh_pipeline_schedule.argtypes = [i, i, i, i, ctypes.POINTER(ctypes.c_int32), i]
        lib.tsh_pipeline_peak_inflight.argtypes = [i, i, i, i]
        lib.tsh_pipeline_schedule_interleaved.argtypes = [i, i, i, i, ctypes.POINTER(ctypes.c_int32), i]
        _cfg = True
    return lib


def assign_buckets(param_bytes: list[int], cap_bytes: int = 25 * 1024 * 1024) -> list[int]:
    """Bucket index per parameter: largest first, greedy fill (``crates/torsh-distributed/src/ddp.rs:268-327``)."""
    n = len(param_bytes)
    if n == 0:
        return []
    arr = (ctypes.c_int64 * n)(*param_bytes)
    out = (ctypes.c_int32 * n)()
    _lib().tsh_ddp_assign_buckets(arr, n, cap_bytes, out)
    return list(out)


def shard_range(numel: int, world: int, rank: int) -> tuple[int, int]:
    s, e = ctypes.c_int64(), ctypes.c_int64()
    _lib().tsh_fsdp_shard_range(numel, world, rank, ctypes.byref(s), ctypes.byref(e))
    return s.value, e.value


def rank_of(dp: int, tp: int, pp: int, dp_size: int, tp_size: int, pp_size: int, tp_fastest: bool = False) -> int:
    return _lib().tsh_rank_of(dp, tp, pp, dp_size, tp_size, pp_size, int(tp_fastest))


def coords_of(rank: int, dp_size: int, tp_size: int, pp_size: int, tp_fastest: bool = False) -> tuple[int, int, int]:
    d, t, p = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    if _lib().tsh_coords_of(rank, dp_size, tp_size, pp_size, int(tp_fastest), ctypes.byref(d), ctypes.byref(t), ctypes.byref(p)) != 0:
        raise ValueError(f"rank {rank} outside the {dp_size}x{tp_size}x{pp_size} mesh")
    return d.value, t.value, p.value


def pipeline_schedule(schedule: str, stage: int, num_stages: int, num_micro: int) -> list[tuple[str, int]]:
    """``[("F", mb) | ("B", mb), ...]`` for ``gpipe`` or ``1f1b``."""
    cap = 2 * num_micro
    buf = (ctypes.c_int32 * (2 * cap))()
    n = _lib().tsh_pipeline_schedule(0 if schedule == "gpipe" else 1, stage, num_stages, num_micro, buf, cap)
    if n < 0:
        raise ValueError("bad pipeline schedule arguments")
    return [("F" if buf[2 * i] == 0 else "B", buf[2 * i + 1]) for i in range(n)]


def pipeline_schedule_interleaved(stage: int, num_stages: int, num_micro: int, num_chunks: int) -> list[tuple[str, int, int]]:
    """``[("F" | "B", micro_batch, chunk), ...]`` of the interleaved 1F1B schedule over ``num_chunks`` virtual stages per
    rank (``num_micro`` must be a multiple of ``num_stages``)."""
    cap = 2 * num_micro * num_chunks
    buf = (ctypes.c_int32 * (3 * cap))()
    n = _lib().tsh_pipeline_schedule_interleaved(stage, num_stages, num_micro, num_chunks, buf, cap)
    if n < 0:
        raise ValueError("interleaved schedule: num_micro must be a positive multiple of num_stages")
    return [("F" if buf[3 * i] == 0 else "B", buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)]


def pipeline_peak_inflight(schedule: str, stage: int, num_stages: int, num_micro: int) -> int:
    return _lib().tsh_pipeline_peak_inflight(0 if schedule == "gpipe" else 1, stage, num_stages, num_micro)
