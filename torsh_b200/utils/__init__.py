"""Utilities: profiler, metrics, environment report, benchmarking helpers."""
from . import metric_objects, metrics, profiler
from .metrics import MetricsLogger
from .profiler import CommunicationProfiler, Profiler, profile_block


def collect_env() -> dict:
    """Environment report (``crates/torsh-utils/src/collect_env.rs``)."""
    import platform
    import sys

    import torch
    info = {"python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__,
            "cuda_runtime": torch.version.cuda, "cuda_available": torch.cuda.is_available(), "gpus": []}
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            info["gpus"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                                 "memory_gb": round(p.total_memory / 2 ** 30, 1)})
        info["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
    from .. import _build
    info["native_libs"] = sorted(p.name for p in _build.LIBDIR.glob("*.so"))
    return info


def benchmark(fn, warmup: int = 3, iters: int = 10) -> dict:
    """Median / min device time of ``fn`` (CUDA events when a GPU is present, wall clock otherwise)."""
    import time

    import torch
    for _ in range(warmup):
        fn()
    ts = []
    if torch.cuda.is_available():
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); b.synchronize()
            ts.append(a.elapsed_time(b))
    else:
        for _ in range(iters):
            t0 = time.perf_counter(); fn(); ts.append((time.perf_counter() - t0) * 1e3)
    ts.sort()
    return {"median_ms": ts[len(ts) // 2], "min_ms": ts[0], "max_ms": ts[-1], "iters": iters}
