"""The single backend of this package, described in the reference's terms
(``crates/torsh-backend/src/backend.rs:17-203,367-586``: ``capabilities()`` / ``performance_hints()``;
``src/cuda/tensor_cores.rs:22-131``: the tensor-core capability table, here for the 5th-generation ``tcgen05`` kinds
instead of Volta…Hopper ``wmma`` tiles; ``src/cuda/backend.rs:43-292``: builder / config), plus a measuring autotuner
(``adaptive_kernel_selection.rs``, ``performance_tuning/*``) whose choices persist in a JSON table."""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field


@dataclass(frozen=True)
class TensorCoreKind:
    """One ``tcgen05.mma`` kind: operand types, accumulator, dense peak per GPU and the instruction's tile limits."""
    name: str
    a_types: tuple[str, ...]
    accumulator: str
    dense_tflops: float
    m: tuple[int, ...]            # M per CTA (cta_group::1); cta_group::2 doubles it across the CTA pair
    n_max: int
    k: int                        # K of one instruction


TENSOR_CORE_KINDS = {
    "f16": TensorCoreKind("kind::f16", ("f16", "bf16"), "f32", 2250.0, (64, 128), 256, 16),
    "tf32": TensorCoreKind("kind::tf32", ("tf32",), "f32", 1100.0, (64, 128), 256, 8),
    "f8f6f4": TensorCoreKind("kind::f8f6f4", ("e4m3", "e5m2", "e2m3", "e3m2", "e2m1"), "f32", 4500.0, (64, 128), 256, 32),
    "i8": TensorCoreKind("kind::i8", ("s8", "u8"), "s32", 4500.0, (64, 128), 256, 32),
    "mxf4": TensorCoreKind("kind::mxf4", ("e2m1 (block-scaled)",), "f32", 9000.0, (128,), 256, 64),
}


@dataclass
class BackendCapabilities:
    name: str = "cuda-sm100a"
    compute_capability: tuple[int, int] = (10, 0)
    sm_count: int = 148
    warp_size: int = 32
    shared_memory_per_block: int = 227 * 1024
    tensor_memory_columns: int = 512
    l2_bytes: int = 126 << 20
    hbm_bytes: int = 180 << 30
    max_cluster_size: int = 8
    dtypes: tuple[str, ...] = ("bf16", "f16", "f32", "f64", "i8", "i32", "i64", "u8", "bool", "e4m3", "e5m2")
    tensor_cores: tuple[str, ...] = tuple(TENSOR_CORE_KINDS)
    features: tuple[str, ...] = ("tma", "tcgen05", "tmem", "clusters", "cuda_graphs", "nvls_multimem", "peer_memory",
                                 "stream_ordered_pools", "pinned_memory")
    unsupported: tuple[str, ...] = ("wgmma (sm_90a only)", "graphics interop")


@dataclass
class PerformanceHints:
    """What a caller should do to run well on this backend (``performance_hints()``)."""
    preferred_dtype: str = "bf16"
    gemm_tile: tuple[int, int, int] = (128, 256, 64)
    grid_multiple: int = 148
    min_bytes_for_nvls: int = 128 << 10
    tma_alignment_bytes: int = 16
    hbm_gbs: float = 6650.0
    bf16_tflops: float = 1590.0
    notes: tuple[str, ...] = (
        "fuse element-wise work into the producing GEMM epilogue",
        "size grids as a multiple of the SM count or run persistent kernels",
        "capture launch-bound loops in CUDA graphs",
        "keep inputs larger than the 126 MB L2 when timing memory-bound kernels",
    )


def capabilities(device: int | None = None) -> BackendCapabilities:
    """Static description refined with what the device reports (when there is one)."""
    caps = BackendCapabilities()
    try:
        import torch
        if torch.cuda.is_available():
            from .runtime import device_info
            info = device_info(device)
            caps = BackendCapabilities(name=f"cuda-sm{info.capability[0]}{info.capability[1]}a", compute_capability=info.capability,
                                       sm_count=info.sm_count, warp_size=info.warp_size,
                                       shared_memory_per_block=info.smem_per_block_optin,
                                       tensor_memory_columns=info.tmem_columns, l2_bytes=info.l2_bytes,
                                       hbm_bytes=info.total_memory)
    except Exception:
        pass
    return caps


def performance_hints(peaks_file: str | None = None) -> PerformanceHints:
    """Roofline denominators come from a measured-peaks JSON file (``hbm_gbs``, ``bf16_tflops``) when one is given or
    ``TORSH_MEASURED_PEAKS`` names one; otherwise from the defaults."""
    hints = PerformanceHints()
    path = peaks_file or os.environ.get("TORSH_MEASURED_PEAKS")
    if path and os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        hints.hbm_gbs = float(d.get("hbm_gbs", hints.hbm_gbs))
        hints.bf16_tflops = float(d.get("bf16_tflops", hints.bf16_tflops))
    return hints


@dataclass
class CudaBackendConfig:
    """``CudaBackendBuilder`` fields (``crates/torsh-backend/src/cuda/backend.rs:43-292``)."""
    device_id: int = 0
    memory_pool_limit_bytes: int = 0
    allow_tf32: bool = True
    enable_profiling: bool = False
    stream_pool_size: int = 4
    use_as_torch_allocator: bool = False

    def apply(self):
        import torch
        if torch.cuda.is_available():
            torch.cuda.set_device(self.device_id)
            torch.backends.cuda.matmul.allow_tf32 = self.allow_tf32
            from . import runtime as rt
            if self.memory_pool_limit_bytes:
                rt.DeviceMemoryPool.set_limit(self.memory_pool_limit_bytes)
            if self.use_as_torch_allocator:
                rt.use_as_torch_allocator()
        return self


class CudaBackendBuilder:
    def __init__(self):
        self.cfg = CudaBackendConfig()

    def device(self, i: int): self.cfg.device_id = i; return self
    def memory_pool_limit(self, n: int): self.cfg.memory_pool_limit_bytes = n; return self
    def allow_tf32(self, flag: bool): self.cfg.allow_tf32 = flag; return self
    def enable_profiling(self, flag: bool = True): self.cfg.enable_profiling = flag; return self
    def stream_pool_size(self, n: int): self.cfg.stream_pool_size = n; return self
    def build(self) -> CudaBackendConfig: return self.cfg.apply()


# ----------------------------------------------------------------------------------------------------------- autotuner
@dataclass
class TuneRecord:
    key: str
    choice: str
    times_ms: dict = field(default_factory=dict)


class Autotuner:
    """Times each candidate of a kernel configuration once per problem key and remembers the winner
    (``adaptive_kernel_selection.rs``). ``timer`` defaults to CUDA events on a GPU and ``perf_counter`` otherwise;
    the table is saved to / loaded from JSON so tuning runs offline."""

    def __init__(self, path: str | None = None, warmup: int = 2, iters: int = 5, timer=None):
        self.path, self.warmup, self.iters, self.timer = path, warmup, iters, timer
        self.table: dict[str, TuneRecord] = {}
        if path and os.path.exists(path):
            with open(path) as f:
                self.table = {k: TuneRecord(**v) for k, v in json.load(f).items()}

    def _time(self, fn) -> float:
        if self.timer is not None:
            return self.timer(fn)
        import torch
        for _ in range(self.warmup):
            fn()
        if torch.cuda.is_available():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(self.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / self.iters
        t0 = time.perf_counter()
        for _ in range(self.iters):
            fn()
        return (time.perf_counter() - t0) * 1e3 / self.iters

    def select(self, key: str, candidates: dict) -> str:
        """``candidates``: name → zero-argument callable. Returns the fastest name (cached per ``key``)."""
        rec = self.table.get(key)
        if rec is not None and rec.choice in candidates:
            return rec.choice
        times = {name: self._time(fn) for name, fn in candidates.items()}
        choice = min(times, key=times.get)
        self.table[key] = TuneRecord(key, choice, times)
        if self.path:
            self.save()
        return choice

    def save(self, path: str | None = None):
        with open(path or self.path, "w") as f:
            json.dump({k: asdict(v) for k, v in self.table.items()}, f, indent=1)
