"""Algorithm choice, cache blocking and cross-configuration validation for tensor operations (``crates/torsh-tensor/src``):
alternative algorithms with crossover selection — Strassen multiplication, Winograd ``F(2x2, 3x3)`` and FFT convolution,
pairwise and compensated summation (``algorithmic_optimizations.rs``); tile sizes from the cache hierarchy and blocked
loops (``cache_optimization.rs``); a tuner that measures candidates per problem class and persists its table
(``adaptive_auto_tuner.rs``); a bottleneck profiler that classifies operations against measured machine balance
(``ultra_performance_profiler.rs``); validation of an operation across dtypes, layouts and devices
(``cross_platform_validator.rs``); a coordinator that applies all of these to a workload description
(``ultimate_integration_optimizer.rs``, ``optimization_cli.rs``); bfloat16 helpers (``bfloat16_ops.rs``) and an operation log
(``operation_logging.rs``)."""
from __future__ import annotations

import json
import math
import statistics
import time
from collections import Counter, defaultdict
from pathlib import Path
from typing import Callable, Sequence

import torch
import torch.nn.functional as F


# ================================================================================================ algorithms
def strassen_matmul(a: torch.Tensor, b: torch.Tensor, leaf: int = 64) -> torch.Tensor:
    """Seven recursive products instead of eight (``O(n^2.81)``); odd sizes are padded by one; below ``leaf`` the library product
    runs.  Loses about one digit per recursion level compared with the classical product."""
    n, k, m = a.shape[0], a.shape[1], b.shape[1]
    if min(n, k, m) <= leaf:
        return a @ b
    pad = lambda t, r, c: F.pad(t, (0, c, 0, r))
    a2, b2 = pad(a, n % 2, k % 2), pad(b, k % 2, m % 2)
    h, kk, w = a2.shape[0] // 2, a2.shape[1] // 2, b2.shape[1] // 2
    a11, a12, a21, a22 = a2[:h, :kk], a2[:h, kk:], a2[h:, :kk], a2[h:, kk:]
    b11, b12, b21, b22 = b2[:kk, :w], b2[:kk, w:], b2[kk:, :w], b2[kk:, w:]
    s = lambda x, y: strassen_matmul(x, y, leaf)
    m1, m2, m3, m4 = s(a11 + a22, b11 + b22), s(a21 + a22, b11), s(a11, b12 - b22), s(a22, b21 - b11)
    m5, m6, m7 = s(a11 + a12, b22), s(a21 - a11, b11 + b12), s(a12 - a22, b21 + b22)
    top = torch.cat([m1 + m4 - m5 + m7, m3 + m5], 1)
    bot = torch.cat([m2 + m4, m1 - m2 + m3 + m6], 1)
    return torch.cat([top, bot])[:n, :m]


_WG, _WB, _WA = torch.tensor([[1.0, 0, 0], [0.5, 0.5, 0.5], [0.5, -0.5, 0.5], [0, 0, 1.0]]), torch.tensor([[1.0, 0, -1, 0], [0, 1, 1, 0], [0, -1, 1, 0], [0, 1, 0, -1]]), torch.tensor([[1.0, 1, 1, 0], [0, 1, -1, -1]])


def winograd_conv2d(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``F(2x2, 3x3)`` Winograd convolution (stride 1, no padding): 16 multiplications per 2x2 output tile instead of 36.  The
    transformed filter ``G g G^T`` and input tiles ``B^T d B`` are multiplied element-wise and summed over input channels as one
    batched product per transform position."""
    N, C, H, W = x.shape
    O = w.shape[0]
    oh, ow = H - 2, W - 2
    th, tw = math.ceil(oh / 2), math.ceil(ow / 2)
    xp = F.pad(x, (0, 2 * tw + 2 - W, 0, 2 * th + 2 - H))
    G, B, A = _WG.to(x), _WB.to(x), _WA.to(x)
    U = G @ w @ G.T                                                                  # [O, C, 4, 4]
    tiles = xp.unfold(2, 4, 2).unfold(3, 4, 2)                                        # [N, C, th, tw, 4, 4]
    V = B @ tiles @ B.T
    M = torch.einsum("ocij,ncabij->noabij", U, V)
    Y = A @ M @ A.T                                                                  # [N, O, th, tw, 2, 2]
    return Y.permute(0, 1, 2, 4, 3, 5).reshape(N, O, 2 * th, 2 * tw)[:, :, :oh, :ow]


def fft_conv2d(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Cross-correlation (what ``conv2d`` computes) by pointwise products in the frequency domain; pays off for large kernels."""
    H, W = x.shape[-2:]
    kh, kw = w.shape[-2:]
    fh, fw = H + kh - 1, W + kw - 1
    X = torch.fft.rfft2(x, s=(fh, fw))
    Wf = torch.fft.rfft2(w.flip(-1, -2), s=(fh, fw))
    y = torch.fft.irfft2(torch.einsum("nchw,ochw->nohw", X, Wf), s=(fh, fw))
    return y[..., kh - 1:H, kw - 1:W]


def choose_conv_algorithm(kernel: int, channels: int, size: int, stride: int = 1) -> str:
    """Crossover rules: Winograd for 3x3 stride-1 with enough channels to amortise the transforms, FFT for kernels of 9 and
    more on large images, implicit GEMM otherwise."""
    if kernel == 3 and stride == 1 and channels >= 16:
        return "winograd"
    if kernel >= 9 and size >= 32 and stride == 1:
        return "fft"
    return "implicit_gemm"


def pairwise_sum(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Summation by halves: the rounding error grows like ``log n`` instead of ``n`` (sequential accumulation)."""
    f = x.flatten()
    pad = (-len(f)) % block
    s = F.pad(f, (0, pad)).view(-1, block).sum(1)
    while len(s) > 1:
        if len(s) % 2:
            s = F.pad(s, (0, 1))
        s = s[0::2] + s[1::2]
    return s[0]


def kahan_sum(x: torch.Tensor, lanes: int = 1024) -> torch.Tensor:
    """Compensated summation in ``lanes`` parallel accumulators (a vectorised Kahan-Babuska loop over chunks)."""
    f = x.flatten()
    pad = (-len(f)) % lanes
    chunks = F.pad(f, (0, pad)).view(-1, lanes)
    s, c = torch.zeros(lanes, dtype=x.dtype, device=x.device), torch.zeros(lanes, dtype=x.dtype, device=x.device)
    for row in chunks:
        t = s + row
        c = c + torch.where(s.abs() >= row.abs(), (s - t) + row, (row - t) + s)
        s = t
    return (s.double() + c.double()).sum().to(x.dtype) if x.dtype != torch.float64 else pairwise_sum(s + c)       # the few lane totals are combined in double


# ================================================================================================ cache blocking
def tile_sizes(m: int, n: int, k: int, element_size: int = 4, cache_bytes: int = 1 << 20, multiple: int = 16) -> tuple[int, int, int]:
    """Largest square-ish tiles ``(tm, tn, tk)`` with ``tm tk + tk tn + tm tn`` elements inside ``cache_bytes``, multiples of
    ``multiple`` and no larger than the problem."""
    budget = cache_bytes // element_size
    t = int(math.sqrt(budget / 3)) // multiple * multiple
    t = max(multiple, t)
    return min(m, t), min(n, t), min(k, t)


def blocked_matmul(a: torch.Tensor, b: torch.Tensor, tiles: tuple[int, int, int] | None = None) -> torch.Tensor:
    tm, tn, tk = tiles or tile_sizes(a.shape[0], b.shape[1], a.shape[1], a.element_size())
    out = torch.zeros(a.shape[0], b.shape[1], dtype=torch.result_type(a, b), device=a.device)
    for i in range(0, a.shape[0], tm):
        for j in range(0, b.shape[1], tn):
            acc = out[i:i + tm, j:j + tn]
            for p in range(0, a.shape[1], tk):
                acc += a[i:i + tm, p:p + tk] @ b[p:p + tk, j:j + tn]
    return out


def memory_traffic_model(m: int, n: int, k: int, tiles: tuple[int, int, int], element_size: int = 4) -> dict:
    """Bytes moved between memory and cache by the blocked loop nest above (``A`` re-read once per column tile, ``B`` once per
    row tile) against the compulsory traffic."""
    tm, tn, tk = tiles
    a_reads = m * k * math.ceil(n / tn)
    b_reads = k * n * math.ceil(m / tm)
    c_traffic = 2 * m * n * math.ceil(k / tk)
    total, compulsory = (a_reads + b_reads + c_traffic) * element_size, (m * k + k * n + m * n) * element_size
    return {"bytes": total, "compulsory_bytes": compulsory, "reuse_factor": total / compulsory, "arithmetic_intensity": 2 * m * n * k / total}


# ================================================================================================ tuner
class AdaptiveTuner:
    """Measures candidate implementations once per problem class (operation, rounded log-sizes, dtype), answers later calls
    from its table, and can save / load the table."""

    def __init__(self, repeats: int = 3, clock=time.perf_counter): self.repeats, self.clock, self.table, self.measurements = repeats, clock, {}, 0
    @staticmethod
    def problem_class(op: str, sizes: Sequence[int], dtype=torch.float32) -> str: return f"{op}|{','.join(str(round(math.log2(max(s, 1)))) for s in sizes)}|{str(dtype).replace('torch.', '')}"

    def select(self, op: str, sizes: Sequence[int], candidates: dict[str, Callable[[], object]], dtype=torch.float32) -> str:
        key = self.problem_class(op, sizes, dtype)
        if key in self.table:
            return self.table[key]["choice"]
        times = {}
        for name, fn in candidates.items():
            fn()
            ts = []
            for _ in range(self.repeats):
                t0 = self.clock(); fn(); ts.append(self.clock() - t0)
            times[name] = statistics.median(ts); self.measurements += 1
        best = min(times, key=times.get)
        self.table[key] = {"choice": best, "times": times}
        return best

    def save(self, path): Path(path).write_text(json.dumps(self.table, indent=1))
    def load(self, path): self.table.update(json.loads(Path(path).read_text())); return self


# ================================================================================================ bottleneck profiler
class BottleneckProfiler:
    """Measures the machine once (copy bandwidth, multiply throughput, call overhead), then classifies recorded operations
    as bound by memory, compute or per-call overhead and estimates the time each would take at the machine's limits."""

    def __init__(self, device: str = "cpu", calibrate: bool = True, bandwidth: float | None = None, flops: float | None = None, overhead: float | None = None):
        self.device, self.records = device, []
        if calibrate and (bandwidth is None or flops is None or overhead is None):
            a = torch.ones(1 << 22, device=device); b = torch.empty_like(a)
            x = torch.randn(256, 256, device=device)
            tiny = torch.ones(1, device=device)
            self.bandwidth = bandwidth or 2 * a.numel() * 4 / self._time(lambda: b.copy_(a))
            self.flops = flops or 2 * 256 ** 3 / self._time(lambda: x @ x)
            self.overhead = overhead or self._time(lambda: tiny + tiny, 20)
        else:
            self.bandwidth, self.flops, self.overhead = bandwidth, flops, overhead

    @staticmethod
    def _time(fn, repeats=5):
        fn()
        ts = []
        for _ in range(repeats):
            t0 = time.perf_counter(); fn(); ts.append(time.perf_counter() - t0)
        return min(ts)

    def record(self, name: str, seconds: float, flops: float, nbytes: float): self.records.append({"name": name, "seconds": seconds, "flops": flops, "bytes": nbytes})

    def measure(self, name: str, fn: Callable, flops: float, nbytes: float):
        self.record(name, self._time(fn, 3), flops, nbytes)

    def analyze(self) -> list[dict]:
        out = []
        for r in self.records:
            t_mem, t_cmp = r["bytes"] / self.bandwidth, r["flops"] / self.flops
            bound = max(t_mem, t_cmp, self.overhead)
            kind = "overhead" if bound == self.overhead else "memory" if t_mem >= t_cmp else "compute"
            out.append({**r, "bound": kind, "ideal_seconds": bound, "efficiency": min(1.0, bound / r["seconds"]) if r["seconds"] else 1.0, "headroom": max(0.0, r["seconds"] - bound)})
        return sorted(out, key=lambda d: -d["headroom"])

    def report(self) -> str:
        rows = self.analyze()
        total = sum(r["seconds"] for r in rows) or 1.0
        lines = [f"machine: {self.bandwidth / 1e9:.1f} GB/s, {self.flops / 1e9:.1f} GFLOP/s, {self.overhead * 1e6:.1f} us per call", f"{'operation':<24}{'ms':>10}{'share':>8}{'bound':>10}{'eff':>7}"]
        lines += [f"{r['name']:<24}{r['seconds'] * 1e3:>10.3f}{r['seconds'] / total:>8.0%}{r['bound']:>10}{r['efficiency']:>7.0%}" for r in rows]
        return "\n".join(lines)


# ================================================================================================ validation across configurations
def validate_across_configurations(fn: Callable[..., torch.Tensor], make_inputs: Callable[[torch.Generator], Sequence[torch.Tensor]], dtypes=(torch.float64, torch.float32, torch.bfloat16, torch.float16), layouts=("contiguous", "transposed", "strided"),
                                   devices: Sequence[str] | None = None, seed: int = 0) -> dict:
    """Runs ``fn`` on the same data in every combination of dtype, memory layout and device and compares with the float64
    contiguous host result; tolerances follow the dtype's precision.  Catches kernels that assume contiguity or mishandle a
    dtype."""
    devices = list(devices or (["cpu"] + (["cuda"] if torch.cuda.is_available() else [])))
    g = torch.Generator().manual_seed(seed)
    base = [t.double() if t.is_floating_point() else t for t in make_inputs(g)]
    ref = fn(*base)
    tol = {torch.float64: 1e-10, torch.float32: 1e-4, torch.bfloat16: 5e-2, torch.float16: 5e-3}
    def relayout(t, how):
        if how == "contiguous" or t.dim() < 2:
            return t.contiguous()
        if how == "transposed":
            return t.transpose(-1, -2).contiguous().transpose(-1, -2)
        big = torch.zeros(*t.shape[:-1], t.shape[-1] * 2, dtype=t.dtype, device=t.device)
        big[..., ::2] = t
        return big[..., ::2]
    rows, failures = [], []
    for dev in devices:
        for dt in dtypes:
            for lay in layouts:
                ins = [relayout((t.to(dt) if t.is_floating_point() else t).to(dev), lay) for t in base]
                try:
                    out = fn(*ins)
                    scale = float(ref.abs().max()) or 1.0
                    err = float((out.double().cpu() - ref).abs().max()) / scale
                    ok = err <= tol[dt] * 10 and out.dtype == dt
                    row = {"device": dev, "dtype": str(dt).replace("torch.", ""), "layout": lay, "relative_error": err, "ok": ok}
                except Exception as e:                                              # an unsupported combination is a finding, not a crash
                    row = {"device": dev, "dtype": str(dt).replace("torch.", ""), "layout": lay, "error": f"{type(e).__name__}: {e}", "ok": False}
                rows.append(row)
                if not row["ok"]:
                    failures.append(row)
    return {"passed": not failures, "checked": len(rows), "failures": failures, "rows": rows}


# ================================================================================================ coordinator
def optimize_workload(description: dict, cache_bytes: int = 1 << 20) -> dict:
    """Plan for a workload ``{"matmuls": [(m, n, k), ...], "convs": [(kernel, channels, size), ...], "reductions": [numel, ...],
    "dtype": ...}``: algorithm and tile choices, summation method, precision advice, with the reasons."""
    plan = {"matmul": [], "conv": [], "reduction": [], "notes": []}
    es = torch.empty(0, dtype=description.get("dtype", torch.float32)).element_size()
    for m, n, k in description.get("matmuls", []):
        tiles = tile_sizes(m, n, k, es, cache_bytes)
        algo = "strassen" if min(m, n, k) >= 2048 and description.get("allow_fast_algorithms") else "blocked" if m * n * k * es > 8 * cache_bytes else "direct"
        plan["matmul"].append({"shape": (m, n, k), "algorithm": algo, "tiles": tiles, **memory_traffic_model(m, n, k, tiles, es)})
    for kernel, ch, size in description.get("convs", []):
        plan["conv"].append({"kernel": kernel, "channels": ch, "size": size, "algorithm": choose_conv_algorithm(kernel, ch, size)})
    for numel in description.get("reductions", []):
        plan["reduction"].append({"numel": numel, "method": "kahan" if numel > 1 << 24 and es <= 4 else "pairwise" if numel > 1 << 16 else "direct"})
    if description.get("dtype") in (torch.float16, torch.bfloat16):
        plan["notes"].append("accumulate reductions and matrix products in float32; keep master weights in float32")
    if any(p["reuse_factor"] > 4 for p in plan["matmul"]):
        plan["notes"].append("some products move more than four times their compulsory traffic: raise the cache budget or the tile size")
    return plan


# ================================================================================================ bfloat16 helpers and operation log
def bf16_round(x: torch.Tensor, mode: str = "nearest", generator: torch.Generator | None = None) -> torch.Tensor:
    """float32 -> bfloat16 by bit manipulation: ``nearest`` (ties to even, what hardware does), ``truncate``, or ``stochastic``
    (unbiased: the discarded 16 bits decide the rounding probability)."""
    bits = x.float().contiguous().view(torch.int32)
    if mode == "truncate":
        r = bits & ~0xFFFF
    elif mode == "nearest":
        r = (bits + 0x7FFF + ((bits >> 16) & 1)) & ~0xFFFF
    elif mode == "stochastic":
        r = (bits + torch.randint(0, 1 << 16, bits.shape, generator=generator, dtype=torch.int32)) & ~0xFFFF
    else:
        raise ValueError(mode)
    out = r.view(torch.float32)
    return torch.where(torch.isfinite(x.float()), out, x.float()).to(torch.bfloat16)


def bf16_error_bound(k: int) -> float:
    """Worst-case relative error of a length-``k`` dot product with bfloat16 inputs and float32 accumulation."""
    return 2 * 2.0 ** -8 + k * 2.0 ** -24


class OperationLog:
    """Structured log of tensor operations (name, shapes, dtype, duration) through a ``__torch_function__`` mode, with filters
    and a summary per operation."""

    def __init__(self, capacity: int = 10000, only: Sequence[str] | None = None): self.capacity, self.only, self.entries = capacity, set(only) if only else None, []

    def __enter__(self):
        log = self
        class _Mode(torch.overrides.TorchFunctionMode):
            def __torch_function__(self, func, types, args=(), kwargs=None):
                name = getattr(func, "__name__", str(func))
                t0 = time.perf_counter()
                out = func(*args, **(kwargs or {}))
                if (log.only is None or name in log.only) and len(log.entries) < log.capacity and not name.startswith("__get"):
                    shapes = [tuple(a.shape) for a in args if isinstance(a, torch.Tensor)]
                    log.entries.append({"op": name, "shapes": shapes, "dtype": str(out.dtype).replace("torch.", "") if isinstance(out, torch.Tensor) else None, "seconds": time.perf_counter() - t0})
                return out
        self._mode = _Mode(); self._mode.__enter__()
        return self

    def __exit__(self, *a): self._mode.__exit__(*a); return False
    def summary(self) -> dict:
        by = defaultdict(list)
        for e in self.entries:
            by[e["op"]].append(e["seconds"])
        return {k: {"count": len(v), "total_seconds": sum(v)} for k, v in sorted(by.items(), key=lambda kv: -sum(kv[1]))}
    def to_jsonl(self) -> str: return "".join(json.dumps(e) + "\n" for e in self.entries)
