"""Performance tooling for sparse tensors (``crates/torsh-sparse/src``): operation profiler with statistics, trends, regressions
and CSV / JSON export (``performance_tools/core.rs``, ``performance_tools/reporting.rs``, ``performance_tools/export/``), memory
analysis per format with compression effectiveness (``performance_tools/memory.rs``, ``memory_management.rs``), format
recommendation from structure and measured format comparison with a learning auto-tuner
(``performance_tools/optimization/``, ``unified_interface.rs``), cache-behaviour probes (``performance/``) and specialised kernels
expressed as segment reductions: CSR times dense, blocked CSR, sampled dense-dense products and fused row operations
(``custom_kernels.rs``)."""
from __future__ import annotations

import csv
import io
import json
import math
import statistics
import time
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch

from .sparse import BsrTensor, CooTensor, CsrTensor, DiaTensor, EllTensor


# ================================================================================================ kernels
def csr_spmm(crow: torch.Tensor, col: torch.Tensor, val: torch.Tensor, dense: torch.Tensor) -> torch.Tensor:
    """``A @ B`` for CSR ``A``: gather the rows of ``B`` named by the column indices, scale, and reduce each row's segment
    (one pass, no intermediate COO row index in memory beyond the segment ids)."""
    n = len(crow) - 1
    rows = torch.repeat_interleave(torch.arange(n, device=val.device), crow[1:] - crow[:-1])
    out = torch.zeros(n, *dense.shape[1:], dtype=torch.result_type(val, dense), device=val.device)
    return out.index_add_(0, rows, val.reshape(-1, *[1] * (dense.dim() - 1)) * dense[col])


def csr_spmm_blocked(crow, col, val, dense, row_block: int = 1024) -> torch.Tensor:
    """The same product in row blocks, so that the gathered ``nnz x k`` intermediate never exceeds one block (for wide ``B``)."""
    n, outs = len(crow) - 1, []
    for r0 in range(0, n, row_block):
        r1 = min(n, r0 + row_block)
        a, b = int(crow[r0]), int(crow[r1])
        outs.append(csr_spmm(crow[r0:r1 + 1] - crow[r0], col[a:b], val[a:b], dense))
    return torch.cat(outs)


def sddmm(crow, col, a: torch.Tensor, b: torch.Tensor, scale: torch.Tensor | None = None) -> torch.Tensor:
    """Sampled dense-dense product: ``(A B^T)`` evaluated only at the stored positions (the attention-score and graph-attention
    kernel); optionally multiplied by the stored values."""
    rows = torch.repeat_interleave(torch.arange(len(crow) - 1, device=col.device), crow[1:] - crow[:-1])
    v = (a[rows] * b[col]).sum(-1)
    return v if scale is None else v * scale


def csr_row_softmax(crow, val: torch.Tensor) -> torch.Tensor:
    """Softmax over each row's stored entries (segment max, exponentiate, segment sum)."""
    n = len(crow) - 1
    rows = torch.repeat_interleave(torch.arange(n, device=val.device), crow[1:] - crow[:-1])
    mx = torch.full((n,), -math.inf, dtype=val.dtype, device=val.device).scatter_reduce(0, rows, val, "amax")
    e = torch.exp(val - mx[rows])
    return e / torch.zeros(n, dtype=val.dtype, device=val.device).index_add_(0, rows, e)[rows]


def csr_row_reduce(crow, val: torch.Tensor, op: str = "sum") -> torch.Tensor:
    n = len(crow) - 1
    rows = torch.repeat_interleave(torch.arange(n, device=val.device), crow[1:] - crow[:-1])
    if op == "sum":
        return torch.zeros(n, dtype=val.dtype, device=val.device).index_add_(0, rows, val)
    if op == "norm2":
        return torch.zeros(n, dtype=val.dtype, device=val.device).index_add_(0, rows, val * val).sqrt()
    if op in ("max", "min"):
        init = -math.inf if op == "max" else math.inf
        return torch.full((n,), init, dtype=val.dtype, device=val.device).scatter_reduce(0, rows, val, "amax" if op == "max" else "amin")
    raise ValueError(op)


def apply_with_threshold(val: torch.Tensor, fn: Callable[[torch.Tensor], torch.Tensor], threshold: float = 0.0) -> tuple[torch.Tensor, torch.Tensor]:
    """Applies ``fn`` to the stored values and reports which results fall below ``threshold`` in magnitude (to be dropped)."""
    out = fn(val)
    return out, out.abs() > threshold


def sparse_attention(crow, col, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Attention restricted to a CSR pattern: sampled scores, row softmax, sparse-times-dense."""
    s = sddmm(crow, col, q, k) / math.sqrt(q.shape[-1])
    return csr_spmm(crow, col, csr_row_softmax(crow, s), v)


# ================================================================================================ profiler
@dataclass
class Measurement:
    operation: str
    seconds: float
    nnz: int = 0
    bytes: int = 0
    step: int = 0
    metadata: dict = field(default_factory=dict)


class SparseProfiler:
    def __init__(self, clock=time.perf_counter): self.clock, self.measurements, self.step_no = clock, [], 0

    def track(self, operation: str, fn: Callable, *args, nnz: int = 0, nbytes: int = 0, **metadata):
        t0 = self.clock(); out = fn(*args); dt = self.clock() - t0
        self.measurements.append(Measurement(operation, dt, nnz, nbytes, self.step_no, metadata)); self.step_no += 1
        return out

    def add(self, m: Measurement): self.measurements.append(m); self.step_no = max(self.step_no, m.step + 1)
    def for_operation(self, op: str) -> list[Measurement]: return [m for m in self.measurements if m.operation == op]

    def statistics(self, op: str) -> dict:
        t = [m.seconds for m in self.for_operation(op)]
        if not t:
            return {"count": 0}
        mean = statistics.fmean(t)
        cv = statistics.pstdev(t) / mean if mean else 0.0
        nnz = statistics.fmean(m.nnz for m in self.for_operation(op))
        return {"count": len(t), "mean": mean, "min": min(t), "max": max(t), "cv": cv, "consistent": cv < 0.1, "nnz_per_second": nnz / mean if mean else 0.0, "operations_per_second": 1 / mean if mean else 0.0}

    def trend(self, op: str) -> dict:
        """Least-squares slope of time against step, relative to the mean: ``degrading`` above +1 % per step, ``improving`` below."""
        ms = self.for_operation(op)
        if len(ms) < 3:
            return {"direction": "unknown", "slope": 0.0}
        xs, ys = [m.step for m in ms], [m.seconds for m in ms]
        mx, my = statistics.fmean(xs), statistics.fmean(ys)
        slope = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / max(sum((x - mx) ** 2 for x in xs), 1e-30)
        rel = slope / my if my else 0.0
        return {"direction": "degrading" if rel > 0.01 else "improving" if rel < -0.01 else "stable", "slope": slope, "relative_slope": rel}

    def detect_regressions(self, baseline: "SparseProfiler", tolerance: float = 0.2) -> list[dict]:
        out = []
        for op in sorted({m.operation for m in self.measurements}):
            a, b = baseline.statistics(op), self.statistics(op)
            if a.get("count") and b["mean"] > a["mean"] * (1 + tolerance):
                out.append({"operation": op, "baseline": a["mean"], "current": b["mean"], "slowdown": b["mean"] / a["mean"]})
        return out

    def fastest(self, ops: Sequence[str] | None = None) -> str: return min(ops or {m.operation for m in self.measurements}, key=lambda o: self.statistics(o)["mean"])
    def top_by_throughput(self, k: int = 3) -> list[str]: return sorted({m.operation for m in self.measurements}, key=lambda o: -self.statistics(o)["nnz_per_second"])[:k]

    def to_csv(self) -> str:
        buf = io.StringIO(); w = csv.writer(buf)
        w.writerow(["operation", "step", "seconds", "nnz", "bytes"])
        w.writerows([m.operation, m.step, f"{m.seconds:.9g}", m.nnz, m.bytes] for m in self.measurements)
        return buf.getvalue()

    def to_json(self) -> str: return json.dumps({"measurements": [m.__dict__ for m in self.measurements], "summary": {o: self.statistics(o) for o in sorted({m.operation for m in self.measurements})}})

    def report(self) -> str:
        ops = sorted({m.operation for m in self.measurements})
        lines = [f"{'operation':<24}{'n':>5}{'mean ms':>12}{'cv':>8}{'Mnnz/s':>12}  trend"]
        for o in ops:
            s, t = self.statistics(o), self.trend(o)
            lines.append(f"{o:<24}{s['count']:>5}{s['mean'] * 1e3:>12.4f}{s['cv']:>8.2f}{s['nnz_per_second'] / 1e6:>12.2f}  {t['direction']}")
        return "\n".join(lines)


# ================================================================================================ memory analysis
def format_bytes(shape: tuple[int, int], nnz: int, fmt: str, value_bytes: int = 4, index_bytes: int = 8, block: int = 4, max_row_nnz: int | None = None, diagonals: int | None = None, filled_blocks: int | None = None) -> int:
    m, n = shape
    if fmt == "dense":
        return m * n * value_bytes
    if fmt == "coo":
        return nnz * (value_bytes + 2 * index_bytes)
    if fmt == "csr":
        return nnz * (value_bytes + index_bytes) + (m + 1) * index_bytes
    if fmt == "csc":
        return nnz * (value_bytes + index_bytes) + (n + 1) * index_bytes
    if fmt == "ell":
        return m * (max_row_nnz if max_row_nnz is not None else math.ceil(nnz / max(m, 1))) * (value_bytes + index_bytes)
    if fmt == "dia":
        return (diagonals if diagonals is not None else min(m, n)) * (min(m, n) * value_bytes + index_bytes)
    if fmt == "bsr":
        nb = filled_blocks if filled_blocks is not None else math.ceil(nnz / (block * block))
        return nb * (block * block * value_bytes + index_bytes) + (math.ceil(m / block) + 1) * index_bytes
    raise ValueError(fmt)


def structure_profile(dense_or_coo) -> dict:
    """Numbers that decide the format: density, row-length spread, number of occupied diagonals, block fill."""
    d = dense_or_coo.to_dense() if hasattr(dense_or_coo, "to_dense") and not isinstance(dense_or_coo, torch.Tensor) else dense_or_coo
    nz = d != 0
    m, n = d.shape
    rows = nz.sum(1)
    r, c = nz.nonzero(as_tuple=True)
    diags = torch.unique(c - r)
    diag_fill = int(nz.sum()) / max(len(diags) * min(m, n), 1)
    bs = 4
    pm, pn = math.ceil(m / bs) * bs, math.ceil(n / bs) * bs
    padded = torch.zeros(pm, pn, dtype=torch.bool); padded[:m, :n] = nz
    blocks = padded.reshape(pm // bs, bs, pn // bs, bs).permute(0, 2, 1, 3).reshape(-1, bs * bs)
    filled = blocks.any(1)
    return {"shape": (m, n), "nnz": int(nz.sum()), "density": float(nz.float().mean()), "max_row_nnz": int(rows.max()) if m else 0, "mean_row_nnz": float(rows.float().mean()) if m else 0.0, "row_cv": float(rows.float().std() / rows.float().mean().clamp_min(1e-12)) if m > 1 else 0.0,
            "diagonals": len(diags), "diagonal_fill": diag_fill, "filled_blocks": int(filled.sum()), "block_fill": float(blocks[filled].float().mean()) if filled.any() else 0.0, "bandwidth": int((c - r).abs().max()) if len(r) else 0}


def analyze_memory(dense_or_coo, value_bytes: int = 4) -> dict:
    p = structure_profile(dense_or_coo)
    sizes = {f: format_bytes(p["shape"], p["nnz"], f, value_bytes, max_row_nnz=p["max_row_nnz"], diagonals=p["diagonals"], filled_blocks=p["filled_blocks"]) for f in ("dense", "coo", "csr", "csc", "ell", "dia", "bsr")}
    best = min((f for f in sizes if f != "dense"), key=sizes.get)
    recs = []
    if sizes[best] > 0.7 * sizes["dense"]:
        recs.append("the matrix is too dense for sparse storage to pay: keep it dense")
    if p["row_cv"] > 1.0 and sizes["ell"] > 2 * sizes["csr"]:
        recs.append("row lengths vary strongly: padded formats (ELL) waste memory, prefer CSR or a hybrid ELL + COO split")
    if p["diagonal_fill"] > 0.7:
        recs.append("entries lie on few, well-filled diagonals: DIA stores no column indices")
    if p["block_fill"] > 0.7 and p["nnz"] >= 16:
        recs.append("non-zeros cluster in dense blocks: BSR shares one index per block and maps to tensor-core tiles")
    return {"profile": p, "bytes": sizes, "most_compact": best, "compression_vs_dense": sizes["dense"] / max(sizes[best], 1), "memory_efficiency": p["nnz"] * value_bytes / max(sizes[best], 1), "recommendations": recs}


# ================================================================================================ format choice
def suggest_format(profile: dict, operation: str = "matmul") -> dict:
    """Rule-based recommendation from the structure and the dominant operation (``matmul``, ``transpose_matmul``, ``build``,
    ``elementwise``), with the reason."""
    if profile["density"] > 0.4:
        return {"format": "dense", "reason": f"density {profile['density']:.0%}: dense kernels run at full rate and indices would double the traffic"}
    if operation == "build":
        return {"format": "coo", "reason": "incremental construction appends triplets; convert once when done"}
    if profile["diagonal_fill"] > 0.7 and profile["diagonals"] <= 16:
        return {"format": "dia", "reason": f"{profile['diagonals']} well-filled diagonals"}
    if profile["block_fill"] > 0.7 and profile["nnz"] >= 64:
        return {"format": "bsr", "reason": f"blocks are {profile['block_fill']:.0%} full"}
    if operation == "transpose_matmul":
        return {"format": "csc", "reason": "column access for products with the transpose"}
    if profile["row_cv"] < 0.25 and profile["max_row_nnz"] <= 2 * max(profile["mean_row_nnz"], 1):
        return {"format": "ell", "reason": "rows have nearly equal length: padded rows give coalesced, branch-free access"}
    return {"format": "csr", "reason": "general sparse rows: compressed rows serve products and row slicing"}


_BUILDERS = {"coo": lambda d: CooTensor.from_dense(d), "csr": lambda d: CooTensor.from_dense(d).to_csr(), "ell": lambda d: EllTensor.from_dense(d), "bsr": lambda d: BsrTensor.from_dense(d, 4), "dia": lambda d: DiaTensor.from_dense(d), "dense": lambda d: d}


def compare_formats(dense: torch.Tensor, rhs: torch.Tensor, formats: Sequence[str] = ("dense", "coo", "csr", "ell", "bsr"), repeats: int = 5) -> dict:
    """Measures ``A @ rhs`` in each format (median of ``repeats``), checks the results agree and ranks the formats."""
    ref, rows = dense @ rhs, {}
    for f in formats:
        if f == "bsr" and (dense.shape[0] % 4 or dense.shape[1] % 4):
            continue
        a = _BUILDERS[f](dense)
        mm = (lambda: a @ rhs) if f == "dense" else (lambda: a.matmul(rhs))
        out = mm()
        ts = []
        for _ in range(repeats):
            t0 = time.perf_counter(); mm(); ts.append(time.perf_counter() - t0)
        rows[f] = {"seconds": statistics.median(ts), "max_error": float((out - ref).abs().max())}
    best = min(rows, key=lambda k: rows[k]["seconds"])
    return {"results": rows, "fastest": best, "ranking": sorted(rows, key=lambda k: rows[k]["seconds"])}


class FormatAutoTuner:
    """Starts from the rule-based suggestion, measures when asked, remembers the winner per structure class (density decade,
    row regularity, blockiness) and answers later queries for similar matrices from memory."""

    def __init__(self): self.memory: dict[tuple, str] = {}; self.trials = 0
    @staticmethod
    def signature(p: dict) -> tuple: return (round(math.log10(max(p["density"], 1e-9))), p["row_cv"] < 0.25, p["block_fill"] > 0.7, p["diagonal_fill"] > 0.7)

    def choose(self, dense: torch.Tensor, rhs: torch.Tensor | None = None, measure: bool = False) -> str:
        p = structure_profile(dense)
        sig = self.signature(p)
        if sig in self.memory:
            return self.memory[sig]
        if measure and rhs is not None:
            self.trials += 1
            self.memory[sig] = compare_formats(dense, rhs)["fastest"]
            return self.memory[sig]
        return suggest_format(p)["format"]

    def learn(self, profile: dict, best: str): self.memory[self.signature(profile)] = best


# ================================================================================================ cache behaviour
def benchmark_access_patterns(n: int = 1 << 20, repeats: int = 3, generator: torch.Generator | None = None) -> dict:
    """Gather with sequential, strided and random indices over the same data: the ratio is what column order costs a sparse
    product on this machine."""
    data = torch.arange(n, dtype=torch.float32)
    idx = {"sequential": torch.arange(n), "strided": (torch.arange(n) * 4099) % n, "random": torch.randperm(n, generator=generator)}
    out = {}
    for k, ix in idx.items():
        data[ix]
        ts = []
        for _ in range(repeats):
            t0 = time.perf_counter(); data[ix].sum(); ts.append(time.perf_counter() - t0)
        out[k] = {"seconds": min(ts), "gb_per_s": n * 4 / min(ts) / 1e9}
    out["random_penalty"] = out["random"]["seconds"] / out["sequential"]["seconds"]
    return out


def column_locality(crow: torch.Tensor, col: torch.Tensor, line_elems: int = 16) -> dict:
    """How cache-friendly the gather of a CSR product is: mean distance between consecutive column indices within rows and
    the share of consecutive accesses that stay in one cache line of the right-hand side."""
    rows = torch.repeat_interleave(torch.arange(len(crow) - 1), crow[1:] - crow[:-1])
    same = rows[1:] == rows[:-1]
    gap = (col[1:] - col[:-1]).abs()[same]
    return {"mean_gap": float(gap.float().mean()) if len(gap) else 0.0, "same_line_fraction": float((gap < line_elems).float().mean()) if len(gap) else 1.0}
