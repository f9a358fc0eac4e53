"""Core utilities (``crates/torsh-core/src``): deprecation management (``api_compat.rs``), chunk sizing (``chunking.rs``),
lossless tensor compression and pruning metadata (``compression.rs``), stable error codes (``error_codes.rs``), IEEE 754
helpers (``ieee754_compliance.rs``), a tensor inspector (``inspector.rs``), access-pattern layout advice
(``layout_optimizer.rs``), text memory maps (``memory_visualization.rs``), MLIR and StableHLO text emission from traced
graphs (``mlir_integration.rs``, ``xla_integration/``), leaky integrate-and-fire neurons with spike coding
(``neuromorphic.rs``), matrix-product-state tensor networks (``tensor_network.rs``), shape validation with explanations
(``shape_validation.rs``, ``shape_debug.rs``), cache-oblivious index orders (``cache_oblivious.rs``) and a windowed
performance monitor (``perf_monitor.rs``, ``perf_metrics.rs``)."""
from __future__ import annotations

import functools
import math
import struct
import time
import warnings
from collections import Counter, defaultdict, deque
from typing import Callable, Sequence

import torch


# ================================================================================================ deprecation management
class ApiCompat:
    """Registry of deprecated names: ``@compat.deprecated(since, removed_in, replacement)`` warns once per call site
    category, raises after the removal version, and ``report()`` lists what a program touched."""

    def __init__(self, current_version: str = "0.1.3"): self.current, self.entries, self.used = self._v(current_version), {}, Counter()
    @staticmethod
    def _v(s): return tuple(int(p) for p in s.split(".")[:3])

    def deprecated(self, since: str, removed_in: str | None = None, replacement: str | None = None):
        def deco(fn):
            name = fn.__qualname__
            self.entries[name] = {"since": since, "removed_in": removed_in, "replacement": replacement}
            @functools.wraps(fn)
            def w(*a, **kw):
                self.used[name] += 1
                if removed_in and self.current >= self._v(removed_in):
                    raise RuntimeError(f"{name} was removed in {removed_in}" + (f"; use {replacement}" if replacement else ""))
                warnings.warn(f"{name} is deprecated since {since}" + (f" and will be removed in {removed_in}" if removed_in else "") + (f"; use {replacement}" if replacement else ""), DeprecationWarning, stacklevel=2)
                return fn(*a, **kw)
            return w
        return deco

    def report(self): return [{"name": n, **self.entries[n], "calls": c} for n, c in self.used.most_common()]


# ================================================================================================ chunking
def optimal_chunk(numel: int, element_size: int, working_tensors: int = 2, cache_bytes: int = 126 << 20, min_chunk: int = 1 << 16, align: int = 128) -> int:
    """Largest chunk (in elements, a multiple of ``align``) such that ``working_tensors`` chunks fit in ``cache_bytes``
    (the B200's L2 by default); never below ``min_chunk``, never above the tensor."""
    fit = cache_bytes // (working_tensors * element_size)
    return min(numel, max(min_chunk, fit // align * align))


def chunked_apply(fn: Callable, x: torch.Tensor, chunk: int | None = None, dim: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    rows = x.shape[dim]
    per = chunk or max(1, optimal_chunk(x.numel(), x.element_size()) // max(x.numel() // max(rows, 1), 1))
    parts = [fn(x.narrow(dim, s, min(per, rows - s))) for s in range(0, rows, per)]
    res = torch.cat(parts, dim)
    return res if out is None else out.copy_(res)


# ================================================================================================ compression
def rle_encode(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, tuple]:
    f = x.reshape(-1)
    if f.numel() == 0:
        return f, torch.zeros(0, dtype=torch.long), tuple(x.shape)
    change = torch.cat([torch.ones(1, dtype=torch.bool, device=f.device), f[1:] != f[:-1]])
    starts = change.nonzero().flatten()
    return f[starts], torch.diff(torch.cat([starts, torch.tensor([f.numel()], device=f.device)])), tuple(x.shape)


def rle_decode(values, lengths, shape): return torch.repeat_interleave(values, lengths).reshape(shape)


def delta_encode(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """First value plus differences (exact for integer tensors; sorted indices compress well afterwards)."""
    f = x.reshape(-1)
    return f[:1].clone(), f[1:] - f[:-1]


def delta_decode(first, deltas, shape): return torch.cat([first, first + deltas.cumsum(0)]).reshape(shape)


def bitmask_encode(x: torch.Tensor) -> dict:
    """Sparse storage: one bit per element marks non-zeros, followed by the non-zero values."""
    f = x.reshape(-1)
    nz = f != 0
    pad = (-f.numel()) % 8
    bits = torch.cat([nz, nz.new_zeros(pad)]).reshape(-1, 8).to(torch.uint8)
    packed = (bits * (1 << torch.arange(8, dtype=torch.uint8))).sum(1).to(torch.uint8)
    return {"mask": packed, "values": f[nz].clone(), "shape": tuple(x.shape), "bytes": packed.numel() + int(nz.sum()) * x.element_size(), "dense_bytes": f.numel() * x.element_size()}


def bitmask_decode(enc: dict) -> torch.Tensor:
    n = math.prod(enc["shape"])
    bits = ((enc["mask"][:, None] >> torch.arange(8, dtype=torch.uint8)) & 1).reshape(-1)[:n].bool()
    out = torch.zeros(n, dtype=enc["values"].dtype)
    out[bits] = enc["values"]
    return out.reshape(enc["shape"])


def pruning_metadata(x: torch.Tensor, block: int = 4) -> dict:
    z = x == 0
    rows = x.reshape(-1, x.shape[-1]) if x.dim() > 1 else x.reshape(1, -1)
    usable = rows.shape[1] // block * block
    groups = (rows[:, :usable].reshape(rows.shape[0], -1, block) != 0).sum(-1)
    return {"sparsity": float(z.float().mean()), "zero_rows": int((rows == 0).all(1).sum()), "zero_columns": int((rows == 0).all(0).sum()), "is_2_4": bool(block == 4 and (groups <= 2).all()),
            "block_sparsity": float((groups == 0).float().mean())}


# ================================================================================================ error codes
ERROR_CODES = {"OK": 0, "INVALID_ARGUMENT": 1001, "SHAPE_MISMATCH": 1002, "DTYPE_MISMATCH": 1003, "DEVICE_MISMATCH": 1004, "INDEX_OUT_OF_BOUNDS": 1005, "OUT_OF_MEMORY": 2001, "ALLOCATION_FAILED": 2002,
               "DEVICE_ERROR": 3001, "DEVICE_NOT_AVAILABLE": 3002, "KERNEL_LAUNCH_FAILED": 3003, "IO_ERROR": 4001, "SERIALIZATION_ERROR": 4002, "CHECKSUM_MISMATCH": 4003, "NOT_IMPLEMENTED": 5001,
               "TIMEOUT": 6001, "COMMUNICATION_ERROR": 6002, "RANK_FAILURE": 6003, "NUMERICAL_ERROR": 7001, "INTERNAL": 9999}
_CATEGORY = {1: "user", 2: "memory", 3: "device", 4: "io", 5: "unsupported", 6: "distributed", 7: "numerical", 9: "internal", 0: "ok"}


def error_code(name: str) -> int: return ERROR_CODES[name]
def error_name(code: int) -> str: return next(k for k, v in ERROR_CODES.items() if v == code)
def error_category(code: int) -> str: return _CATEGORY[code // 1000]
def is_retryable(code: int) -> bool: return code in (ERROR_CODES["TIMEOUT"], ERROR_CODES["COMMUNICATION_ERROR"], ERROR_CODES["OUT_OF_MEMORY"])


def classify_exception(e: BaseException) -> int:
    msg = str(e).lower()
    if isinstance(e, MemoryError) or "out of memory" in msg:
        return ERROR_CODES["OUT_OF_MEMORY"]
    if isinstance(e, TimeoutError):
        return ERROR_CODES["TIMEOUT"]
    if isinstance(e, NotImplementedError):
        return ERROR_CODES["NOT_IMPLEMENTED"]
    if isinstance(e, IndexError):
        return ERROR_CODES["INDEX_OUT_OF_BOUNDS"]
    if isinstance(e, (OSError, IOError)):
        return ERROR_CODES["IO_ERROR"]
    if isinstance(e, (FloatingPointError, ZeroDivisionError, OverflowError)):
        return ERROR_CODES["NUMERICAL_ERROR"]
    if "shape" in msg or "size mismatch" in msg or "must match" in msg:
        return ERROR_CODES["SHAPE_MISMATCH"]
    if "dtype" in msg:
        return ERROR_CODES["DTYPE_MISMATCH"]
    if "cuda" in msg or "device" in msg:
        return ERROR_CODES["DEVICE_ERROR"]
    return ERROR_CODES["INVALID_ARGUMENT"] if isinstance(e, (ValueError, TypeError)) else ERROR_CODES["INTERNAL"]


# ================================================================================================ IEEE 754
def float_bits(x: float, double: bool = False) -> int: return struct.unpack("<Q" if double else "<I", struct.pack("<d" if double else "<f", x))[0]


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Units in the last place between same-dtype floats (monotone integer mapping of the bit patterns)."""
    it = {torch.float32: torch.int32, torch.float64: torch.int64, torch.float16: torch.int16, torch.bfloat16: torch.int16}[a.dtype]
    def key(t):
        i = t.contiguous().view(it).to(torch.int64)
        sign_bit = 1 << (t.element_size() * 8 - 1)
        return torch.where(i < 0, -(i + sign_bit) , i)
    return (key(a) - key(b)).abs()


def classify_floats(x: torch.Tensor) -> dict:
    tiny = torch.finfo(x.dtype).tiny
    return {"nan": int(torch.isnan(x).sum()), "inf": int(torch.isinf(x).sum()), "zero": int((x == 0).sum()), "negative_zero": int(((x == 0) & torch.signbit(x)).sum()),
            "subnormal": int(((x != 0) & (x.abs() < tiny)).sum()), "normal": int((torch.isfinite(x) & (x.abs() >= tiny)).sum())}


def ieee754_compliance_report(dtype=torch.float32, device="cpu") -> dict:
    """Spot checks of the arithmetic the framework relies on."""
    t = lambda v: torch.tensor(v, dtype=dtype, device=device)
    inf, nan, fi = t(float("inf")), t(float("nan")), torch.finfo(dtype)
    return {"nan_not_equal": bool(nan != nan), "inf_minus_inf_is_nan": bool(torch.isnan(inf - inf)), "zero_div_zero_is_nan": bool(torch.isnan(t(0.0) / t(0.0))), "one_div_zero_is_inf": bool(torch.isinf(t(1.0) / t(0.0))),
            "signed_zero": bool(torch.signbit(t(-0.0)) and t(-0.0) == t(0.0)), "round_half_even": bool(torch.round(t(0.5)) == 0 and torch.round(t(1.5)) == 2 and torch.round(t(2.5)) == 2),
            "epsilon": bool(t(1.0) + t(fi.eps) > t(1.0) and t(1.0) + t(fi.eps / 4) == t(1.0)), "gradual_underflow": bool(t(fi.tiny) / 2 > 0) if dtype in (torch.float32, torch.float64) else None,
            "overflow_to_inf": bool(torch.isinf(t(fi.max) * 2)), "sqrt_negative_is_nan": bool(torch.isnan(torch.sqrt(t(-1.0))))}


# ================================================================================================ inspector
def inspect_tensor(x: torch.Tensor, name: str = "tensor", bins: int = 8) -> dict:
    info = {"name": name, "shape": tuple(x.shape), "dtype": str(x.dtype).replace("torch.", ""), "device": str(x.device), "strides": tuple(x.stride()), "contiguous": x.is_contiguous(),
            "numel": x.numel(), "bytes": x.numel() * x.element_size(), "storage_bytes": x.untyped_storage().nbytes(), "storage_offset": x.storage_offset(), "requires_grad": x.requires_grad,
            "is_view": x._base is not None, "channels_last": x.dim() == 4 and x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous()}
    if x.numel() and (x.is_floating_point() or x.dtype in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)):
        v = x.detach().double().flatten()
        fin = v[torch.isfinite(v)]
        info.update(min=float(fin.min()) if len(fin) else None, max=float(fin.max()) if len(fin) else None, mean=float(fin.mean()) if len(fin) else None, std=float(fin.std()) if len(fin) > 1 else 0.0,
                    zeros=int((v == 0).sum()), nan=int(torch.isnan(v).sum()), inf=int(torch.isinf(v).sum()))
        if len(fin) and fin.max() > fin.min():
            info["histogram"] = torch.histc(fin.float(), bins, float(fin.min()), float(fin.max())).long().tolist()
        issues = []
        if info["nan"] or info["inf"]:
            issues.append("non-finite values")
        if x.is_floating_point() and len(fin) and fin.abs().max() > 0.5 * torch.finfo(x.dtype).max:
            issues.append("values close to the dtype's range")
        if info["storage_bytes"] > 4 * max(info["bytes"], 1):
            issues.append("small view keeps a large storage alive")
        info["issues"] = issues
    return info


def format_inspection(info: dict) -> str:
    lines = [f"{info['name']}: {info['dtype']}{list(info['shape'])} on {info['device']}  ({info['bytes']:,} B, strides {list(info['strides'])}{'' if info['contiguous'] else ', non-contiguous'})"]
    if "mean" in info and info["mean"] is not None:
        lines.append(f"  range [{info['min']:.4g}, {info['max']:.4g}]  mean {info['mean']:.4g}  std {info['std']:.4g}  zeros {info['zeros']}  nan {info['nan']}  inf {info['inf']}")
    if "histogram" in info:
        top = max(info["histogram"]) or 1
        lines.append("  " + "".join(" ▁▂▃▄▅▆▇█"[min(8, math.ceil(8 * h / top))] for h in info["histogram"]))
    lines += [f"  ! {i}" for i in info.get("issues", [])]
    return "\n".join(lines)


# ================================================================================================ layout advice
class LayoutOptimizer:
    """Records how a tensor is traversed (which dimension the innermost loop walks) and recommends the layout whose unit
    stride matches the dominant access."""

    def __init__(self): self.access = defaultdict(Counter)
    def record_access(self, name: str, inner_dim: int, count: int = 1): self.access[name][inner_dim] += count

    def recommend(self, name: str, x: torch.Tensor) -> dict:
        acc = self.access[name]
        if not acc:
            return {"action": "none", "reason": "no access recorded"}
        dim, hits = acc.most_common(1)[0]
        dim %= x.dim()
        unit = min(range(x.dim()), key=lambda d: (x.stride(d) if x.shape[d] > 1 else math.inf))
        share = hits / sum(acc.values())
        if dim == unit:
            return {"action": "none", "reason": f"dimension {dim} already has the smallest stride", "share": share}
        if x.dim() == 4 and dim == 1:
            return {"action": "channels_last", "apply": lambda t: t.contiguous(memory_format=torch.channels_last), "share": share, "reason": "channel dimension is walked innermost"}
        perm = [d for d in range(x.dim()) if d != dim] + [dim]
        return {"action": "permute_contiguous", "permutation": perm, "apply": lambda t: t.permute(perm).contiguous(), "share": share,
                "reason": f"dimension {dim} is walked innermost in {share:.0%} of accesses but has stride {x.stride(dim)}"}


# ================================================================================================ memory maps
def memory_map(blocks: Sequence[tuple[str, int, int]], capacity: int, width: int = 64) -> str:
    """One text row: every cell covers ``capacity / width`` bytes, shows the first letter of the block that owns most of it
    or ``.`` when free; a legend with sizes follows."""
    cell = capacity / width
    row = []
    for c in range(width):
        lo, hi = c * cell, (c + 1) * cell
        best, cover = ".", 0.0
        for name, off, size in blocks:
            ov = max(0.0, min(hi, off + size) - max(lo, off))
            if ov > cover:
                best, cover = name[0], ov
        row.append(best if cover >= cell / 2 else ".")
    used = sum(s for _, _, s in blocks)
    legend = [f"  {n[0]} = {n} @{o} ({s:,} B)" for n, o, s in blocks]
    return "\n".join(["|" + "".join(row) + "|", f"  {used:,} / {capacity:,} B used ({used / capacity:.0%})"] + legend)


def memory_timeline(samples: Sequence[tuple[float, int]], height: int = 6, width: int = 40) -> str:
    if not samples:
        return ""
    peak = max(b for _, b in samples) or 1
    cols = [samples[min(len(samples) - 1, int(i * len(samples) / width))][1] for i in range(width)]
    rows = ["".join("#" if c / peak * height >= level else " " for c in cols) for level in range(height, 0, -1)]
    return "\n".join(f"{r}|" for r in rows) + f"\npeak {peak:,} B over {samples[-1][0] - samples[0][0]:.3g} s"


# ================================================================================================ MLIR / StableHLO text
def _fx_nodes(gm):
    from .. import fx as tfx
    return list(gm.graph.nodes), dict(gm.named_modules())


def _mlir_type(shape, dtype="f32"): return f"tensor<{'x'.join(map(str, shape))}x{dtype}>" if len(shape) else f"tensor<{dtype}>"


def emit_mlir(gm, example_inputs: Sequence[torch.Tensor], dialect: str = "linalg", name: str = "forward") -> str:
    """Textual module for a traced graph of linear / matmul / add / mul / relu / tanh / sigmoid nodes: ``linalg`` + ``arith``
    / ``math`` named ops, or ``stablehlo`` ops (the HLO text XLA accepts).  Shapes come from one run on ``example_inputs``."""
    from ..fx import ShapeProp
    ShapeProp(gm).run(*example_inputs)
    nodes, mods = _fx_nodes(gm)
    ty = lambda n: _mlir_type(n.meta["shape"])
    args, body, names, consts = [], [], {}, 0
    hlo = dialect == "stablehlo"
    ew = {"add": ("stablehlo.add", "arith.addf"), "mul": ("stablehlo.multiply", "arith.mulf"), "sub": ("stablehlo.subtract", "arith.subf"), "relu": ("stablehlo.maximum", "arith.maximumf"),
          "tanh": ("stablehlo.tanh", "math.tanh"), "sigmoid": ("stablehlo.logistic", "math.sigmoid"), "exp": ("stablehlo.exponential", "math.exp")}
    for n in nodes:
        if n.op == "placeholder":
            names[n] = f"%arg{len(args)}"; args.append(f"{names[n]}: {ty(n)}")
        elif n.op == "output":
            src = n.args[0]
            body.append(f"    {'stablehlo.return' if hlo else 'return'} {names[src]} : {ty(src)}")
            ret = ty(src)
        else:
            names[n] = f"%{len(names)}"
            m = mods.get(n.target) if n.op == "call_module" else None
            kind = type(m).__name__.lower() if m is not None else getattr(n.target, "__name__", str(n.target))
            ins = [names[a] for a in n.all_input_nodes]
            if isinstance(m, torch.nn.Linear):
                w_ty = _mlir_type(tuple(m.weight.shape))
                body.append(f"    %w{consts} = {'stablehlo.constant' if hlo else 'arith.constant'} dense_resource<{n.target}.weight> : {w_ty}")
                if hlo:
                    body.append(f"    {names[n]} = stablehlo.dot_general {ins[0]}, %w{consts}, contracting_dims = [{len(n.all_input_nodes[0].meta['shape']) - 1}] x [1] : ({ty(n.all_input_nodes[0])}, {w_ty}) -> {ty(n)}")
                else:
                    body.append(f"    %init{consts} = tensor.empty() : {ty(n)}")
                    body.append(f"    {names[n]} = linalg.matmul_transpose_b ins({ins[0]}, %w{consts} : {ty(n.all_input_nodes[0])}, {w_ty}) outs(%init{consts} : {ty(n)}) -> {ty(n)}")
                consts += 1
            elif kind == "matmul":
                body.append(f"    {names[n]} = {'stablehlo.dot' if hlo else 'linalg.matmul'} {'' if hlo else 'ins('}{ins[0]}, {ins[1]}{'' if hlo else ')'} : ({ty(n.all_input_nodes[0])}, {ty(n.all_input_nodes[1])}) -> {ty(n)}")
            elif kind in ew:
                op = ew[kind][0 if hlo else 1]
                if kind == "relu":
                    body.append(f"    %zero{consts} = {'stablehlo.constant' if hlo else 'arith.constant'} dense<0.0> : {ty(n)}")
                    ins.append(f"%zero{consts}"); consts += 1
                body.append(f"    {names[n]} = {op} {', '.join(ins)} : {ty(n)}")
            else:
                raise NotImplementedError(f"no MLIR lowering for {kind}")
    head = f"module {{\n  func.func @{name}({', '.join(args)}) -> {ret} {{"
    return "\n".join([head] + body + ["  }", "}"]) + "\n"


# ================================================================================================ neuromorphic
class LIFNeurons:
    """Leaky integrate-and-fire layer: ``v <- v + dt / tau (v_rest - v + R I)``; a neuron at threshold emits a spike, resets
    and stays silent for ``refractory`` steps."""

    def __init__(self, n: int, tau: float = 20.0, threshold: float = 1.0, v_rest: float = 0.0, v_reset: float = 0.0, resistance: float = 1.0, refractory: int = 0, dt: float = 1.0):
        self.tau, self.th, self.rest, self.reset, self.r, self.ref_steps, self.dt = tau, threshold, v_rest, v_reset, resistance, refractory, dt
        self.v, self.ref = torch.full((n,), v_rest), torch.zeros(n, dtype=torch.long)

    def step(self, current: torch.Tensor) -> torch.Tensor:
        active = self.ref == 0
        self.v = torch.where(active, self.v + self.dt / self.tau * (self.rest - self.v + self.r * current), self.v)
        spikes = active & (self.v >= self.th)
        self.v = torch.where(spikes, torch.full_like(self.v, self.reset), self.v)
        self.ref = torch.where(spikes, torch.full_like(self.ref, self.ref_steps), (self.ref - 1).clamp(min=0))
        return spikes

    def run(self, currents: torch.Tensor) -> torch.Tensor: return torch.stack([self.step(c) for c in currents])

    def rate_for_constant_input(self, current: float) -> float:
        """Closed-form firing rate for a constant drive above threshold (per time unit)."""
        drive = self.r * current + self.rest
        if drive <= self.th:
            return 0.0
        return 1.0 / (self.ref_steps * self.dt + self.tau * math.log((drive - self.reset) / (drive - self.th)))


def rate_encode(x: torch.Tensor, steps: int, generator=None) -> torch.Tensor: return torch.rand(steps, *x.shape, generator=generator) < x.clamp(0, 1)
def latency_encode(x: torch.Tensor, steps: int) -> torch.Tensor:
    """One spike per input: stronger inputs fire earlier; zero never fires."""
    t = ((1 - x.clamp(0, 1)) * (steps - 1)).round().long()
    out = torch.zeros(steps, *x.shape, dtype=torch.bool)
    out.scatter_(0, t[None], (x > 0)[None])
    return out


def rate_decode(spikes: torch.Tensor) -> torch.Tensor: return spikes.float().mean(0)


# ================================================================================================ tensor networks
class MatrixProductState:
    """Chain of cores ``[r_{k-1}, d_k, r_k]`` built by successive truncated SVDs of a state tensor; supports inner products,
    norms and reconstruction without forming the full tensor except on request."""

    def __init__(self, cores): self.cores = cores

    @classmethod
    def from_tensor(cls, t: torch.Tensor, max_bond: int = 64, cutoff: float = 0.0):
        cores, r, cur, discarded = [], 1, t, 0.0
        for d in t.shape[:-1]:
            u, s, vh = torch.linalg.svd(cur.reshape(r * d, -1), full_matrices=False)
            keep = max(1, min(max_bond, int((s > cutoff * s[0]).sum())))
            discarded += float((s[keep:] ** 2).sum())
            cores.append(u[:, :keep].reshape(r, d, keep))
            cur, r = s[:keep, None] * vh[:keep], keep
        cores.append(cur.reshape(r, t.shape[-1], 1))
        mps = cls(cores)
        mps.truncation_error = math.sqrt(discarded)
        return mps

    def bond_dimensions(self): return [c.shape[2] for c in self.cores[:-1]]
    def num_parameters(self): return sum(c.numel() for c in self.cores)

    def to_tensor(self):
        out = self.cores[0]
        for c in self.cores[1:]:
            out = torch.tensordot(out, c, dims=([-1], [0]))
        return out.squeeze(0).squeeze(-1)

    def inner(self, other: "MatrixProductState") -> torch.Tensor:
        env = torch.ones(1, 1, dtype=self.cores[0].dtype)
        for a, b in zip(self.cores, other.cores):
            env = torch.einsum("ij,idk,jdl->kl", env, a.conj(), b)
        return env[0, 0]

    def norm(self): return self.inner(self).real.sqrt() if self.cores[0].is_complex() else self.inner(self).sqrt()

    def amplitude(self, index: Sequence[int]) -> torch.Tensor:
        v = torch.ones(1, dtype=self.cores[0].dtype)
        for c, i in zip(self.cores, index):
            v = v @ c[:, i, :]
        return v[0]


def contraction_order(shapes: dict[str, dict[str, int]], output: Sequence[str] = ()) -> tuple[list, int]:
    """Greedy pairwise contraction order for a tensor network given ``{tensor: {index: dimension}}``: at every step the pair
    with the cheapest contraction; returns ``(order, total scalar multiplications)``."""
    live, order, cost = {k: dict(v) for k, v in shapes.items()}, [], 0
    while len(live) > 1:
        best = None
        for a in live:
            for b in live:
                if a >= b or not set(live[a]) & set(live[b]):
                    continue
                others = set(output) | {i for k, v in live.items() if k not in (a, b) for i in v}
                allidx = {**live[a], **live[b]}
                c = math.prod(allidx.values())
                if best is None or c < best[0]:
                    best = (c, a, b, {i: d for i, d in allidx.items() if not (i in live[a] and i in live[b]) or i in others})
        if best is None:                                                      # disconnected pieces: outer product of the two smallest
            a, b = sorted(live, key=lambda k: math.prod(live[k].values()))[:2]
            best = (math.prod({**live[a], **live[b]}.values()), a, b, {**live[a], **live[b]})
        c, a, b, res = best
        order.append((a, b)); cost += c
        del live[a], live[b]
        live[f"({a}{b})"] = res
    return order, cost


# ================================================================================================ shape validation
class ShapeError(ValueError):
    pass


def validate_shapes(op: str, **tensors) -> None:
    """Checks operand shapes for common operations and raises :class:`ShapeError` with the operand names, shapes and the
    rule that failed (``matmul``, ``elementwise``, ``cat:<dim>``, ``linear``, ``conv2d``, ``attention``)."""
    s = {k: tuple(v.shape) if isinstance(v, torch.Tensor) else tuple(v) for k, v in tensors.items()}
    names = list(s)
    fail = lambda rule, hint="": (_ for _ in ()).throw(ShapeError(f"{op}: {rule}; got " + ", ".join(f"{k}{list(v)}" for k, v in s.items()) + (f". {hint}" if hint else "")))
    if op == "matmul":
        a, b = s[names[0]], s[names[1]]
        if a[-1] != (b[-2] if len(b) > 1 else b[-1]):
            fail(f"inner dimensions differ ({a[-1]} vs {b[-2] if len(b) > 1 else b[-1]})", f"transpose {names[1]}?" if len(b) > 1 and b[-1] == a[-1] else "")
    elif op == "elementwise":
        try:
            torch.broadcast_shapes(*s.values())
        except RuntimeError:
            fail("shapes are not broadcastable")
    elif op.startswith("cat"):
        dim = int(op.split(":")[1]) if ":" in op else 0
        ref = list(s[names[0]])
        for k in names[1:]:
            if len(s[k]) != len(ref) or any(x != y for i, (x, y) in enumerate(zip(s[k], ref)) if i != dim % len(ref)):
                fail(f"all dimensions except {dim} must agree")
    elif op == "linear":
        x, w = s[names[0]], s[names[1]]
        if x[-1] != w[1]:
            fail(f"input features {x[-1]} != weight in_features {w[1]}")
        if len(names) > 2 and s[names[2]] != (w[0],):
            fail(f"bias must have {w[0]} entries")
    elif op == "conv2d":
        x, w = s[names[0]], s[names[1]]
        if len(x) != 4 or len(w) != 4:
            fail("input and weight must be 4-D (NCHW, OIHW)")
        if x[1] % w[1] or (x[1] // w[1]) and w[0] % (x[1] // w[1]):
            fail(f"channels {x[1]} are not a multiple of weight in-channels {w[1]} (groups)")
        if x[2] < w[2] or x[3] < w[3]:
            fail("kernel is larger than the input")
    elif op == "attention":
        q, k, v = (s[n] for n in names[:3])
        if q[-1] != k[-1]:
            fail(f"query and key head dimensions differ ({q[-1]} vs {k[-1]})")
        if k[-2] != v[-2]:
            fail(f"key and value lengths differ ({k[-2]} vs {v[-2]})")
    else:
        raise ValueError(f"unknown operation {op!r}")


def explain_broadcast(a: Sequence[int], b: Sequence[int]) -> str:
    n = max(len(a), len(b))
    pa, pb = (1,) * (n - len(a)) + tuple(a), (1,) * (n - len(b)) + tuple(b)
    rows = []
    for i, (x, y) in enumerate(zip(pa, pb)):
        rows.append(f"  dim {i}: {x} vs {y} -> " + (str(max(x, y)) if x == y or 1 in (x, y) else "INCOMPATIBLE"))
    return f"broadcast {list(a)} with {list(b)}:\n" + "\n".join(rows)


# ================================================================================================ cache-oblivious orders
def morton_encode(y: torch.Tensor, x: torch.Tensor, bits: int = 16) -> torch.Tensor:
    """Interleaves the bits of two coordinates (Z-order): neighbours in 2-D stay close in the 1-D order."""
    out = torch.zeros_like(y, dtype=torch.long)
    for b in range(bits):
        out |= ((x.long() >> b) & 1) << (2 * b)
        out |= ((y.long() >> b) & 1) << (2 * b + 1)
    return out


def morton_decode(code: torch.Tensor, bits: int = 16) -> tuple[torch.Tensor, torch.Tensor]:
    y, x = torch.zeros_like(code), torch.zeros_like(code)
    for b in range(bits):
        x |= ((code >> (2 * b)) & 1) << b
        y |= ((code >> (2 * b + 1)) & 1) << b
    return y, x


def morton_order(h: int, w: int) -> torch.Tensor:
    ys, xs = torch.meshgrid(torch.arange(h), torch.arange(w), indexing="ij")
    return morton_encode(ys.flatten(), xs.flatten()).argsort()


def cache_oblivious_transpose(a: torch.Tensor, base: int = 32) -> torch.Tensor:
    """Recursive halving of the longer side until blocks of ``base`` (then a direct copy): touches both matrices in
    blocks that fit every level of cache without knowing their sizes."""
    out = torch.empty(a.shape[1], a.shape[0], dtype=a.dtype)
    def rec(r0, r1, c0, c1):
        if r1 - r0 <= base and c1 - c0 <= base:
            out[c0:c1, r0:r1] = a[r0:r1, c0:c1].t()
        elif r1 - r0 >= c1 - c0:
            m = (r0 + r1) // 2
            rec(r0, m, c0, c1); rec(m, r1, c0, c1)
        else:
            m = (c0 + c1) // 2
            rec(r0, r1, c0, m); rec(r0, r1, m, c1)
    rec(0, a.shape[0], 0, a.shape[1])
    return out


# ================================================================================================ performance monitor
class PerfMonitor:
    """Sliding windows of named measurements with percentiles, throughput and threshold alerts (``on_alert`` callback)."""

    def __init__(self, window: int = 100, on_alert: Callable[[dict], None] | None = None, clock=time.perf_counter):
        self.window, self.on_alert, self.clock = window, on_alert or (lambda a: None), clock
        self.series, self.thresholds, self.alerts, self.stamps = defaultdict(lambda: deque(maxlen=window)), {}, [], defaultdict(lambda: deque(maxlen=window))

    def set_threshold(self, name: str, p95_above: float | None = None, mean_above: float | None = None): self.thresholds[name] = (p95_above, mean_above)

    def record(self, name: str, value: float):
        self.series[name].append(float(value)); self.stamps[name].append(self.clock())
        th = self.thresholds.get(name)
        if th and len(self.series[name]) >= 5:
            s = self.summary(name)
            for kind, limit, val in (("p95", th[0], s["p95"]), ("mean", th[1], s["mean"])):
                if limit is not None and val > limit:
                    a = {"metric": name, "kind": kind, "value": val, "limit": limit}
                    self.alerts.append(a); self.on_alert(a)

    def time(self, name: str):
        mon = self
        class _T:
            def __enter__(self): self.t0 = mon.clock(); return self
            def __exit__(self, *a): mon.record(name, mon.clock() - self.t0)
        return _T()

    def summary(self, name: str) -> dict:
        v = sorted(self.series[name])
        if not v:
            return {"count": 0}
        q = lambda p: v[min(len(v) - 1, int(p * len(v)))]
        span = self.stamps[name][-1] - self.stamps[name][0] if len(v) > 1 else 0.0
        return {"count": len(v), "mean": sum(v) / len(v), "min": v[0], "max": v[-1], "p50": q(0.5), "p95": q(0.95), "p99": q(0.99), "rate_per_s": (len(v) - 1) / span if span > 0 else 0.0}

    def snapshot(self): return {k: self.summary(k) for k in self.series}
