"""Quantisation methods and tooling beyond :mod:`torsh_b200.quantization` (``crates/torsh-quantization/src``): learned step
size (LSQ) and PACT activations, vector quantisation with k-means codebooks (incl. product quantisation), layer
sensitivity and Hessian-trace (HAWQ-style) scoring, mixed-precision bit allocation under a size budget, AdaRound-style
layer reconstruction, bias correction, cross-layer equalisation, histogram (entropy / KL, MSE, percentile) calibration,
lossless packing of low-bit tensors with Huffman coding, quantisation metrics and a per-layer report."""
from __future__ import annotations

import copy
import heapq
import math
from collections import Counter
from typing import Callable, Sequence

import torch
import torch.nn.functional as F
from torch import nn


# ================================================================================================ learned quantisers
def _grad_scale(x, s): return (x - x * s).detach() + x * s
def _round_ste(x): return (x.round() - x).detach() + x


class LSQQuantizer(nn.Module):
    """Learned step size quantisation (Esser et al.): ``x_q = round(clamp(x / s)) * s`` with the step ``s`` trained by the
    straight-through estimator and its gradient scaled by ``1 / sqrt(numel * q_max)``; ``s`` is initialised from the
    first batch as ``2 mean|x| / sqrt(q_max)``."""

    def __init__(self, bits: int = 4, signed: bool = True, per_channel: int | None = None):
        super().__init__()
        self.qn, self.qp = (-(2 ** (bits - 1)), 2 ** (bits - 1) - 1) if signed else (0, 2 ** bits - 1)
        self.per_channel, self.step, self.ready = per_channel, nn.Parameter(torch.ones(1)), False

    def _init(self, x):
        if self.per_channel is None:
            s = 2 * x.detach().abs().mean() / math.sqrt(self.qp)
            self.step = nn.Parameter(s.reshape(1).clamp(min=1e-8))
        else:
            dims = [d for d in range(x.dim()) if d != self.per_channel]
            shape = [1] * x.dim(); shape[self.per_channel] = -1
            self.step = nn.Parameter((2 * x.detach().abs().mean(dims) / math.sqrt(self.qp)).clamp(min=1e-8).reshape(shape))
        self.ready = True

    def forward(self, x):
        if not self.ready:
            self._init(x)
        n = x.numel() if self.per_channel is None else x.numel() / x.shape[self.per_channel]
        s = _grad_scale(self.step, 1.0 / math.sqrt(n * self.qp))
        return _round_ste((x / s).clamp(self.qn, self.qp)) * s


class PACT(nn.Module):
    """Activation clipping with a learned upper bound ``alpha`` followed by uniform quantisation on ``[0, alpha]``."""

    def __init__(self, bits: int = 4, alpha: float = 6.0): super().__init__(); self.alpha, self.levels = nn.Parameter(torch.tensor(alpha)), 2 ** bits - 1

    def forward(self, x):
        y = torch.minimum(F.relu(x), self.alpha)
        return _round_ste(y / self.alpha * self.levels) * self.alpha / self.levels


class LSQLinear(nn.Linear):
    def __init__(self, in_features, out_features, bias=True, w_bits: int = 4, a_bits: int = 8):
        super().__init__(in_features, out_features, bias)
        self.wq, self.aq = LSQQuantizer(w_bits, True, per_channel=0), LSQQuantizer(a_bits, True)

    def forward(self, x): return F.linear(self.aq(x), self.wq(self.weight), self.bias)


# ================================================================================================ vector quantisation
def kmeans_codebook(x: torch.Tensor, k: int, iters: int = 25, seed: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """``x``: ``[n, d]``; returns ``(codebook [k, d], assignment [n])``; empty clusters are re-seeded at the worst-fit points."""
    g = torch.Generator().manual_seed(seed)
    c = x[torch.randint(0, len(x), (1,), generator=g)].clone()               # k-means++ seeding
    while len(c) < k:
        d2 = torch.cdist(x, c).min(1).values.double() ** 2
        nxt = torch.multinomial(d2 / d2.sum(), 1, generator=g) if float(d2.sum()) > 0 else torch.randint(0, len(x), (1,), generator=g)
        c = torch.cat([c, x[nxt]])
    for _ in range(iters):
        d = torch.cdist(x, c)
        a = d.argmin(1)
        for j in range(k):
            m = a == j
            c[j] = x[m].mean(0) if m.any() else x[d.min(1).values.argmax()]
    return c, torch.cdist(x, c).argmin(1)


class VectorQuantizedTensor:
    """Product quantisation of a matrix: columns are split into groups of ``dim`` consecutive values (per row), every
    group is replaced by the index of its nearest code in that sub-space's codebook (``2^bits`` codes)."""

    def __init__(self, w: torch.Tensor, dim: int = 4, bits: int = 8, subspaces: int = 1, seed: int = 0):
        self.shape, self.dim, self.subspaces = tuple(w.shape), dim, subspaces
        vecs = w.detach().reshape(-1, dim)
        parts = vecs.reshape(len(vecs), subspaces, dim // subspaces)
        self.codebooks, self.codes = [], []
        for s in range(subspaces):
            cb, a = kmeans_codebook(parts[:, s], min(2 ** bits, len(vecs)), seed=seed + s)
            self.codebooks.append(cb); self.codes.append(a.to(torch.int32))
        self.bits = bits

    def dequantize(self) -> torch.Tensor:
        return torch.cat([cb[a.long()] for cb, a in zip(self.codebooks, self.codes)], 1).reshape(self.shape)

    def nbytes(self) -> int:
        return sum(cb.numel() * 2 for cb in self.codebooks) + math.ceil(sum(a.numel() for a in self.codes) * self.bits / 8)

    def compression_ratio(self, source_bytes_per_value: int = 2) -> float:
        return math.prod(self.shape) * source_bytes_per_value / self.nbytes()


# ================================================================================================ sensitivity / mixed precision
def _fake_quant_weight(w: torch.Tensor, bits: int) -> torch.Tensor:
    q = 2 ** (bits - 1) - 1
    s = w.abs().flatten(1).amax(1).clamp(min=1e-12).reshape(-1, *[1] * (w.dim() - 1)) / q
    return (w / s).round().clamp(-q - 1, q) * s


def layer_sensitivity(model: nn.Module, loss_fn: Callable[[nn.Module], torch.Tensor], bits: Sequence[int] = (8, 4, 2)) -> dict:
    """Loss increase when one layer at a time has its weight quantised to each bit width (everything else full precision)."""
    base = float(loss_fn(model))
    out = {}
    for name, m in model.named_modules():
        if isinstance(m, (nn.Linear, nn.Conv2d)):
            keep = m.weight.data.clone()
            out[name] = {}
            for b in bits:
                m.weight.data = _fake_quant_weight(keep, b)
                with torch.no_grad():
                    out[name][b] = float(loss_fn(model)) - base
            m.weight.data = keep
    return out


def hessian_trace(model: nn.Module, loss_fn: Callable[[nn.Module], torch.Tensor], samples: int = 16, seed: int = 0) -> dict:
    """Hutchinson estimate ``E[v^T H v]`` of the Hessian trace per weight tensor (Rademacher probes), divided by the
    parameter count: the curvature that HAWQ uses to rank layers."""
    g = torch.Generator().manual_seed(seed)
    params = {n: p for n, p in model.named_parameters() if p.dim() > 1}
    loss = loss_fn(model)
    grads = torch.autograd.grad(loss, list(params.values()), create_graph=True)
    acc = {n: 0.0 for n in params}
    for _ in range(samples):
        vs = [(torch.randint(0, 2, p.shape, generator=g) * 2 - 1).to(p.dtype) for p in params.values()]
        hv = torch.autograd.grad(grads, list(params.values()), vs, retain_graph=True)
        for n, v, h in zip(params, vs, hv):
            acc[n] += float((v * h).sum()) / samples
    return {n: acc[n] / params[n].numel() for n in params}


def allocate_bits(sizes: dict[str, int], sensitivity: dict[str, dict[int, float]], budget_bits: float, choices: Sequence[int] = (8, 4, 2)) -> dict[str, int]:
    """Greedy mixed-precision assignment: start from the highest precision everywhere, repeatedly lower the layer whose
    next step costs the least loss per bit saved, until the total fits ``budget_bits``."""
    choices = sorted(choices, reverse=True)
    cur = {n: 0 for n in sizes}
    total = lambda: sum(sizes[n] * choices[cur[n]] for n in sizes)
    while total() > budget_bits:
        best = None
        for n in sizes:
            if cur[n] + 1 < len(choices):
                b0, b1 = choices[cur[n]], choices[cur[n] + 1]
                cost = (sensitivity[n][b1] - sensitivity[n][b0]) / (sizes[n] * (b0 - b1))
                if best is None or cost < best[0]:
                    best = (cost, n)
        if best is None:
            break
        cur[best[1]] += 1
    return {n: choices[i] for n, i in cur.items()}


# ================================================================================================ post-training refinements
def adaround_layer(weight: torch.Tensor, x: torch.Tensor, bits: int = 4, iters: int = 300, lr: float = 1e-2, lam: float = 0.01) -> torch.Tensor:
    """Learns whether to round each weight up or down so that the layer output ``x W^T`` is preserved (rectified sigmoid
    relaxation with an annealed regulariser that drives the choices to 0 / 1).  Returns the quantised weight."""
    q = 2 ** (bits - 1) - 1
    s = weight.abs().amax(1, keepdim=True).clamp(min=1e-12) / q
    floor = torch.floor(weight / s)
    rest = weight / s - floor
    v = nn.Parameter(-torch.log(1.2 / (rest.clamp(1e-4, 1 - 1e-4) + 0.1) - 1))       # h(v) starts at the fractional part
    h = lambda: (torch.sigmoid(v) * 1.2 - 0.1).clamp(0, 1)
    target = x @ weight.t()
    opt = torch.optim.Adam([v], lr)
    for i in range(iters):
        beta = 20 - (20 - 2) * i / iters
        wq = (floor + h()).clamp(-q - 1, q) * s
        loss = F.mse_loss(x @ wq.t(), target) + lam * (1 - (2 * h() - 1).abs().pow(beta)).sum() / v.numel() * (i > 0.2 * iters)
        opt.zero_grad(); loss.backward(); opt.step()
    return ((floor + (h() >= 0.5).float()).clamp(-q - 1, q) * s).detach()


def bias_correction(layer: nn.Linear, quantized_weight: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """New bias that cancels the mean output shift caused by weight quantisation: ``b - E[x] (W_q - W)^T``."""
    shift = x.reshape(-1, x.shape[-1]).mean(0) @ (quantized_weight - layer.weight.detach()).t()
    b = layer.bias.detach() if layer.bias is not None else torch.zeros(layer.out_features)
    return b - shift


def cross_layer_equalization(a: nn.Linear, b: nn.Linear) -> torch.Tensor:
    """Rescales the output channels of ``a`` and the matching input channels of ``b`` (valid across ReLU) so both have equal
    per-channel ranges; the composed function is unchanged.  Returns the scales."""
    ra, rb = a.weight.detach().abs().amax(1), b.weight.detach().abs().amax(0)
    s = torch.sqrt(ra / rb.clamp(min=1e-12)).clamp(min=1e-8)
    with torch.no_grad():
        a.weight.div_(s[:, None])
        if a.bias is not None:
            a.bias.div_(s)
        b.weight.mul_(s[None])
    return s


class HistogramCalibrator:
    """Collects an absolute-value histogram over batches and picks the clipping threshold by ``percentile``, ``mse`` of the
    quantised histogram, or ``entropy`` (KL divergence between the clipped reference and its quantised version)."""

    def __init__(self, bins: int = 2048): self.bins, self.hist, self.max = bins, None, 0.0

    def collect(self, x: torch.Tensor):
        m = float(x.detach().abs().max())
        if self.hist is None:
            self.max, self.hist = max(m, 1e-12), torch.zeros(self.bins, dtype=torch.float64)
        elif m > self.max:                                                    # re-bin the old counts onto the wider range
            old_edges = torch.linspace(0, self.max, self.bins + 1)[:-1] + self.max / self.bins / 2
            new = torch.zeros(self.bins, dtype=torch.float64)
            new.index_add_(0, (old_edges / m * self.bins).long().clamp(max=self.bins - 1), self.hist)
            self.hist, self.max = new, m
        self.hist += torch.histc(x.detach().abs().float(), self.bins, 0, self.max).double()

    def threshold(self, method: str = "entropy", bits: int = 8, percentile: float = 99.99) -> float:
        width = self.max / self.bins
        if method == "percentile":
            cdf = self.hist.cumsum(0) / self.hist.sum()
            return float((int((cdf >= percentile / 100).nonzero()[0]) + 1) * width)
        levels = 2 ** (bits - 1)
        centers = (torch.arange(self.bins, dtype=torch.float64) + 0.5) * width
        best, best_t = math.inf, self.max
        for i in range(levels, self.bins + 1, max(1, self.bins // 256)):
            t = i * width
            if method == "mse":
                step = t / levels
                q = ((centers / step).round().clamp(max=levels) * step)
                err = float((self.hist * (centers - q) ** 2).sum())
            else:
                ref = self.hist[:i].clone()
                ref[-1] += self.hist[i:].sum()
                chunks = torch.tensor_split(self.hist[:i], levels)
                quant = torch.cat([torch.where(c > 0, c.sum() / max(int((c > 0).sum()), 1), torch.zeros_like(c)) for c in chunks])
                p, qd = ref / ref.sum(), quant / quant.sum().clamp(min=1e-300)
                nz = p > 0
                err = float((p[nz] * torch.log(p[nz] / qd[nz].clamp(min=1e-12))).sum())
            if err < best:
                best, best_t = err, t
        return float(best_t)


# ================================================================================================ packing / entropy coding
def pack_bits(values: torch.Tensor, bits: int) -> torch.Tensor:
    """Packs non-negative integers below ``2^bits`` (1, 2 or 4 bits) into bytes, low positions first."""
    per = 8 // bits
    v = values.reshape(-1).to(torch.uint8)
    pad = (-len(v)) % per
    v = torch.cat([v, v.new_zeros(pad)]).reshape(-1, per)
    out = torch.zeros(len(v), dtype=torch.uint8)
    for i in range(per):
        out |= v[:, i] << (i * bits)
    return out


def unpack_bits(packed: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    per, mask = 8 // bits, (1 << bits) - 1
    return torch.stack([(packed >> (i * bits)) & mask for i in range(per)], 1).reshape(-1)[:count]


class HuffmanCodec:
    """Canonical Huffman code over integer symbols; ``encode`` returns the bit string packed into bytes plus the bit
    count, ``decode`` inverts it."""

    def fit(self, symbols: Sequence[int]):
        freq = Counter(int(s) for s in symbols)
        heap = [[f, i, [s]] for i, (s, f) in enumerate(sorted(freq.items()))]
        length = {s: 0 for s in freq}
        heapq.heapify(heap)
        uid = len(heap)
        if len(heap) == 1:
            length[heap[0][2][0]] = 1
        while len(heap) > 1:
            a, b = heapq.heappop(heap), heapq.heappop(heap)
            for s in a[2] + b[2]:
                length[s] += 1
            heapq.heappush(heap, [a[0] + b[0], uid, a[2] + b[2]]); uid += 1
        code, prev_len, self.table = 0, 0, {}
        for s in sorted(length, key=lambda s: (length[s], s)):
            code <<= length[s] - prev_len
            self.table[s] = (code, length[s]); prev_len = length[s]; code += 1
        self.inverse = {v: k for k, v in self.table.items()}
        return self

    def encode(self, symbols) -> tuple[bytes, int]:
        acc, n = 0, 0
        for s in symbols:
            c, l = self.table[int(s)]
            acc, n = (acc << l) | c, n + l
        return acc.to_bytes((n + 7) // 8, "big") if n else b"", n

    def decode(self, data: bytes, nbits: int) -> list[int]:
        acc = int.from_bytes(data, "big")
        out, code, length = [], 0, 0
        for i in range(nbits - 1, -1, -1):
            code, length = (code << 1) | ((acc >> i) & 1), length + 1
            if (code, length) in self.inverse:
                out.append(self.inverse[(code, length)]); code, length = 0, 0
        return out

    def mean_code_length(self, symbols) -> float: c = Counter(int(s) for s in symbols); return sum(self.table[s][1] * f for s, f in c.items()) / sum(c.values())


def entropy_bits(symbols) -> float:
    c = Counter(int(s) for s in symbols)
    n = sum(c.values())
    return -sum(f / n * math.log2(f / n) for f in c.values())


# ================================================================================================ metrics / report
def quantization_metrics(ref: torch.Tensor, q: torch.Tensor) -> dict:
    e = (ref - q).double()
    p = ref.double().pow(2).mean()
    cos = float(F.cosine_similarity(ref.double().flatten(), q.double().flatten(), dim=0))
    return {"mse": float(e.pow(2).mean()), "max_abs": float(e.abs().max()), "sqnr_db": float(10 * torch.log10(p / e.pow(2).mean().clamp(min=1e-300))),
            "psnr_db": float(10 * torch.log10(ref.double().abs().max() ** 2 / e.pow(2).mean().clamp(min=1e-300))), "cosine": cos, "relative_l2": float(e.norm() / ref.double().norm().clamp(min=1e-300))}


def kl_divergence_hist(a: torch.Tensor, b: torch.Tensor, bins: int = 128) -> float:
    lo, hi = float(min(a.min(), b.min())), float(max(a.max(), b.max()))
    pa, pb = torch.histc(a.float(), bins, lo, hi).double() + 1e-6, torch.histc(b.float(), bins, lo, hi).double() + 1e-6
    pa, pb = pa / pa.sum(), pb / pb.sum()
    return float((pa * torch.log(pa / pb)).sum())


def model_quantization_report(model: nn.Module, bits: int | dict[str, int] = 8) -> dict:
    """Per-layer weight error at the given precision (one width or ``{layer: width}``) with totals and the model size."""
    rows, total_bits = [], 0
    for name, m in model.named_modules():
        if isinstance(m, (nn.Linear, nn.Conv2d)):
            b = bits if isinstance(bits, int) else bits.get(name, 8)
            qm = quantization_metrics(m.weight.detach(), _fake_quant_weight(m.weight.detach(), b))
            rows.append({"layer": name, "bits": b, "parameters": m.weight.numel(), "sqnr_db": qm["sqnr_db"], "relative_l2": qm["relative_l2"]})
            total_bits += m.weight.numel() * b
    n = sum(r["parameters"] for r in rows)
    return {"layers": rows, "mean_bits": total_bits / max(n, 1), "size_bytes": total_bits // 8, "fp16_bytes": 2 * n, "compression": 16 * n / max(total_bits, 1),
            "worst_layer": min(rows, key=lambda r: r["sqnr_db"])["layer"] if rows else None}


def apply_mixed_precision(model: nn.Module, bits: dict[str, int]) -> nn.Module:
    """Copy of the model with every listed layer's weight replaced by its fake-quantised value at the assigned width."""
    m = copy.deepcopy(model)
    for name, mod in m.named_modules():
        if name in bits and hasattr(mod, "weight"):
            mod.weight.data = _fake_quant_weight(mod.weight.data, bits[name])
    return m
