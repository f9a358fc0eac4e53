"""Gradient compression with error feedback (``crates/torsh-distributed/src/gradient_compression.rs:17-276``):
TopK, RandomK, Threshold, Quantization(bits), SignSGD, PowerSGD(rank), Ternary, EF21. Each compressor returns a compact
payload and can decompress it; ``ErrorFeedback`` keeps the residual that compression dropped and adds it to the next
gradient. On one NVSwitch box the uncompressed fused collectives are faster than any of these; they matter across
nodes and are kept for parity."""
from __future__ import annotations

import math

import torch


class Compressor:
    def compress(self, g: torch.Tensor): raise NotImplementedError
    def decompress(self, payload, shape, dtype=torch.float32, device=None) -> torch.Tensor: raise NotImplementedError

    def ratio(self, g: torch.Tensor) -> float:
        p = self.compress(g)
        nbytes = sum(t.numel() * t.element_size() for t in p if isinstance(t, torch.Tensor))
        return g.numel() * g.element_size() / max(nbytes, 1)


class TopK(Compressor):
    def __init__(self, ratio: float = 0.01):
        self.r = ratio

    def compress(self, g):
        flat = g.reshape(-1)
        k = max(1, int(flat.numel() * self.r))
        idx = flat.abs().topk(k).indices
        return idx.to(torch.int32), flat[idx]

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        idx, val = payload
        out = torch.zeros(math.prod(shape), dtype=dtype, device=device or val.device)
        out[idx.long()] = val.to(dtype)
        return out.view(shape)


class RandomK(TopK):
    def __init__(self, ratio: float = 0.01, seed: int = 0):
        super().__init__(ratio)
        self.gen = torch.Generator().manual_seed(seed)

    def compress(self, g):
        flat = g.reshape(-1)
        k = max(1, int(flat.numel() * self.r))
        idx = torch.randperm(flat.numel(), generator=self.gen)[:k].to(flat.device)
        return idx.to(torch.int32), flat[idx] * (flat.numel() / k)


def threshold_sparsify(g: torch.Tensor, threshold: float, capacity: int | None = None):
    """``(indices int32, values fp32)`` of ``|g| > threshold``; on a GPU one compaction kernel (order not defined)."""
    n = g.numel()
    if _gpu(g) and n < 2 ** 31:
        from .. import _native as nv
        from ..ops._dispatch import F, I, L, P, call, dtype_code
        cap = capacity or n
        idx = torch.empty(cap, dtype=torch.int32, device=g.device)
        vals = torch.empty(cap, dtype=torch.float32, device=g.device)
        cnt = torch.empty(1, dtype=torch.int32, device=g.device)
        call("tb_threshold_sparsify", [P, F, P, P, P, I, L, I, P], g.data_ptr(), float(threshold), idx.data_ptr(), vals.data_ptr(),
             cnt.data_ptr(), cap, n, dtype_code(g), nv.stream_ptr())
        k = min(int(cnt.item()), cap)
        return idx[:k], vals[:k]
    flat = g.reshape(-1)
    i = (flat.abs() > threshold).nonzero().flatten()
    return i.to(torch.int32), flat[i].float()


class Threshold(TopK):
    def __init__(self, threshold: float = 1e-3):
        self.t = threshold

    def compress(self, g):
        flat = g.reshape(-1)
        idx = (flat.abs() >= self.t).nonzero().squeeze(1)
        return idx.to(torch.int32), flat[idx]


def _gpu(g):
    return g.is_cuda and g.dtype in (torch.float32, torch.bfloat16) and g.is_contiguous()


class Int8BlockQuantization(Compressor):
    """Symmetric int8 with one fp32 scale per 1024 values: one kernel pass each way on a GPU
    (``csrc/kernels/compress.cu``), the same arithmetic in PyTorch elsewhere."""
    CHUNK = 1024

    def compress(self, g):
        n = g.numel()
        nch = (n + self.CHUNK - 1) // self.CHUNK
        if _gpu(g):
            from .. import _native as nv
            from ..ops._dispatch import I, L, P, call, dtype_code
            q = torch.empty(n, dtype=torch.int8, device=g.device)
            scales = torch.empty(nch, dtype=torch.float32, device=g.device)
            call("tb_quantize_int8", [P, P, P, L, I, P], g.data_ptr(), q.data_ptr(), scales.data_ptr(), n, dtype_code(g), nv.stream_ptr())
            return q, scales
        f = torch.nn.functional.pad(g.float().reshape(-1), (0, nch * self.CHUNK - n)).view(nch, self.CHUNK)
        amax = f.abs().amax(1)
        scales = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
        q = (f / scales[:, None]).round().clamp(-127, 127).to(torch.int8).reshape(-1)[:n]
        return q, scales

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        q, scales = payload
        n = q.numel()
        if q.is_cuda and dtype in (torch.float32, torch.bfloat16):
            from .. import _native as nv
            from ..ops._dispatch import I, L, P, call
            y = torch.empty(n, dtype=dtype, device=q.device)
            call("tb_dequantize_int8", [P, P, P, L, I, P], q.data_ptr(), scales.data_ptr(), y.data_ptr(), n, 0 if dtype == torch.bfloat16 else 1,
                 nv.stream_ptr())
            return y.view(shape)
        return (q.to(dtype) * scales.repeat_interleave(self.CHUNK)[:n].to(dtype)).view(shape)


class PackedSignSGD(Compressor):
    """1 bit per value (32 signs per word) plus the mean magnitude."""

    def compress(self, g):
        n = g.numel()
        if _gpu(g):
            from .. import _native as nv
            from ..ops._dispatch import I, L, P, call, dtype_code
            bits = torch.empty((n + 31) // 32, dtype=torch.int32, device=g.device)
            s = torch.empty(1, dtype=torch.float32, device=g.device)
            call("tb_sign_pack", [P, P, P, L, I, P], g.data_ptr(), bits.data_ptr(), s.data_ptr(), n, dtype_code(g), nv.stream_ptr())
            return bits, s, n
        pos = torch.nn.functional.pad((g.reshape(-1) >= 0).to(torch.int64), (0, (-n) % 32)).view(-1, 32)
        words = (pos << torch.arange(32)).sum(1)
        bits = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
        return bits, g.float().abs().sum().reshape(1), n

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        bits, s, n = payload
        if bits.is_cuda and dtype in (torch.float32, torch.bfloat16):
            from .. import _native as nv
            from ..ops._dispatch import I, L, P, call
            y = torch.empty(n, dtype=dtype, device=bits.device)
            call("tb_sign_unpack", [P, P, P, L, I, P], bits.data_ptr(), s.data_ptr(), y.data_ptr(), n, 0 if dtype == torch.bfloat16 else 1,
                 nv.stream_ptr())
            return y.view(shape)
        b = ((bits.to(torch.int64)[:, None] >> torch.arange(32)) & 1).reshape(-1)[:n]
        return ((b.to(dtype) * 2 - 1) * (s / n).to(dtype)).view(shape)


class Quantization(Compressor):
    def __init__(self, bits: int = 8):
        self.bits = bits

    def compress(self, g):
        lo, hi = g.min(), g.max()
        levels = 2 ** self.bits - 1
        scale = (hi - lo).clamp(min=1e-12) / levels
        q = ((g - lo) / scale).round().clamp(0, levels).to(torch.uint8 if self.bits <= 8 else torch.int32)
        return q, torch.stack([lo, scale]).float()

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        q, meta = payload
        return (q.to(dtype) * meta[1] + meta[0]).view(shape)


class SignSGD(Compressor):
    def compress(self, g):
        return (g >= 0).to(torch.uint8), g.abs().mean().reshape(1)

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        s, scale = payload
        return ((s.to(dtype) * 2 - 1) * scale).view(shape)


class Ternary(Compressor):
    def compress(self, g):
        t = 0.7 * g.abs().mean()
        m = (g.abs() > t)
        scale = g.abs()[m].mean() if m.any() else g.new_zeros(())
        return (torch.sign(g) * m).to(torch.int8), scale.reshape(1)

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        s, scale = payload
        return (s.to(dtype) * scale).view(shape)


class PowerSGD(Compressor):
    """Rank-``r`` factorisation ``G ≈ P Qᵀ`` by one power iteration with a warm-started ``Q``."""

    def __init__(self, rank: int = 4):
        self.rank, self._q = rank, {}

    def compress(self, g):
        m = g.reshape(g.shape[0], -1) if g.dim() > 1 else g.reshape(1, -1)
        key = tuple(m.shape)
        q = self._q.get(key)
        if q is None or q.device != m.device:
            q = torch.randn(m.shape[1], self.rank, device=m.device, dtype=m.dtype)
        p, _ = torch.linalg.qr(m @ q)
        q = m.t() @ p
        self._q[key] = q
        return p, q

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        p, q = payload
        return (p @ q.t()).to(dtype).view(shape)


class ErrorFeedback:
    """Adds the residual of the previous round before compressing and stores the new residual (EF / EF21)."""

    def __init__(self, compressor: Compressor, warmup_steps: int = 0):
        self.c, self.residual, self.warmup, self.step = compressor, {}, warmup_steps, 0

    def compress(self, name: str, g: torch.Tensor):
        self.step += 1
        if self.step <= self.warmup:
            return None, g
        acc = g + self.residual.get(name, 0)
        payload = self.c.compress(acc)
        approx = self.c.decompress(payload, acc.shape, acc.dtype, acc.device)
        self.residual[name] = acc - approx
        return payload, approx


class CountSketch(Compressor):
    """Sketching (``gradient_compression.rs``: ``Sketching``): ``rows`` independent count sketches of ``cols`` buckets
    (sign hash × bucket hash); an element is recovered as the median over rows of ``sign · bucket``. Sketches are
    linear, so the sketches of all ranks can be summed before decoding."""

    def __init__(self, rows: int = 5, cols: int = 4096, seed: int = 0):
        self.rows, self.cols, self.seed, self._tables = rows, cols, seed, {}

    def _hashes(self, n: int, device):
        key = (n, str(device))
        if key not in self._tables:
            gen = torch.Generator().manual_seed(self.seed)
            bucket = torch.randint(0, self.cols, (self.rows, n), generator=gen)
            sign = torch.randint(0, 2, (self.rows, n), generator=gen) * 2 - 1
            self._tables[key] = (bucket.to(device), sign.to(device))
        return self._tables[key]

    def compress(self, g):
        flat = g.reshape(-1).float()
        bucket, sign = self._hashes(flat.numel(), flat.device)
        sk = torch.zeros(self.rows, self.cols, device=flat.device)
        sk.scatter_add_(1, bucket, sign * flat[None])
        return (sk,)

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        sk = payload[0]
        n = math.prod(shape)
        bucket, sign = self._hashes(n, sk.device)
        est = sk.gather(1, bucket) * sign
        return est.median(0).values.to(dtype).view(shape)


class NaturalCompression(Compressor):
    """Natural compression: every value is rounded, without bias, to one of the two neighbouring powers of two, so only
    sign and exponent (9 bits) travel."""

    def __init__(self, seed: int = 0):
        self.gen = torch.Generator().manual_seed(seed)

    def compress(self, g):
        a = g.abs().float().clamp(min=1e-38)
        e = torch.floor(torch.log2(a))
        lo = torch.exp2(e)
        p_up = (a - lo) / lo                                   # in [0, 1): probability of rounding up to 2^(e+1)
        up = torch.rand(a.shape, generator=self.gen).to(a.device) < p_up
        exp = (e + up.float()).clamp(-126, 127).to(torch.int8)
        sign = torch.where(g == 0, torch.zeros_like(exp), torch.sign(g).to(torch.int8))
        return exp, sign

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        exp, sign = payload
        return (torch.exp2(exp.float()) * sign.float()).to(dtype).view(shape)


class Bimodal(Compressor):
    """Two-level quantisation (``Bimodal``): values are split at the mean magnitude into a "small" and a "large" mode and
    each element is replaced by the mean magnitude of its mode, keeping its sign: 2 bits per element plus two scalars."""

    def compress(self, g):
        a = g.abs().float()
        t = a.mean()
        big = a > t
        m_small = a[~big].mean() if (~big).any() else a.new_zeros(())
        m_big = a[big].mean() if big.any() else a.new_zeros(())
        code = (big.to(torch.uint8) << 1) | (g >= 0).to(torch.uint8)
        return code, torch.stack([m_small, m_big])

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        code, modes = payload
        mag = modes[(code >> 1).long()]
        sign = (code & 1).float() * 2 - 1
        return (mag * sign).to(dtype).view(shape)


class LayerwiseAdaptive(Compressor):
    """Chooses the compressor per tensor from its size and density (``LayerwiseAdaptive``): small tensors travel
    uncompressed, matrices above ``lowrank_numel`` use PowerSGD, the rest Top-K with a ratio that grows with the
    tensor's kurtosis-free sparsity estimate (share of elements below a tenth of the mean magnitude)."""

    def __init__(self, small_numel: int = 4096, lowrank_numel: int = 1 << 20, base_ratio: float = 0.01, rank: int = 4):
        self.small, self.lowrank, self.base, self.psgd = small_numel, lowrank_numel, base_ratio, PowerSGD(rank)

    def choose(self, g: torch.Tensor):
        if g.numel() <= self.small:
            return "none", None
        if g.dim() >= 2 and g.numel() >= self.lowrank:
            return "powersgd", self.psgd
        a = g.abs()
        sparse_share = float((a < 0.1 * a.mean()).float().mean())
        ratio = min(0.25, max(self.base, self.base * (1.0 + 4.0 * (1.0 - sparse_share))))
        return "topk", TopK(ratio)

    def compress(self, g):
        kind, c = self.choose(g)
        return (kind, g.clone()) if c is None else (kind, c.compress(g), c)

    def decompress(self, payload, shape, dtype=torch.float32, device=None):
        if payload[0] == "none":
            return payload[1].to(dtype).view(shape)
        return payload[2].decompress(payload[1], shape, dtype, device)


class EF21:
    """EF21 (``gradient_compression.rs``: ``EF21``): every rank keeps a state ``h``; it sends ``c = C(g - h)`` and sets
    ``h += c``; the receivers track the same ``h``, so the estimate of the gradient is ``h`` itself."""

    def __init__(self, compressor: Compressor):
        self.c, self.h = compressor, {}

    def compress(self, name: str, g: torch.Tensor):
        h = self.h.get(name)
        if h is None:
            h = torch.zeros_like(g)
        payload = self.c.compress(g - h)
        h = h + self.c.decompress(payload, g.shape, g.dtype, g.device)
        self.h[name] = h
        return payload, h
