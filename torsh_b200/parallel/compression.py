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
