"""Research and specialised layers (``crates/torsh-nn/src/{research,sparse,lazy,compile_time,hardware_opts}.rs`` and
``layers/{blocks,ip_adapter,upsampling,regularization,recurrent}.rs``): Neural ODE block, capsule layer with dynamic
routing, squeeze-and-excitation, IP-adapter cross attention, 1-D pixel shuffle, DropConnect, Cutout, a cell-factory RNN,
ConvLSTM, modern Hopfield layer, hyper-network linear, adaptive softmax head, masked sparse layers with a gradual
pruning schedule, lazily shaped linear, and fused linear + activation blocks on the package's GEMM epilogues."""
from __future__ import annotations

import math
from typing import Callable

import torch
import torch.nn.functional as F
from torch import nn


class NeuralODE(nn.Module):
    """``x(t1) = x(t0) + integral f(t, x) dt`` with a fixed-step solver (``euler``, ``midpoint``, ``rk4``); gradients flow
    through the unrolled steps.  ``func(t, x)`` is any module or callable."""

    def __init__(self, func, t0: float = 0.0, t1: float = 1.0, steps: int = 10, method: str = "rk4"):
        super().__init__()
        self.func, self.t0, self.t1, self.steps, self.method = func, t0, t1, steps, method

    def forward(self, x, return_trajectory: bool = False):
        h, t, traj = (self.t1 - self.t0) / self.steps, self.t0, [x]
        for _ in range(self.steps):
            if self.method == "euler":
                x = x + h * self.func(t, x)
            elif self.method == "midpoint":
                x = x + h * self.func(t + h / 2, x + h / 2 * self.func(t, x))
            else:
                k1 = self.func(t, x)
                k2 = self.func(t + h / 2, x + h / 2 * k1)
                k3 = self.func(t + h / 2, x + h / 2 * k2)
                k4 = self.func(t + h, x + h * k3)
                x = x + h / 6 * (k1 + 2 * k2 + 2 * k3 + k4)
            t += h
            traj.append(x)
        return torch.stack(traj) if return_trajectory else x


def squash(s, dim=-1):
    n2 = (s * s).sum(dim, keepdim=True)
    return n2 / (1 + n2) * s / torch.sqrt(n2 + 1e-9)


class CapsuleLayer(nn.Module):
    """Fully connected capsules with routing by agreement: input ``[B, in_caps, in_dim]`` to ``[B, out_caps, out_dim]``."""

    def __init__(self, in_caps, in_dim, out_caps, out_dim, routing_iters: int = 3):
        super().__init__()
        self.w = nn.Parameter(0.01 * torch.randn(1, in_caps, out_caps, out_dim, in_dim))
        self.iters = routing_iters

    def forward(self, x):
        u = (self.w @ x[:, :, None, :, None]).squeeze(-1)                    # [B, in, out, out_dim]
        b = torch.zeros(*u.shape[:3], device=x.device, dtype=x.dtype)
        for i in range(self.iters):
            c = b.softmax(2)
            v = squash((c[..., None] * u).sum(1))
            if i < self.iters - 1:
                b = b + (u * v[:, None]).sum(-1)
        self.coupling = c
        return v


class SEBlock(nn.Module):
    def __init__(self, channels, reduction: int = 16):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(channels, max(channels // reduction, 1)), nn.Linear(max(channels // reduction, 1), channels)

    def forward(self, x):
        s = torch.sigmoid(self.fc2(F.relu(self.fc1(x.mean((-2, -1))))))
        return x * s[..., None, None]


class IPAdapterCrossAttention(nn.Module):
    """Decoupled cross attention: the text branch and an image-prompt branch share the query and are summed with ``scale``
    on the image branch (scale 0 reproduces plain text cross attention)."""

    def __init__(self, dim, ctx_dim, heads: int = 8, image_ctx_dim: int | None = None, scale: float = 1.0):
        super().__init__()
        self.h, self.scale = heads, scale
        self.q, self.k, self.v, self.o = nn.Linear(dim, dim, bias=False), nn.Linear(ctx_dim, dim, bias=False), nn.Linear(ctx_dim, dim, bias=False), nn.Linear(dim, dim)
        self.k_ip, self.v_ip = nn.Linear(image_ctx_dim or ctx_dim, dim, bias=False), nn.Linear(image_ctx_dim or ctx_dim, dim, bias=False)

    def _heads(self, t): return t.reshape(*t.shape[:2], self.h, -1).transpose(1, 2)

    def forward(self, x, text_ctx, image_ctx=None):
        q = self._heads(self.q(x))
        out = F.scaled_dot_product_attention(q, self._heads(self.k(text_ctx)), self._heads(self.v(text_ctx)))
        if image_ctx is not None and self.scale != 0:
            out = out + self.scale * F.scaled_dot_product_attention(q, self._heads(self.k_ip(image_ctx)), self._heads(self.v_ip(image_ctx)))
        return self.o(out.transpose(1, 2).reshape(x.shape))


class PixelShuffle1d(nn.Module):
    def __init__(self, factor): super().__init__(); self.r = factor
    def forward(self, x): b, c, l = x.shape; return x.reshape(b, c // self.r, self.r, l).permute(0, 1, 3, 2).reshape(b, c // self.r, l * self.r)


class PixelUnshuffle1d(nn.Module):
    def __init__(self, factor): super().__init__(); self.r = factor
    def forward(self, x): b, c, l = x.shape; return x.reshape(b, c, l // self.r, self.r).permute(0, 1, 3, 2).reshape(b, c * self.r, l // self.r)


class DropConnect(nn.Module):
    """Linear layer whose weights (not activations) are dropped during training, rescaled to keep the expectation."""

    def __init__(self, in_features, out_features, p: float = 0.5, bias: bool = True):
        super().__init__()
        self.lin, self.p = nn.Linear(in_features, out_features, bias), p

    def forward(self, x):
        if not self.training or self.p == 0:
            return self.lin(x)
        mask = (torch.rand_like(self.lin.weight) >= self.p).to(x.dtype) / (1 - self.p)
        return F.linear(x, self.lin.weight * mask, self.lin.bias)


class Cutout(nn.Module):
    def __init__(self, size: int, p: float = 1.0): super().__init__(); self.size, self.p = size, p

    def forward(self, x):
        if not self.training:
            return x
        b, _, h, w = x.shape
        cy, cx = torch.randint(0, h, (b,), device=x.device), torch.randint(0, w, (b,), device=x.device)
        ys, xs = torch.arange(h, device=x.device)[None, :, None], torch.arange(w, device=x.device)[None, None, :]
        hole = ((ys - cy[:, None, None]).abs() <= self.size // 2) & ((xs - cx[:, None, None]).abs() <= self.size // 2)
        hole &= (torch.rand(b, device=x.device) < self.p)[:, None, None]
        return x * (~hole)[:, None].to(x.dtype)


class CustomRNN(nn.Module):
    """Unrolls any cell ``cell(x_t, state) -> (output, state)`` over ``[B, T, ...]`` (optionally reversed)."""

    def __init__(self, cell, reverse: bool = False): super().__init__(); self.cell, self.reverse = cell, reverse

    def forward(self, x, state=None):
        steps = range(x.shape[1] - 1, -1, -1) if self.reverse else range(x.shape[1])
        outs = []
        for t in steps:
            o, state = self.cell(x[:, t], state)
            outs.append(o)
        if self.reverse:
            outs.reverse()
        return torch.stack(outs, 1), state


class ConvLSTMCell(nn.Module):
    def __init__(self, cin, hidden, kernel_size: int = 3):
        super().__init__()
        self.hidden, self.conv = hidden, nn.Conv2d(cin + hidden, 4 * hidden, kernel_size, padding=kernel_size // 2)

    def forward(self, x, state=None):
        if state is None:
            z = x.new_zeros(x.shape[0], self.hidden, *x.shape[-2:])
            state = (z, z)
        h, c = state
        i, f, g, o = self.conv(torch.cat([x, h], 1)).chunk(4, 1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        h = torch.sigmoid(o) * torch.tanh(c)
        return h, (h, c)


class ConvLSTM(CustomRNN):
    def __init__(self, cin, hidden, kernel_size: int = 3): super().__init__(ConvLSTMCell(cin, hidden, kernel_size))


class HopfieldLayer(nn.Module):
    """Modern (continuous) Hopfield retrieval: ``softmax(beta * q K^T) V`` iterated ``steps`` times on the query; with
    ``stored`` patterns as keys and values it completes noisy patterns in one step."""

    def __init__(self, dim, beta: float | None = None, steps: int = 1, project: bool = False):
        super().__init__()
        self.beta, self.steps = beta or 1 / math.sqrt(dim), steps
        self.q = nn.Linear(dim, dim, bias=False) if project else nn.Identity()
        self.k = nn.Linear(dim, dim, bias=False) if project else nn.Identity()

    def forward(self, query, stored):
        k, xi = self.k(stored), self.q(query)
        for _ in range(self.steps):
            xi = torch.softmax(self.beta * xi @ k.transpose(-1, -2), -1) @ stored
        return xi


class HyperLinear(nn.Module):
    """A linear layer whose weight and bias are produced by a small network from a conditioning vector ``z`` (one set of
    weights per batch element)."""

    def __init__(self, z_dim, in_features, out_features, hidden: int = 64):
        super().__init__()
        self.inf, self.outf = in_features, out_features
        self.net = nn.Sequential(nn.Linear(z_dim, hidden), nn.ReLU(), nn.Linear(hidden, in_features * out_features + out_features))
        with torch.no_grad():
            self.net[-1].weight.mul_(0.1)

    def forward(self, x, z):
        p = self.net(z)
        w, b = p[:, :self.inf * self.outf].reshape(-1, self.outf, self.inf), p[:, self.inf * self.outf:]
        return torch.einsum("boi,b...i->b...o", w, x) + b.reshape(b.shape[0], *[1] * (x.dim() - 2), -1)


class AdaptiveSoftmaxHead(nn.Module):
    """Frequency-clustered softmax (Grave et al.): a head over the frequent words plus one slot per tail cluster, tails
    projected to a smaller width.  ``log_prob`` returns the full ``[N, vocab]`` table; ``forward`` the NLL of targets."""

    def __init__(self, dim, vocab, cutoffs, div_value: float = 4.0):
        super().__init__()
        self.cut = [0] + list(cutoffs) + [vocab]
        self.head = nn.Linear(dim, self.cut[1] + len(cutoffs))
        self.tails = nn.ModuleList()
        for i in range(1, len(self.cut) - 1):
            d = max(1, int(dim / div_value ** i))
            self.tails.append(nn.Sequential(nn.Linear(dim, d, bias=False), nn.Linear(d, self.cut[i + 1] - self.cut[i])))

    def log_prob(self, x):
        head = self.head(x).log_softmax(-1)
        parts = [head[:, :self.cut[1]]]
        for i, tail in enumerate(self.tails):
            parts.append(head[:, self.cut[1] + i:self.cut[1] + i + 1] + tail(x).log_softmax(-1))
        return torch.cat(parts, 1)

    def forward(self, x, target):
        """Evaluates a tail only for the rows whose target falls in it."""
        head = self.head(x).log_softmax(-1)
        out = x.new_zeros(len(target))
        short = target < self.cut[1]
        out[short] = head[short, target[short]]
        for i, tail in enumerate(self.tails):
            m = (target >= self.cut[i + 1]) & (target < self.cut[i + 2])
            if m.any():
                out[m] = head[m, self.cut[1] + i] + tail(x[m]).log_softmax(-1).gather(1, (target[m] - self.cut[i + 1])[:, None]).squeeze(1)
        return -out.mean()


# ---- sparse training -----------------------------------------------------------------------------------------------------
class SparseLinear(nn.Linear):
    """Linear layer with a fixed-shape binary mask on the weight; pruned weights get no gradient."""

    def __init__(self, in_features, out_features, bias=True, sparsity: float = 0.0):
        super().__init__(in_features, out_features, bias)
        self.register_buffer("mask", torch.ones_like(self.weight))
        if sparsity > 0:
            self.prune_to(sparsity)

    def prune_to(self, sparsity: float):
        """Keeps the largest-magnitude weights among those still alive so that ``sparsity`` of all weights are zero."""
        k = int(round(sparsity * self.weight.numel()))
        if k > 0:
            score = (self.weight.detach().abs() * self.mask).reshape(-1)
            score[self.mask.reshape(-1) == 0] = -1
            self.mask.reshape(-1)[score.argsort()[:k]] = 0

    def sparsity(self) -> float: return float(1 - self.mask.mean())
    def forward(self, x): return F.linear(x, self.weight * self.mask, self.bias)


class SparseConv2d(nn.Conv2d):
    def __init__(self, *a, sparsity: float = 0.0, **kw):
        super().__init__(*a, **kw)
        self.register_buffer("mask", torch.ones_like(self.weight))
        if sparsity > 0:
            self.prune_to(sparsity)

    prune_to, sparsity = SparseLinear.prune_to, SparseLinear.sparsity
    def forward(self, x): return self._conv_forward(x, self.weight * self.mask, self.bias)


class GradualPruningScheduler:
    """Cubic sparsity ramp of Zhu & Gupta: ``s_t = s_f + (s_i - s_f) (1 - (t - t0) / (n dt))^3`` applied every
    ``frequency`` steps to every sparse layer of a model."""

    def __init__(self, model, final_sparsity: float, begin_step: int = 0, end_step: int = 1000, frequency: int = 100, initial_sparsity: float = 0.0):
        self.layers = [m for m in model.modules() if hasattr(m, "prune_to")]
        self.sf, self.si, self.t0, self.t1, self.freq, self.t = final_sparsity, initial_sparsity, begin_step, end_step, frequency, 0

    def target(self, t=None) -> float:
        t = self.t if t is None else t
        if t < self.t0:
            return self.si
        frac = min(1.0, (t - self.t0) / max(self.t1 - self.t0, 1))
        return self.sf + (self.si - self.sf) * (1 - frac) ** 3

    def step(self):
        self.t += 1
        if self.t >= self.t0 and (self.t - self.t0) % self.freq == 0 and self.t <= self.t1 + self.freq:
            for l in self.layers:
                l.prune_to(self.target())


# ---- shape inference and fused blocks --------------------------------------------------------------------------------------
class LazyLinear(nn.Module):
    """Linear layer whose input width is taken from the first batch; parameters exist after that call."""

    def __init__(self, out_features, bias=True): super().__init__(); self.out_features, self.use_bias, self.inner = out_features, bias, None
    def is_initialized(self): return self.inner is not None

    def forward(self, x):
        if self.inner is None:
            self.inner = nn.Linear(x.shape[-1], self.out_features, self.use_bias, device=x.device, dtype=x.dtype)
        return self.inner(x)


class FusedLinearActivation(nn.Module):
    """``activation(x W^T + b)`` as one op: on a CUDA device in bf16 the package's GEMM applies bias and activation in its
    epilogue (``ops.linear``); elsewhere the same arithmetic runs through PyTorch."""

    def __init__(self, in_features, out_features, activation: str = "gelu", bias: bool = True):
        super().__init__()
        self.lin, self.activation = nn.Linear(in_features, out_features, bias), activation

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and self.activation in ("gelu", "none"):
            from ..ops.linear import linear
            return linear(x, self.lin.weight, self.lin.bias, gelu=self.activation == "gelu")
        y = self.lin(x)
        return {"gelu": lambda t: F.gelu(t, approximate="tanh"), "relu": F.relu, "silu": F.silu, "tanh": torch.tanh, "none": lambda t: t}[self.activation](y)


class StaticMLP(nn.Sequential):
    """Fixed-width stack of fused linear + activation blocks, the last one linear."""

    def __init__(self, widths, activation: str = "gelu"):
        super().__init__(*[FusedLinearActivation(a, b, activation if i < len(widths) - 2 else "none") for i, (a, b) in enumerate(zip(widths[:-1], widths[1:]))])
