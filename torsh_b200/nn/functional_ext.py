"""Functional operators beyond the layer set (``crates/torsh-functional/src``): tensor decompositions
(``tensor_decomposition.rs``), wavelets (``wavelet.rs``), numerical calculus and root finding (``numerical.rs``),
higher-order tensor transformations (``transformations.rs``), gradient penalties (``regularization.rs``),
interpolation (``interpolation.rs``), counting ops (``data_ops.rs``), lazy expression chains (``lazy.rs``), dtype
promotion (``type_promotion.rs``), fusion analysis of op sequences (``fusion/``), classical optimisation routines
(``optimization/``) and random sampling (``random_ops/``).  All tensor code is device-agnostic."""
from __future__ import annotations

import math
from typing import Callable, Sequence

import torch
import torch.nn.functional as F


# ================================================================================================ tensor decompositions
def unfold(t: torch.Tensor, mode: int) -> torch.Tensor:
    return t.movedim(mode, 0).reshape(t.shape[mode], -1)


def khatri_rao(mats: Sequence[torch.Tensor]) -> torch.Tensor:
    out = mats[0]
    for m in mats[1:]:
        out = (out[:, None, :] * m[None, :, :]).reshape(-1, out.shape[1])
    return out


def cp_reconstruct(weights, factors):
    r = weights.numel()
    out = khatri_rao(factors) @ weights
    return out.reshape([f.shape[0] for f in factors])


def cp_decomposition(t: torch.Tensor, rank: int, iters: int = 200, tol: float = 1e-8, seed: int = 0):
    """CANDECOMP / PARAFAC by alternating least squares.  Returns ``(weights [rank], factors, relative error)`` with
    unit-norm factor columns."""
    g = torch.Generator().manual_seed(seed)
    facs = [torch.randn(n, rank, generator=g, dtype=t.dtype) for n in t.shape]
    norm_t, prev = t.norm(), math.inf
    w = torch.ones(rank, dtype=t.dtype)
    for _ in range(iters):
        for m in range(t.dim()):
            others = [facs[i] for i in range(t.dim()) if i != m]
            gram = torch.ones(rank, rank, dtype=t.dtype)
            for o in others:
                gram = gram * (o.t() @ o)
            facs[m] = unfold(t, m) @ khatri_rao(others) @ torch.linalg.pinv(gram)
            w = facs[m].norm(dim=0).clamp(min=1e-30)
            facs[m] = facs[m] / w
        err = float((t - cp_reconstruct(w, facs)).norm() / norm_t)
        if abs(prev - err) < tol:
            break
        prev = err
    return w, facs, err


def mode_dot(t: torch.Tensor, m: torch.Tensor, mode: int) -> torch.Tensor:
    return torch.tensordot(m, t, dims=([1], [mode])).movedim(0, mode)


def tucker_reconstruct(core, factors):
    out = core
    for i, f in enumerate(factors):
        out = mode_dot(out, f, i)
    return out


def tucker_decomposition(t: torch.Tensor, ranks: Sequence[int], iters: int = 50, tol: float = 1e-9):
    """Higher-order SVD initialisation followed by higher-order orthogonal iteration.  Returns ``(core, factors, error)``."""
    facs = [torch.linalg.svd(unfold(t, m), full_matrices=False).U[:, :r] for m, r in enumerate(ranks)]
    prev = math.inf
    for _ in range(iters):
        for m in range(t.dim()):
            y = t
            for i, f in enumerate(facs):
                if i != m:
                    y = mode_dot(y, f.t(), i)
            facs[m] = torch.linalg.svd(unfold(y, m), full_matrices=False).U[:, :ranks[m]]
        core = t
        for i, f in enumerate(facs):
            core = mode_dot(core, f.t(), i)
        err = float((t - tucker_reconstruct(core, facs)).norm() / t.norm())
        if abs(prev - err) < tol:
            break
        prev = err
    return core, facs, err


def tensor_train(t: torch.Tensor, max_rank: int, tol: float = 0.0):
    """TT-SVD: a chain of 3-way cores ``[r_{k-1}, n_k, r_k]``."""
    cores, r, cur = [], 1, t
    for n in t.shape[:-1]:
        cur = cur.reshape(r * n, -1)
        u, s, vh = torch.linalg.svd(cur, full_matrices=False)
        keep = min(max_rank, int((s > tol * s[0]).sum()) if tol > 0 else len(s))
        cores.append(u[:, :keep].reshape(r, n, keep))
        cur, r = s[:keep, None] * vh[:keep], keep
    cores.append(cur.reshape(r, t.shape[-1], 1))
    return cores


def tt_reconstruct(cores):
    out = cores[0]
    for c in cores[1:]:
        out = torch.tensordot(out, c, dims=([-1], [0]))
    return out.squeeze(0).squeeze(-1)


# ================================================================================================ wavelets
_S3 = math.sqrt(3)
WAVELETS = {
    "haar": [1 / math.sqrt(2), 1 / math.sqrt(2)],
    "db2": [(1 + _S3) / (4 * math.sqrt(2)), (3 + _S3) / (4 * math.sqrt(2)), (3 - _S3) / (4 * math.sqrt(2)), (1 - _S3) / (4 * math.sqrt(2))],
    "db3": [0.3326705529500826, 0.8068915093110925, 0.4598775021184915, -0.1350110200102546, -0.0854412738820267, 0.0352262918857095],
    "db4": [0.2303778133088965, 0.7148465705529157, 0.6308807679298589, -0.0279837694168599, -0.1870348117190930, 0.0308413818355607,
            0.0328830116668852, -0.0105974017850690],
    "sym4": [0.0322231006040427, -0.0126039672620378, -0.0992195435768472, 0.2978577956052774, 0.8037387518059161, 0.4976186676320155,
             -0.0296355276459985, -0.0757657147892733],
}


def _filters(name, like):
    h = like.new_tensor(WAVELETS[name])                                        # scaling (low-pass) reconstruction filter
    g = h.flip(0) * like.new_tensor([(-1.0) ** k for k in range(len(h))])      # wavelet (high-pass): quadrature mirror
    return h, g


def dwt_1d(x: torch.Tensor, wavelet: str = "haar"):
    """One level of the periodic orthogonal DWT along the last axis (even length): ``(approximation, detail)``."""
    h, g = _filters(wavelet, x)
    n, L = x.shape[-1], len(h)
    idx = (torch.arange(0, n, 2, device=x.device)[:, None] + torch.arange(L, device=x.device)[None]) % n
    win = x[..., idx]                                                          # [..., n/2, L]
    return win @ h, win @ g


def idwt_1d(a: torch.Tensor, d: torch.Tensor, wavelet: str = "haar"):
    h, g = _filters(wavelet, a)
    n, L = 2 * a.shape[-1], len(h)
    idx = (torch.arange(0, n, 2, device=a.device)[:, None] + torch.arange(L, device=a.device)[None]) % n
    contrib = a[..., None] * h + d[..., None] * g                              # [..., n/2, L]
    out = a.new_zeros(*a.shape[:-1], n)
    return out.index_add_(-1, idx.reshape(-1), contrib.reshape(*a.shape[:-1], -1))


def wavedec(x, wavelet="haar", level: int | None = None):
    """``[cA_n, cD_n, ..., cD_1]``."""
    level = level or max(1, int(math.log2(x.shape[-1] / (len(WAVELETS[wavelet]) - 1))) if len(WAVELETS[wavelet]) > 2 else int(math.log2(x.shape[-1])))
    out, a = [], x
    for _ in range(level):
        if a.shape[-1] % 2 or a.shape[-1] < 2:
            break
        a, d = dwt_1d(a, wavelet)
        out.append(d)
    return [a] + out[::-1]


def waverec(coeffs, wavelet="haar"):
    a = coeffs[0]
    for d in coeffs[1:]:
        a = idwt_1d(a, d, wavelet)
    return a


def dwt_2d(x, wavelet="haar"):
    """``(LL, (LH, HL, HH))`` of the last two axes."""
    lo, hi = dwt_1d(x, wavelet)
    ll, lh = dwt_1d(lo.transpose(-1, -2), wavelet)
    hl, hh = dwt_1d(hi.transpose(-1, -2), wavelet)
    t = lambda z: z.transpose(-1, -2)
    return t(ll), (t(lh), t(hl), t(hh))


def idwt_2d(ll, details, wavelet="haar"):
    lh, hl, hh = details
    t = lambda z: z.transpose(-1, -2)
    lo = t(idwt_1d(t(ll), t(lh), wavelet))
    hi = t(idwt_1d(t(hl), t(hh), wavelet))
    return idwt_1d(lo, hi, wavelet)


def cwt(x: torch.Tensor, scales, wavelet: str = "morlet", w0: float = 6.0):
    """Continuous wavelet transform along the last axis by FFT convolution; rows are scales.  ``morlet`` (complex) or
    ``mexican_hat`` (real)."""
    n = x.shape[-1]
    freqs = torch.fft.fftfreq(n, device=x.device) * 2 * math.pi
    xf = torch.fft.fft(x.to(torch.complex64 if x.dtype != torch.float64 else torch.complex128))
    rows = []
    for s in scales:
        sw = s * freqs
        if wavelet == "morlet":
            psi = math.pi ** -0.25 * torch.exp(-0.5 * (sw - w0) ** 2) * (freqs > 0)
        else:
            psi = (2 / math.sqrt(3)) * math.pi ** -0.25 * sw ** 2 * torch.exp(-0.5 * sw ** 2) * math.sqrt(2 * math.pi) / math.sqrt(2 * math.pi)
        rows.append(torch.fft.ifft(xf * psi * math.sqrt(s)))
    return torch.stack(rows, -2)


def wavelet_denoise(x, wavelet="db4", level=3, mode="soft"):
    """Universal-threshold shrinkage of the detail coefficients (noise level from the finest scale's median)."""
    c = wavedec(x, wavelet, level)
    sigma = c[-1].abs().median() / 0.6745
    thr = sigma * math.sqrt(2 * math.log(x.shape[-1]))
    shrink = (lambda d: torch.sign(d) * (d.abs() - thr).clamp(min=0)) if mode == "soft" else (lambda d: d * (d.abs() > thr))
    return waverec([c[0]] + [shrink(d) for d in c[1:]], wavelet)


# ================================================================================================ numerical calculus
def trapz(y, x=None, dx=1.0, dim=-1): return torch.trapezoid(y, x, dim=dim) if x is not None else torch.trapezoid(y, dx=dx, dim=dim)
def cumtrapz(y, x=None, dx=1.0, dim=-1): return torch.cumulative_trapezoid(y, x, dim=dim) if x is not None else torch.cumulative_trapezoid(y, dx=dx, dim=dim)


def simps(y, dx=1.0):
    """Composite Simpson over the last axis (odd sample count; an even count adds a trapezoid for the last interval)."""
    n = y.shape[-1]
    if n % 2 == 0:
        return simps(y[..., :-1], dx) + 0.5 * dx * (y[..., -2] + y[..., -1])
    return dx / 3 * (y[..., 0] + y[..., -1] + 4 * y[..., 1:-1:2].sum(-1) + 2 * y[..., 2:-1:2].sum(-1))


def gaussian_quad(f: Callable, a: float, b: float, n: int = 16, dtype=torch.float64):
    """Gauss-Legendre rule with ``n`` nodes (nodes from the Jacobi matrix eigenvalues)."""
    k = torch.arange(1, n, dtype=dtype)
    beta = k / torch.sqrt(4 * k * k - 1)
    nodes, vec = torch.linalg.eigh(torch.diag(beta, 1) + torch.diag(beta, -1))
    w = 2 * vec[0] ** 2
    return ((b - a) / 2 * (w * f((b - a) / 2 * nodes + (a + b) / 2)).sum())


def adaptive_quad(f: Callable, a: float, b: float, tol: float = 1e-8, max_depth: int = 40) -> float:
    """Adaptive Simpson with Richardson error control."""
    def simpson(fa, fm, fb, a, b): return (b - a) / 6 * (fa + 4 * fm + fb)
    def rec(a, b, fa, fm, fb, whole, tol, depth):
        m = (a + b) / 2
        flm, frm = f((a + m) / 2), f((m + b) / 2)
        left, right = simpson(fa, flm, fm, a, m), simpson(fm, frm, fb, m, b)
        if depth >= max_depth or abs(left + right - whole) <= 15 * tol:
            return left + right + (left + right - whole) / 15
        return rec(a, m, fa, flm, fm, left, tol / 2, depth + 1) + rec(m, b, fm, frm, fb, right, tol / 2, depth + 1)
    fa, fm, fb = f(a), f((a + b) / 2), f(b)
    return rec(a, b, fa, fm, fb, simpson(fa, fm, fb, a, b), tol, 0)


def gradient(y: torch.Tensor, dx: float = 1.0, dim: int = -1): return torch.gradient(y, spacing=dx, dim=dim)[0]
def second_derivative(f: Callable, x: torch.Tensor, h: float = 1e-3): return (f(x + h) - 2 * f(x) + f(x - h)) / (h * h)


def partial_derivative(f: Callable, x: torch.Tensor, index: int, h: float = 1e-4):
    e = torch.zeros_like(x)
    e[..., index] = h
    return (f(x + e) - f(x - e)) / (2 * h)


def bisection(f: Callable, a: float, b: float, tol: float = 1e-10, max_iter: int = 200) -> float:
    fa, fb = f(a), f(b)
    if fa * fb > 0:
        raise ValueError("bisection needs a sign change over [a, b]")
    for _ in range(max_iter):
        m = (a + b) / 2
        fm = f(m)
        if abs(fm) < tol or (b - a) / 2 < tol:
            return m
        a, fa, b = (m, fm, b) if fa * fm > 0 else (a, fa, m)
    return (a + b) / 2


def newton_raphson(f: Callable, x0, tol: float = 1e-10, max_iter: int = 50):
    """Newton's method for a scalar or vector function; the Jacobian comes from autograd."""
    x = torch.as_tensor(x0, dtype=torch.float64).clone()
    for _ in range(max_iter):
        fx = f(x)
        if fx.abs().max() < tol:
            break
        if x.dim() == 0:
            x = x - fx / torch.autograd.functional.jacobian(f, x)
        else:
            x = x - torch.linalg.solve(torch.autograd.functional.jacobian(f, x), fx)
    return x


# ================================================================================================ transformations
def tensor_map(f: Callable, t: torch.Tensor, dim: int | None = None):
    """Apply ``f`` to every element (``dim=None``, vectorised with ``vmap``) or to every slice along ``dim``."""
    if dim is None:
        return torch.vmap(f)(t.reshape(-1)).reshape(t.shape)
    return torch.stack([f(s) for s in t.unbind(dim)], dim)


def tensor_zip(f: Callable, a: torch.Tensor, b: torch.Tensor): a, b = torch.broadcast_tensors(a, b); return torch.vmap(f)(a.reshape(-1), b.reshape(-1)).reshape(a.shape)


def tensor_fold(f: Callable, t: torch.Tensor, init, dim: int = 0):
    acc = init
    for s in t.unbind(dim):
        acc = f(acc, s)
    return acc


def tensor_scan(f: Callable, t: torch.Tensor, init=None, dim: int = 0):
    """Inclusive scan with a binary function along ``dim``."""
    out, acc = [], init
    for s in t.unbind(dim):
        acc = s if acc is None else f(acc, s)
        out.append(acc)
    return torch.stack(out, dim)


def tensor_reduce(f: Callable, t: torch.Tensor, dim: int = 0):
    parts = list(t.unbind(dim))
    while len(parts) > 1:                                                     # pairwise tree: log depth, better rounding than a chain
        parts = [f(parts[i], parts[i + 1]) if i + 1 < len(parts) else parts[i] for i in range(0, len(parts), 2)]
    return parts[0]


def tensor_outer(*ts: torch.Tensor):
    out = ts[0]
    for t in ts[1:]:
        out = out[(...,) + (None,) * t.dim()] * t
    return out


def tensor_contract(a, b, dims_a: Sequence[int], dims_b: Sequence[int]): return torch.tensordot(a, b, dims=(list(dims_a), list(dims_b)))


def einsum_optimized(eq: str, *ops: torch.Tensor):
    """Greedy pairwise contraction order chosen by the size of each intermediate; returns ``(result, order, cost)``."""
    ins, out = eq.replace(" ", "").split("->")
    terms = ins.split(",")
    size = {c: t.shape[i] for term, t in zip(terms, ops) for i, c in enumerate(term)}
    live, tens, order, cost = list(terms), list(ops), [], 0
    while len(live) > 1:
        best = None
        for i in range(len(live)):
            for j in range(i + 1, len(live)):
                rest = set("".join(live[k] for k in range(len(live)) if k not in (i, j))) | set(out)
                keep = "".join(c for c in dict.fromkeys(live[i] + live[j]) if c in rest)
                flops = math.prod(size[c] for c in set(live[i] + live[j]))
                inter = math.prod(size[c] for c in keep) if keep else 1
                if best is None or (inter, flops) < best[0]:
                    best = ((inter, flops), i, j, keep)
        (_, flops), i, j, keep = best
        tens_ij = torch.einsum(f"{live[i]},{live[j]}->{keep}", tens[i], tens[j])
        order.append((live[i], live[j], keep))
        cost += flops
        for k in sorted((i, j), reverse=True):
            live.pop(k); tens.pop(k)
        live.append(keep); tens.append(tens_ij)
    return torch.einsum(f"{live[0]}->{out}", tens[0]), order, cost


# ================================================================================================ gradient penalties
def gradient_penalty(critic: Callable, real: torch.Tensor, fake: torch.Tensor, target: float = 1.0, generator=None):
    """WGAN-GP: ``(||grad critic(x_hat)|| - target)^2`` at random interpolates of real and fake samples."""
    eps = torch.rand(real.shape[0], *[1] * (real.dim() - 1), generator=generator).to(real)
    xh = (eps * real + (1 - eps) * fake).detach().requires_grad_(True)
    g, = torch.autograd.grad(critic(xh).sum(), xh, create_graph=True)
    return ((g.flatten(1).norm(dim=1) - target) ** 2).mean()


def r1_gradient_penalty(critic: Callable, real: torch.Tensor):
    x = real.detach().requires_grad_(True)
    g, = torch.autograd.grad(critic(x).sum(), x, create_graph=True)
    return 0.5 * g.flatten(1).pow(2).sum(1).mean()


def r2_gradient_penalty(critic: Callable, fake: torch.Tensor): return r1_gradient_penalty(critic, fake)


def spectral_gradient_penalty(weight: torch.Tensor, iters: int = 20):
    """Largest singular value of a weight matrix by power iteration (differentiable through the final products)."""
    w = weight.flatten(1)
    v = F.normalize(torch.ones(w.shape[1], dtype=w.dtype, device=w.device), dim=0)
    with torch.no_grad():
        for _ in range(iters):
            u = F.normalize(w @ v, dim=0)
            v = F.normalize(w.t() @ u, dim=0)
    return u @ w @ v


def consistency_penalty(model: Callable, x: torch.Tensor, augment: Callable):
    return (model(x) - model(augment(x))).pow(2).mean()


# ================================================================================================ interpolation
def interp1d(x: torch.Tensor, xp: torch.Tensor, fp: torch.Tensor, kind: str = "linear"):
    """Values at ``x`` of the function sampled at increasing ``xp``; ends are clamped (``nearest`` / ``linear``)."""
    i = torch.searchsorted(xp, x.contiguous()).clamp(1, len(xp) - 1)
    x0, x1 = xp[i - 1], xp[i]
    if kind == "nearest":
        return torch.where((x - x0).abs() <= (x1 - x).abs(), fp[i - 1], fp[i])
    t = ((x - x0) / (x1 - x0)).clamp(0, 1)
    return fp[i - 1] + t * (fp[i] - fp[i - 1])


def spline1d(x: torch.Tensor, xp: torch.Tensor, fp: torch.Tensor):
    """Natural cubic spline (second derivative zero at both ends)."""
    n = len(xp)
    h = xp[1:] - xp[:-1]
    a = torch.zeros(n, n, dtype=fp.dtype)
    rhs = torch.zeros(n, dtype=fp.dtype)
    a[0, 0] = a[-1, -1] = 1
    for k in range(1, n - 1):
        a[k, k - 1], a[k, k], a[k, k + 1] = h[k - 1], 2 * (h[k - 1] + h[k]), h[k]
        rhs[k] = 3 * ((fp[k + 1] - fp[k]) / h[k] - (fp[k] - fp[k - 1]) / h[k - 1])
    c = torch.linalg.solve(a, rhs)
    b = (fp[1:] - fp[:-1]) / h - h * (2 * c[:-1] + c[1:]) / 3
    d = (c[1:] - c[:-1]) / (3 * h)
    i = (torch.searchsorted(xp, x.contiguous()) - 1).clamp(0, n - 2)
    t = x - xp[i]
    return fp[i] + b[i] * t + c[i] * t ** 2 + d[i] * t ** 3


def lanczos_interp1d(x: torch.Tensor, fp: torch.Tensor, a: int = 3):
    """Resampling of uniformly spaced samples ``fp`` (at 0, 1, 2, ...) at positions ``x`` with the Lanczos-``a`` kernel."""
    k = torch.arange(-a + 1, a + 1)
    base = torch.floor(x).long()
    idx = (base[:, None] + k[None]).clamp(0, len(fp) - 1)
    t = x[:, None] - (base[:, None] + k[None]).to(x)
    w = torch.where(t.abs() < a, torch.sinc(t) * torch.sinc(t / a), torch.zeros_like(t))
    return (w * fp[idx]).sum(1) / w.sum(1)


def barycentric_interp(x: torch.Tensor, xp: torch.Tensor, fp: torch.Tensor):
    """Polynomial through all nodes, evaluated in barycentric form (stable for Chebyshev nodes)."""
    diff = xp[:, None] - xp[None, :]
    diff.fill_diagonal_(1.0)
    w = 1 / diff.prod(1)
    d = x[:, None] - xp[None, :]
    exact = d == 0
    d = torch.where(exact, torch.ones_like(d), d)
    val = ((w * fp) / d).sum(1) / (w / d).sum(1)
    return torch.where(exact.any(1), fp[exact.float().argmax(1)], val)


def interp2d(img: torch.Tensor, x: torch.Tensor, y: torch.Tensor, mode: str = "bilinear"):
    """Samples a ``[H, W]`` grid at pixel coordinates."""
    h, w = img.shape
    grid = torch.stack([(2 * x + 1) / w - 1, (2 * y + 1) / h - 1], -1).reshape(1, 1, -1, 2).to(img)
    return F.grid_sample(img[None, None], grid, mode=mode, padding_mode="border", align_corners=False).reshape(x.shape)


# ================================================================================================ counting
def bincount(x, minlength=0, weights=None): return torch.bincount(x, weights=weights, minlength=minlength)
def unique(x, sorted=True, return_inverse=False, return_counts=False): return torch.unique(x, sorted=sorted, return_inverse=return_inverse, return_counts=return_counts)


def histogram(x, bins=10, range=None, density=False):
    lo, hi = range if range is not None else (float(x.min()), float(x.max()))
    edges = torch.linspace(lo, hi, bins + 1, dtype=torch.float64)
    return histogram_with_edges(x, edges, density), edges


def histogram_with_edges(x, edges, density=False):
    """Right-open bins except the last, which includes its upper edge."""
    xv = x.reshape(-1).double()
    keep = (xv >= edges[0]) & (xv <= edges[-1])
    idx = (torch.searchsorted(edges, xv[keep], right=True) - 1).clamp(max=len(edges) - 2)
    h = torch.bincount(idx, minlength=len(edges) - 1).double()
    return h / (h.sum() * (edges[1:] - edges[:-1])) if density else h


def value_counts(x, normalize=False, sort=True):
    v, c = torch.unique(x, return_counts=True)
    if sort:
        o = c.argsort(descending=True, stable=True)
        v, c = v[o], c[o]
    return v, (c.double() / c.sum() if normalize else c)


# ================================================================================================ lazy expressions
class LazyTensor:
    """Records a chain of element-wise operations and evaluates it once.  ``optimize`` folds consecutive scalar
    additions / multiplications and removes identities before evaluation."""

    _UNARY = {"abs": torch.abs, "exp": torch.exp, "log": torch.log, "sin": torch.sin, "cos": torch.cos, "tanh": torch.tanh, "relu": torch.relu}

    def __init__(self, source, ops=()):
        self.source, self.ops = source, list(ops)

    def _push(self, *op): return LazyTensor(self.source, self.ops + [op])
    def add_scalar(self, s): return self._push("add_scalar", s)
    def sub_scalar(self, s): return self._push("add_scalar", -s)
    def mul_scalar(self, s): return self._push("mul_scalar", s)
    def add(self, o): return self._push("add", o)
    def sub(self, o): return self._push("sub", o)
    def mul(self, o): return self._push("mul", o)
    def div(self, o): return self._push("div", o)
    def sum(self, dim=None): return self._push("sum", dim)
    def mean(self, dim=None): return self._push("mean", dim)
    def reshape(self, *shape): return self._push("reshape", shape)
    def transpose(self, a, b): return self._push("transpose", a, b)
    def depth(self): return len(self.ops)

    def __getattr__(self, name):
        if name in LazyTensor._UNARY:
            return lambda: self._push(name)
        raise AttributeError(name)

    def optimize(self) -> "LazyTensor":
        out: list = []
        for op in self.ops:
            if out and op[0] == out[-1][0] == "add_scalar":
                out[-1] = ("add_scalar", out[-1][1] + op[1])
            elif out and op[0] == out[-1][0] == "mul_scalar":
                out[-1] = ("mul_scalar", out[-1][1] * op[1])
            elif out and op[0] == out[-1][0] and op[0] in ("abs", "relu"):
                continue                                                      # idempotent
            else:
                out.append(op)
        out = [op for op in out if op not in (("add_scalar", 0), ("add_scalar", 0.0), ("mul_scalar", 1), ("mul_scalar", 1.0))]
        return LazyTensor(self.source, out)

    def evaluate(self) -> torch.Tensor:
        val = lambda o: o.evaluate() if isinstance(o, LazyTensor) else o
        x = val(self.source)
        for op in self.ops:
            k = op[0]
            if k in self._UNARY:
                x = self._UNARY[k](x)
            elif k == "add_scalar":
                x = x + op[1]
            elif k == "mul_scalar":
                x = x * op[1]
            elif k in ("add", "sub", "mul", "div"):
                x = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}[k](x, val(op[1]))
            elif k in ("sum", "mean"):
                x = getattr(x, k)() if op[1] is None else getattr(x, k)(op[1])
            elif k == "reshape":
                x = x.reshape(*op[1])
            elif k == "transpose":
                x = x.transpose(op[1], op[2])
        return x


def lazy(t): return LazyTensor(t)


# ================================================================================================ type promotion
_CATEGORY = {torch.bool: 0, torch.uint8: 1, torch.int8: 1, torch.int16: 1, torch.int32: 1, torch.int64: 1, torch.float16: 2, torch.bfloat16: 2,
             torch.float32: 2, torch.float64: 2, torch.complex64: 3, torch.complex128: 3}


def get_type_category(dt): return ["bool", "integer", "floating", "complex"][_CATEGORY[dt]]
def get_type_precision(dt): return torch.finfo(dt).bits if dt.is_floating_point or dt.is_complex else (1 if dt == torch.bool else torch.iinfo(dt).bits)
def promote_types(a, b): return torch.promote_types(a, b)
def can_cast_safely(src, dst): return torch.can_cast(src, dst) and torch.promote_types(src, dst) == dst


def promote_multiple_types(dts):
    out = dts[0]
    for d in dts[1:]:
        out = torch.promote_types(out, d)
    return out


def result_type(*operands):
    """Tensors with dimensions outrank zero-dimensional tensors and Python scalars of the same category."""
    out = operands[0] if isinstance(operands[0], torch.Tensor) else torch.tensor(operands[0])
    dt = out.dtype
    for o in operands[1:]:
        dt = torch.result_type(torch.empty(out.shape, dtype=dt) if out.dim() else torch.tensor(0, dtype=dt), o)
        out = out if out.dim() or not isinstance(o, torch.Tensor) else o
    return dt


def promote_tensors(*ts):
    dt = promote_multiple_types([t.dtype for t in ts])
    return tuple(t.to(dt) for t in ts)


def reduction_result_type(dt, op: str):
    if op in ("mean", "var", "std") and not (dt.is_floating_point or dt.is_complex):
        return torch.float32
    if op in ("sum", "prod") and _CATEGORY[dt] <= 1:
        return torch.int64
    if op in ("argmax", "argmin", "count"):
        return torch.int64
    if op in ("any", "all"):
        return torch.bool
    return dt


# ================================================================================================ fusion analysis
_ELEMENTWISE = {"add", "sub", "mul", "div", "relu", "sigmoid", "tanh", "silu", "gelu", "exp", "neg", "scale", "bias"}
_FUSED = {("mul", "add"): "fused_mul_add", ("add", "mul"): "fused_add_mul", ("add", "relu"): "fused_add_relu", ("relu", "add"): "fused_relu_add",
          ("sigmoid", "mul"): "fused_sigmoid_mul", ("tanh", "scale"): "fused_tanh_scale", ("add", "relu", "mul"): "fused_add_relu_mul"}


def detect_fusible_patterns(ops: Sequence[str]) -> list[dict]:
    """Longest-first scan of an op-name sequence for patterns with a fused kernel in :mod:`torsh_b200.nn.functional`, plus
    maximal runs of element-wise ops that a generated kernel could cover."""
    out, i = [], 0
    while i < len(ops):
        for n in (3, 2):
            if tuple(ops[i:i + n]) in _FUSED:
                out.append({"start": i, "length": n, "kernel": _FUSED[tuple(ops[i:i + n])]})
                i += n
                break
        else:
            j = i
            while j < len(ops) and ops[j] in _ELEMENTWISE:
                j += 1
            if j - i >= 2:
                out.append({"start": i, "length": j - i, "kernel": "generated_elementwise"})
                i = j
            else:
                i += 1
    return out


def fusion_benefit_estimate(ops: Sequence[str], numel: int, bytes_per_element: int = 2, bandwidth: float = 6.6e12, launch: float = 3e-6) -> dict:
    """Memory-bound model: unfused, every op reads and writes the tensor and pays a launch; fused, the run does so once."""
    pats = detect_fusible_patterns(ops)
    unfused = len(ops) * (2 * numel * bytes_per_element / bandwidth + launch)
    covered = sum(p["length"] for p in pats)
    fused = (len(ops) - covered + len(pats)) * (2 * numel * bytes_per_element / bandwidth + launch)
    return {"patterns": pats, "unfused_s": unfused, "fused_s": fused, "speedup": unfused / fused if fused else 1.0}


class AdaptiveFusion:
    """Learns from measurements whether fusing a pattern pays: an exponential average of observed speed-ups per pattern."""

    def __init__(self, learning_rate: float = 0.3, threshold: float = 1.05):
        self.lr, self.threshold, self.history = learning_rate, threshold, {}

    def record_performance(self, pattern, unfused_s: float, fused_s: float):
        s = unfused_s / max(fused_s, 1e-12)
        self.history[pattern] = s if pattern not in self.history else (1 - self.lr) * self.history[pattern] + self.lr * s

    def should_fuse_adaptive(self, pattern, default: bool = True): return self.history[pattern] >= self.threshold if pattern in self.history else default
    def history_size(self): return len(self.history)
    def clear_history(self): self.history.clear()


# ================================================================================================ optimisation routines
def backtracking_line_search(f: Callable, x, d, g, t0=1.0, c1=1e-4, shrink=0.5, max_iter=50):
    fx, slope, t = f(x), float(g @ d), t0
    for _ in range(max_iter):
        if f(x + t * d) <= fx + c1 * t * slope:
            return t
        t *= shrink
    return t


def wolfe_line_search(f: Callable, grad: Callable, x, d, t0=1.0, c1=1e-4, c2=0.9, max_iter=30):
    """Bracketing search for a step meeting the strong Wolfe conditions."""
    fx, slope, lo, hi, t = f(x), float(grad(x) @ d), 0.0, math.inf, t0
    for _ in range(max_iter):
        if f(x + t * d) > fx + c1 * t * slope:
            hi = t
        elif abs(float(grad(x + t * d) @ d)) > c2 * abs(slope):
            if float(grad(x + t * d) @ d) > 0:
                hi = t
            else:
                lo = t
        else:
            return t
        t = (lo + hi) / 2 if hi < math.inf else 2 * t
    return t


def gradient_descent(f, grad, x0, lr=0.1, momentum=0.0, iters=500, tol=1e-8):
    x, v = x0.clone(), torch.zeros_like(x0)
    for i in range(iters):
        g = grad(x)
        if g.norm() < tol:
            break
        v = momentum * v - lr * g
        x = x + v
    return x, i + 1


def bfgs(f, grad, x0, iters=200, tol=1e-8):
    n = x0.numel()
    x, hinv = x0.clone(), torch.eye(n, dtype=x0.dtype)
    g = grad(x)
    for i in range(iters):
        if g.norm() < tol:
            break
        d = -hinv @ g
        t = wolfe_line_search(f, grad, x, d)
        s = t * d
        xn = x + s
        gn = grad(xn)
        y = gn - g
        sy = float(s @ y)
        if sy > 1e-12:
            rho, eye = 1 / sy, torch.eye(n, dtype=x0.dtype)
            hinv = (eye - rho * torch.outer(s, y)) @ hinv @ (eye - rho * torch.outer(y, s)) + rho * torch.outer(s, s)
        x, g = xn, gn
    return x, i + 1


def conjugate_gradient_minimize(f, grad, x0, iters=500, tol=1e-8):
    """Polak-Ribiere+ with restarts."""
    x, g = x0.clone(), grad(x0)
    d = -g
    for i in range(iters):
        if g.norm() < tol:
            break
        if float(g @ d) >= 0:
            d = -g
        t = wolfe_line_search(f, grad, x, d, c2=0.4)
        x = x + t * d
        gn = grad(x)
        beta = max(0.0, float(gn @ (gn - g) / (g @ g)))
        d, g = -gn + beta * d, gn
    return x, i + 1


# ================================================================================================ random sampling
def _gen(seed): return torch.Generator().manual_seed(seed) if seed is not None else None
def uniform(shape, lo=0.0, hi=1.0, seed=None): return lo + (hi - lo) * torch.rand(shape, generator=_gen(seed))
def normal(shape, mean=0.0, std=1.0, seed=None): return mean + std * torch.randn(shape, generator=_gen(seed))
def exponential(shape, rate=1.0, seed=None): return -torch.log1p(-torch.rand(shape, generator=_gen(seed))) / rate
def laplace(shape, loc=0.0, scale=1.0, seed=None): u = torch.rand(shape, generator=_gen(seed)) - 0.5; return loc - scale * torch.sign(u) * torch.log1p(-2 * u.abs())
def cauchy(shape, loc=0.0, scale=1.0, seed=None): return loc + scale * torch.tan(math.pi * (torch.rand(shape, generator=_gen(seed)) - 0.5))
def log_normal(shape, mean=0.0, std=1.0, seed=None): return torch.exp(normal(shape, mean, std, seed))
def bernoulli(shape, p=0.5, seed=None): return (torch.rand(shape, generator=_gen(seed)) < p).float()
def geometric(shape, p=0.5, seed=None): return torch.floor(torch.log1p(-torch.rand(shape, generator=_gen(seed))) / math.log1p(-p)) + 1
def randint(shape, lo, hi, seed=None): return torch.randint(lo, hi, shape, generator=_gen(seed))
def randperm(n, seed=None): return torch.randperm(n, generator=_gen(seed))
def multinomial(probs, n, replacement=True, seed=None): return torch.multinomial(probs, n, replacement, generator=_gen(seed))


def gamma(shape, alpha: float, rate: float = 1.0, seed=None):
    """Marsaglia-Tsang squeeze (with the ``alpha < 1`` boost), vectorised with rejection rounds."""
    g = _gen(seed)
    boost = alpha < 1
    a = alpha + 1 if boost else alpha
    d, out = a - 1 / 3, torch.empty(shape).reshape(-1)
    c, todo = 1 / math.sqrt(9 * d), torch.ones(out.numel(), dtype=torch.bool)
    while todo.any():
        n = int(todo.sum())
        x, u = torch.randn(n, generator=g), torch.rand(n, generator=g)
        v = (1 + c * x) ** 3
        ok = (v > 0) & (torch.log(u) < 0.5 * x * x + d - d * v + d * torch.log(v.clamp(min=1e-30)))
        idx = todo.nonzero().flatten()[ok]
        out[idx] = d * v[ok]
        todo[idx] = False
    if boost:
        out = out * torch.rand(out.shape, generator=g) ** (1 / alpha)
    return (out / rate).reshape(shape)


def beta(shape, a: float, b: float, seed=None):
    x = gamma(shape, a, seed=seed)
    y = gamma(shape, b, seed=None if seed is None else seed + 1)
    return x / (x + y)


def dirichlet(alpha: torch.Tensor, n: int, seed=None):
    g = torch.stack([gamma((n,), float(a), seed=None if seed is None else seed + i) for i, a in enumerate(alpha)], 1)
    return g / g.sum(1, keepdim=True)


def poisson(shape, lam: float, seed=None): return torch.poisson(torch.full(shape, float(lam)), generator=_gen(seed))
def binomial(shape, n: int, p: float, seed=None): return (torch.rand(*shape, n, generator=_gen(seed)) < p).sum(-1).float()


def multivariate_normal(mean: torch.Tensor, cov: torch.Tensor, n: int, seed=None):
    return mean + torch.randn(n, len(mean), generator=_gen(seed), dtype=mean.dtype) @ torch.linalg.cholesky(cov).t()


def truncated_normal(shape, mean=0.0, std=1.0, lo=-2.0, hi=2.0, seed=None):
    """Inverse-CDF sampling between ``lo`` and ``hi`` standard deviations."""
    cdf = lambda z: 0.5 * (1 + math.erf(z / math.sqrt(2)))
    u = torch.rand(shape, generator=_gen(seed)) * (cdf(hi) - cdf(lo)) + cdf(lo)
    return mean + std * math.sqrt(2) * torch.erfinv(2 * u - 1)
