"""Linear algebra beyond :mod:`torsh_b200.linalg` (``crates/torsh-linalg/src``): geometric multigrid, preconditioners and
equilibration, pivoted LU variants, iterative refinement, randomised range finding / eigendecomposition / Nystrom,
Lanczos and power iterations, scaling-and-squaring and Krylov matrix exponentials, low-rank updates, tridiagonal and
banded solves, subspace utilities, Procrustes alignment and a structural matrix report."""
from __future__ import annotations

import math

import torch


# ================================================================================================ multigrid
class MultigridSolver:
    """Geometric multigrid for the 1-D or 2-D Poisson problem ``-laplace(u) = f`` on the unit interval / square with zero
    boundary values (interior grid of ``n = 2^k - 1`` points per side): weighted Jacobi or red-black Gauss-Seidel
    smoothing, full-weighting restriction, linear interpolation, V or W cycles, exact solve on the coarsest grid."""

    def __init__(self, dim: int = 2, pre: int = 2, post: int = 2, smoother: str = "jacobi", omega: float = 0.8, cycle: str = "V", coarsest: int = 3):
        self.dim, self.pre, self.post, self.smoother, self.omega, self.gamma, self.coarsest = dim, pre, post, smoother, omega, 1 if cycle == "V" else 2, coarsest

    def apply(self, u):
        n = u.shape[-1]
        h2 = (1.0 / (n + 1)) ** 2
        p = torch.nn.functional.pad(u, (1, 1) * self.dim)
        if self.dim == 1:
            return (2 * u - p[:-2] - p[2:]) / h2
        return (4 * u - p[:-2, 1:-1] - p[2:, 1:-1] - p[1:-1, :-2] - p[1:-1, 2:]) / h2

    def _smooth(self, u, f, iters):
        n = u.shape[-1]
        h2, diag = (1.0 / (n + 1)) ** 2, 2.0 * self.dim
        for _ in range(iters):
            if self.smoother == "jacobi":
                u = u + self.omega * h2 / diag * (f - self.apply(u))
            else:
                idx = torch.arange(n)
                parity = (idx[:, None] + idx[None]) % 2 if self.dim == 2 else idx % 2
                for color in (0, 1):
                    r = f - self.apply(u)
                    u = torch.where(parity == color, u + h2 / diag * r, u)
        return u

    def _restrict(self, r):
        if self.dim == 1:
            return (r[:-2:2] + 2 * r[1:-1:2] + r[2::2]) / 4
        k = torch.tensor([[1.0, 2, 1], [2, 4, 2], [1, 2, 1]], dtype=r.dtype) / 16
        return torch.nn.functional.conv2d(r[None, None], k[None, None], stride=2)[0, 0]

    def _prolong(self, e, n):
        mode = "linear" if self.dim == 1 else "bilinear"
        p = torch.nn.functional.pad(e, (1, 1) * self.dim)[None, None]
        size = (n + 2,) * self.dim
        return torch.nn.functional.interpolate(p, size=size, mode=mode, align_corners=True)[0, 0][(slice(1, -1),) * self.dim]

    def _exact(self, f):
        n = f.shape[-1]
        a = torch.zeros(f.numel(), f.numel(), dtype=f.dtype)
        for i in range(f.numel()):
            e = torch.zeros(f.numel(), dtype=f.dtype); e[i] = 1
            a[:, i] = self.apply(e.reshape(f.shape)).reshape(-1)
        return torch.linalg.solve(a, f.reshape(-1)).reshape(f.shape)

    def cycle(self, u, f):
        n = u.shape[-1]
        if n <= self.coarsest:
            return self._exact(f)
        u = self._smooth(u, f, self.pre)
        rc = self._restrict(f - self.apply(u))
        ec = torch.zeros_like(rc)
        for _ in range(self.gamma):
            ec = self.cycle(ec, rc)
        return self._smooth(u + self._prolong(ec, n), f, self.post)

    def solve(self, f, tol: float = 1e-8, max_cycles: int = 50):
        u, history = torch.zeros_like(f), []
        fn = f.norm().clamp(min=1e-300)
        for _ in range(max_cycles):
            u = self.cycle(u, f)
            history.append(float((f - self.apply(u)).norm() / fn))
            if history[-1] < tol:
                break
        return u, history


# ================================================================================================ conditioning helpers
def equilibrate(a: torch.Tensor, iters: int = 10) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Ruiz scaling: diagonal ``r, c`` with ``diag(r) A diag(c)`` having rows and columns of unit max-norm; returns
    ``(scaled matrix, r, c)``."""
    r, c = torch.ones(a.shape[0], dtype=a.dtype), torch.ones(a.shape[1], dtype=a.dtype)
    b = a.clone()
    for _ in range(iters):
        dr, dc = b.abs().amax(1).clamp(min=1e-300).rsqrt(), b.abs().amax(0).clamp(min=1e-300).rsqrt()
        b, r, c = dr[:, None] * b * dc[None], r * dr, c * dc
    return b, r, c


def diagonal_preconditioner(a): d = a.diagonal().clone(); return lambda v: v / d


def ssor_preconditioner(a: torch.Tensor, omega: float = 1.0):
    d = torch.diag(a.diagonal())
    lo = torch.tril(a, -1)
    m1, m2 = d / omega + lo, d / omega + lo.t()
    scale = omega / (2 - omega)
    return lambda v: scale * torch.linalg.solve_triangular(m2, (d / omega) @ torch.linalg.solve_triangular(m1, v[:, None], upper=False), upper=True)[:, 0]


def lu_pivoted(a: torch.Tensor, strategy: str = "partial"):
    """``P A Q = L U`` with ``partial`` (row), ``complete`` (row and column) or ``rook`` pivoting; returns ``(P, L, U, Q)``
    as permutation index vectors and triangular factors, plus the growth factor ``max|U| / max|A|``."""
    n = a.shape[0]
    u, l = a.clone(), torch.eye(n, dtype=a.dtype)
    p, q = torch.arange(n), torch.arange(n)
    for k in range(n - 1):
        sub = u[k:, k:].abs()
        if strategy == "partial":
            i, j = int(sub[:, 0].argmax()), 0
        elif strategy == "complete":
            i, j = divmod(int(sub.argmax()), n - k)
        else:
            i, j = int(sub[:, 0].argmax()), 0
            for _ in range(2 * n):
                j2 = int(sub[i].argmax())
                i2 = int(sub[:, j2].argmax())
                if sub[i2, j2] <= sub[i, j]:
                    break
                i, j = i2, j2
        i, j = i + k, j + k
        if i != k:
            u[[k, i]] = u[[i, k]]; p[[k, i]] = p[[i, k]]; l[[k, i], :k] = l[[i, k], :k]
        if j != k:
            u[:, [k, j]] = u[:, [j, k]]; q[[k, j]] = q[[j, k]]
        if u[k, k] != 0:
            l[k + 1:, k] = u[k + 1:, k] / u[k, k]
            u[k + 1:] -= l[k + 1:, k:k + 1] * u[k:k + 1]
    return p, l, torch.triu(u), q, float(u.abs().max() / a.abs().max())


def solve_refined(a: torch.Tensor, b: torch.Tensor, low=torch.float32, iters: int = 5):
    """Mixed-precision iterative refinement: factor and solve in ``low`` precision, accumulate residual corrections in the
    precision of ``a``; returns the solution and the residual history."""
    lu, piv = torch.linalg.lu_factor(a.to(low))
    x = torch.linalg.lu_solve(lu, piv, b.to(low)[:, None])[:, 0].to(a.dtype)
    hist = []
    for _ in range(iters):
        r = b - a @ x
        hist.append(float(r.norm() / b.norm()))
        x = x + torch.linalg.lu_solve(lu, piv, r.to(low)[:, None])[:, 0].to(a.dtype)
    hist.append(float((b - a @ x).norm() / b.norm()))
    return x, hist


def solve_tridiagonal(lower, diag, upper, rhs):
    """Thomas algorithm (no pivoting; for diagonally dominant or SPD systems)."""
    n = len(diag)
    c, d = torch.zeros(n, dtype=diag.dtype), torch.zeros(n, dtype=diag.dtype)
    c[0], d[0] = (upper[0] / diag[0] if n > 1 else 0.0), rhs[0] / diag[0]
    for i in range(1, n):
        m = diag[i] - lower[i - 1] * c[i - 1]
        c[i] = upper[i] / m if i < n - 1 else 0.0
        d[i] = (rhs[i] - lower[i - 1] * d[i - 1]) / m
    x = d.clone()
    for i in range(n - 2, -1, -1):
        x[i] = d[i] - c[i] * x[i + 1]
    return x


def woodbury_solve(a_inv_apply, u: torch.Tensor, v: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Solves ``(A + U V^T) x = b`` given a routine for ``A^-1 y``: one small ``k x k`` solve."""
    aib = a_inv_apply(b)
    aiu = torch.stack([a_inv_apply(u[:, j]) for j in range(u.shape[1])], 1)
    small = torch.eye(u.shape[1], dtype=b.dtype) + v.t() @ aiu
    return aib - aiu @ torch.linalg.solve(small, v.t() @ aib)


# ================================================================================================ randomised and Krylov methods
def randomized_range_finder(a: torch.Tensor, rank: int, oversample: int = 8, power_iters: int = 2, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    q = torch.linalg.qr(a @ torch.randn(a.shape[1], rank + oversample, generator=g, dtype=a.dtype)).Q
    for _ in range(power_iters):
        q = torch.linalg.qr(a @ torch.linalg.qr(a.t() @ q).Q).Q
    return q


def randomized_eigh(a: torch.Tensor, rank: int, **kw):
    q = randomized_range_finder(a, rank, **kw)
    w, v = torch.linalg.eigh(q.t() @ a @ q)
    order = w.abs().argsort(descending=True)[:rank]
    return w[order], (q @ v)[:, order]


def nystrom(a: torch.Tensor, rank: int, seed: int = 0):
    """Low-rank factor ``F`` with ``A ~ F F^T`` for a positive semi-definite matrix (stabilised by a small shift)."""
    g = torch.Generator().manual_seed(seed)
    om = torch.linalg.qr(torch.randn(a.shape[0], rank, generator=g, dtype=a.dtype)).Q
    y = a @ om
    nu = 1e-10 * y.norm()
    y = y + nu * om
    c = torch.linalg.cholesky(om.t() @ y)
    return torch.linalg.solve_triangular(c, y.t(), upper=False).t()


def power_iteration(a: torch.Tensor, iters: int = 500, tol: float = 1e-12, seed: int = 0):
    v = torch.randn(a.shape[0], generator=torch.Generator().manual_seed(seed), dtype=a.dtype)
    v, lam = v / v.norm(), 0.0
    for _ in range(iters):
        w = a @ v
        new = float(v @ w)
        v = w / w.norm()
        if abs(new - lam) < tol * max(abs(new), 1):
            lam = new
            break
        lam = new
    return lam, v


def lanczos(a_apply, n: int, k: int, dtype=torch.float64, seed: int = 0):
    """``k`` steps with full re-orthogonalisation; returns the Ritz values and vectors of the symmetric operator."""
    q = torch.randn(n, generator=torch.Generator().manual_seed(seed), dtype=dtype)
    Q, alpha, beta = [q / q.norm()], [], []
    for j in range(k):
        w = a_apply(Q[j])
        alpha.append(float(w @ Q[j]))
        w = w - alpha[j] * Q[j] - (beta[j - 1] * Q[j - 1] if j else 0)
        for qi in Q:
            w = w - (w @ qi) * qi
        b = float(w.norm())
        if b < 1e-12 or j == k - 1:
            break
        beta.append(b); Q.append(w / b)
    m = len(alpha)
    T = torch.diag(torch.tensor(alpha, dtype=dtype)) + torch.diag(torch.tensor(beta[:m - 1], dtype=dtype), 1) + torch.diag(torch.tensor(beta[:m - 1], dtype=dtype), -1)
    w, s = torch.linalg.eigh(T)
    return w, torch.stack(Q[:m], 1) @ s


def expm_taylor(a: torch.Tensor, order: int = 18) -> torch.Tensor:
    """Scaling and squaring with a truncated Taylor series."""
    s = max(0, int(math.ceil(math.log2(max(float(torch.linalg.matrix_norm(a, 1)), 1e-300)))) + 1)
    x = a / 2 ** s
    out, term = torch.eye(a.shape[0], dtype=a.dtype), torch.eye(a.shape[0], dtype=a.dtype)
    for k in range(1, order + 1):
        term = term @ x / k
        out = out + term
    for _ in range(s):
        out = out @ out
    return out


def expm_multiply(a_apply, v: torch.Tensor, t: float = 1.0, k: int = 30) -> torch.Tensor:
    """``exp(t A) v`` from a ``k``-step Arnoldi projection (no dense exponential of ``A``)."""
    beta = v.norm()
    V, H = [v / beta], torch.zeros(k + 1, k, dtype=v.dtype)
    m = k
    for j in range(k):
        w = a_apply(V[j])
        for i in range(j + 1):
            H[i, j] = w @ V[i]
            w = w - H[i, j] * V[i]
        H[j + 1, j] = w.norm()
        if H[j + 1, j] < 1e-12:
            m = j + 1
            break
        V.append(w / H[j + 1, j])
    e1 = torch.zeros(m, dtype=v.dtype); e1[0] = 1
    return beta * torch.stack(V[:m], 1) @ (torch.linalg.matrix_exp(t * H[:m, :m]) @ e1)


# ================================================================================================ subspaces / alignment / report
def null_space(a: torch.Tensor, rtol: float = 1e-10) -> torch.Tensor:
    u, s, vh = torch.linalg.svd(a, full_matrices=True)
    rank = int((s > rtol * s.max()).sum()) if len(s) else 0
    return vh[rank:].t()


def orth(a: torch.Tensor, rtol: float = 1e-10) -> torch.Tensor:
    u, s, _ = torch.linalg.svd(a, full_matrices=False)
    return u[:, s > rtol * s.max()]


def subspace_angles(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    qa, qb = orth(a), orth(b)
    return torch.acos(torch.linalg.svdvals(qa.t() @ qb).clamp(-1, 1))


def procrustes(a: torch.Tensor, b: torch.Tensor) -> tuple[torch.Tensor, float]:
    """Orthogonal ``R`` minimising ``||A R - B||_F``; returns ``(R, residual)``."""
    u, _, vh = torch.linalg.svd(a.t() @ b)
    r = u @ vh
    return r, float(torch.linalg.matrix_norm(a @ r - b))


def matrix_analysis(a: torch.Tensor) -> dict:
    sq = a.shape[0] == a.shape[1]
    s = torch.linalg.svdvals(a)
    sym = sq and bool(torch.allclose(a, a.t(), atol=1e-10 * float(a.abs().max() + 1e-300)))
    eig = torch.linalg.eigvalsh(a) if sym else None
    lower_bw = max((i - j for i, j in (a != 0).nonzero().tolist()), default=0)
    upper_bw = max((j - i for i, j in (a != 0).nonzero().tolist()), default=0)
    return {"shape": tuple(a.shape), "rank": int((s > 1e-10 * s.max()).sum()), "condition": float(s.max() / s.min().clamp(min=1e-300)), "symmetric": sym,
            "positive_definite": bool(sym and eig.min() > 0), "definiteness": ("positive" if eig.min() > 0 else "negative" if eig.max() < 0 else "indefinite") if sym else None,
            "orthogonal": bool(sq and torch.allclose(a.t() @ a, torch.eye(a.shape[0], dtype=a.dtype), atol=1e-8)), "sparsity": float((a == 0).double().mean()),
            "bandwidth": (lower_bw, upper_bw), "diagonally_dominant": bool(sq and (a.diagonal().abs() >= a.abs().sum(1) - a.diagonal().abs()).all()),
            "norms": {"fro": float(torch.linalg.matrix_norm(a)), "1": float(torch.linalg.matrix_norm(a, 1)), "inf": float(torch.linalg.matrix_norm(a, float("inf"))), "2": float(s.max())},
            "nuclear": float(s.sum()), "stable_rank": float((s ** 2).sum() / s.max() ** 2)}
