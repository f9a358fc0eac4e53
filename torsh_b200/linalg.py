"""Linear algebra and special functions (``crates/torsh-linalg``, ``crates/torsh-special``) over ``torch.linalg`` /
``torch.special``: decompositions, solvers, matrix functions, randomized SVD; gamma / Bessel / erf families."""
from __future__ import annotations

import torch

lu, qr, svd, eig, eigh, cholesky = torch.linalg.lu, torch.linalg.qr, torch.linalg.svd, torch.linalg.eig, torch.linalg.eigh, torch.linalg.cholesky
solve, lstsq, inv, pinv, det, slogdet = torch.linalg.solve, torch.linalg.lstsq, torch.linalg.inv, torch.linalg.pinv, torch.linalg.det, torch.linalg.slogdet
norm, matrix_norm, vector_norm, cond, matrix_rank = torch.linalg.norm, torch.linalg.matrix_norm, torch.linalg.vector_norm, torch.linalg.cond, torch.linalg.matrix_rank
matrix_exp, matrix_power = torch.linalg.matrix_exp, torch.linalg.matrix_power
solve_triangular = torch.linalg.solve_triangular


def matrix_sqrt(a: torch.Tensor) -> torch.Tensor:
    """Principal square root of a symmetric positive semi-definite matrix."""
    w, v = torch.linalg.eigh(a)
    return (v * w.clamp(min=0).sqrt()) @ v.mT


def matrix_log(a: torch.Tensor) -> torch.Tensor:
    w, v = torch.linalg.eigh(a)
    return (v * w.log()) @ v.mT


def randomized_svd(a: torch.Tensor, rank: int, oversample: int = 8, power_iters: int = 2, seed: int = 0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(a.shape[1], rank + oversample, generator=g).to(a)
    y = a @ q
    for _ in range(power_iters):
        y = a @ (a.mT @ torch.linalg.qr(y)[0])
    qm = torch.linalg.qr(y)[0]
    u, s, vh = torch.linalg.svd(qm.mT @ a, full_matrices=False)
    return (qm @ u)[:, :rank], s[:rank], vh[:rank]


def conjugate_gradient(a, b, iters: int = 100, tol: float = 1e-8):
    x = torch.zeros_like(b)
    r = b - a @ x
    p, rs = r.clone(), (r * r).sum()
    for _ in range(iters):
        ap = a @ p
        alpha = rs / (p * ap).sum()
        x, r = x + alpha * p, r - alpha * ap
        rs_new = (r * r).sum()
        if rs_new.sqrt() < tol:
            break
        p, rs = r + (rs_new / rs) * p, rs_new
    return x


class special:  # noqa: N801  (namespace mirroring the crate name)
    gamma = staticmethod(lambda x: torch.lgamma(x).exp())
    lgamma, digamma, polygamma = staticmethod(torch.lgamma), staticmethod(torch.digamma), staticmethod(torch.polygamma)
    erf, erfc, erfinv = staticmethod(torch.erf), staticmethod(torch.erfc), staticmethod(torch.erfinv)
    bessel_j0, bessel_j1 = staticmethod(torch.special.bessel_j0), staticmethod(torch.special.bessel_j1)
    bessel_y0, bessel_y1 = staticmethod(torch.special.bessel_y0), staticmethod(torch.special.bessel_y1)
    i0, i0e, i1, i1e = staticmethod(torch.special.i0), staticmethod(torch.special.i0e), staticmethod(torch.special.i1), staticmethod(torch.special.i1e)
    expit, logit, xlogy, zeta = staticmethod(torch.special.expit), staticmethod(torch.special.logit), staticmethod(torch.special.xlogy), staticmethod(torch.special.zeta)
    gammainc, gammaincc = staticmethod(torch.special.gammainc), staticmethod(torch.special.gammaincc)
    sinc, log1p, expm1 = staticmethod(torch.special.sinc), staticmethod(torch.special.log1p), staticmethod(torch.special.expm1)
    beta = staticmethod(lambda a, b: (torch.lgamma(a) + torch.lgamma(b) - torch.lgamma(a + b)).exp())


# ---- matrix equations (crates/torsh-linalg/src/matrix_equations.rs) ------------------------------------------------
def kron(a, b):
    return torch.kron(a, b)


def solve_sylvester(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """X with A X + X B = C, through the eigen-decompositions of A and B (both diagonalisable)."""
    wa, va = torch.linalg.eig(a)
    wb, vb = torch.linalg.eig(b)
    ct = torch.linalg.solve(va, c.to(va.dtype)) @ vb
    x = va @ (ct / (wa[:, None] + wb[None, :])) @ torch.linalg.inv(vb)
    return x.real if not (a.is_complex() or b.is_complex() or c.is_complex()) else x


def solve_lyapunov(a: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """Continuous Lyapunov equation A X + X A^T = Q."""
    return solve_sylvester(a, a.mT, q)


def solve_discrete_lyapunov(a: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """X with A X A^T - X + Q = 0, by the Kronecker linear system (small matrices)."""
    n = a.shape[0]
    lhs = torch.eye(n * n, dtype=a.dtype) - torch.kron(a, a)
    return torch.linalg.solve(lhs, q.reshape(-1)).reshape(n, n)


def solve_continuous_are(a, b, q, r) -> torch.Tensor:
    """Stabilising solution of A^T X + X A - X B R^-1 B^T X + Q = 0 from the stable invariant subspace of the Hamiltonian."""
    n = a.shape[0]
    g = b @ torch.linalg.solve(r, b.mT)
    h = torch.cat([torch.cat([a, -g], 1), torch.cat([-q, -a.mT], 1)], 0)
    w, v = torch.linalg.eig(h)
    stable = v[:, w.real < 0]
    x = stable[n:] @ torch.linalg.inv(stable[:n])
    return x.real


# ---- matrix functions (matrix_functions.rs) --------------------------------------------------------------------------
def funm(a: torch.Tensor, f) -> torch.Tensor:
    """f(A) for a diagonalisable A via its eigen-decomposition (real result for a real input when the imaginary part vanishes)."""
    w, v = torch.linalg.eig(a)
    out = v @ torch.diag_embed(f(w)) @ torch.linalg.inv(v)
    return out.real if not a.is_complex() and out.imag.abs().max() < 1e-6 * (1 + out.real.abs().max()) else out


def sqrtm(a):
    return funm(a, torch.sqrt)


def logm(a):
    return funm(a, torch.log)


def signm(a):
    return funm(a, lambda w: torch.sgn(w.real).to(w.dtype))


def cosm(a):
    return funm(a, torch.cos)


def sinm(a):
    return funm(a, torch.sin)


def polar(a: torch.Tensor):
    """A = U P with U orthogonal / unitary and P symmetric positive semi-definite."""
    u, s, vh = torch.linalg.svd(a, full_matrices=False)
    return u @ vh, (vh.mH * s) @ vh


# ---- special matrices (special_matrices.rs) --------------------------------------------------------------------------
def hilbert(n: int, dtype=torch.float64):
    i = torch.arange(1, n + 1, dtype=dtype)
    return 1.0 / (i[:, None] + i[None, :] - 1)


def toeplitz(c: torch.Tensor, r: torch.Tensor | None = None):
    r = c if r is None else r
    n, m = c.numel(), r.numel()
    idx = torch.arange(n)[:, None] - torch.arange(m)[None, :]
    vals = torch.cat([r.flip(0)[:-1], c])                       # index m - 1 + (i - j)
    return vals[idx + m - 1]


def hankel(c: torch.Tensor, r: torch.Tensor | None = None):
    n = c.numel()
    r = torch.zeros_like(c) if r is None else r
    vals = torch.cat([c, r[1:]])
    return vals[torch.arange(n)[:, None] + torch.arange(r.numel())[None, :]]


def circulant(c: torch.Tensor):
    n = c.numel()
    return c[(torch.arange(n)[:, None] - torch.arange(n)[None, :]) % n]


def vandermonde(x: torch.Tensor, n: int | None = None, increasing: bool = False):
    n = n or x.numel()
    p = torch.arange(n, dtype=x.dtype)
    v = x[:, None] ** p[None, :]
    return v if increasing else v.flip(1)


def companion(coeffs: torch.Tensor):
    """Companion matrix of the monic polynomial x^n + c[n-1] x^(n-1) + ... + c[0] (``coeffs`` = c[0..n-1])."""
    n = coeffs.numel()
    m = torch.zeros(n, n, dtype=coeffs.dtype)
    m[1:, :-1] = torch.eye(n - 1, dtype=coeffs.dtype)
    m[:, -1] = -coeffs
    return m


# ---- iterative solvers (solvers/) ----------------------------------------------------------------------------------
def gmres(a, b, x0=None, restart: int = 30, iters: int = 200, tol: float = 1e-8):
    """Restarted GMRES for a general square system; ``a`` is a matrix or a callable ``v -> A v``."""
    mv = a if callable(a) else (lambda v: a @ v)
    x = torch.zeros_like(b) if x0 is None else x0.clone()
    bn = b.norm().clamp(min=1e-30)
    done = 0
    while done < iters:
        r = b - mv(x)
        beta = r.norm()
        if beta / bn < tol:
            break
        m = min(restart, iters - done)
        Q = torch.zeros(b.numel(), m + 1, dtype=b.dtype)
        H = torch.zeros(m + 1, m, dtype=b.dtype)
        Q[:, 0] = r / beta
        k_used = 0
        for k in range(m):
            w = mv(Q[:, k])
            for j in range(k + 1):                       # modified Gram-Schmidt
                H[j, k] = Q[:, j] @ w
                w = w - H[j, k] * Q[:, j]
            H[k + 1, k] = w.norm()
            k_used = k + 1
            if H[k + 1, k] < 1e-14:
                break
            Q[:, k + 1] = w / H[k + 1, k]
        e1 = torch.zeros(k_used + 1, dtype=b.dtype)
        e1[0] = beta
        y = torch.linalg.lstsq(H[:k_used + 1, :k_used], e1[:, None]).solution[:, 0]
        x = x + Q[:, :k_used] @ y
        done += k_used
    return x


def bicgstab(a, b, x0=None, iters: int = 500, tol: float = 1e-8):
    mv = a if callable(a) else (lambda v: a @ v)
    x = torch.zeros_like(b) if x0 is None else x0.clone()
    r = b - mv(x)
    rhat, rho, alpha, omega = r.clone(), 1.0, 1.0, 1.0
    v, p = torch.zeros_like(b), torch.zeros_like(b)
    bn = b.norm().clamp(min=1e-30)
    for _ in range(iters):
        rho_new = rhat @ r
        beta = (rho_new / rho) * (alpha / omega)
        p = r + beta * (p - omega * v)
        v = mv(p)
        alpha = rho_new / (rhat @ v)
        s = r - alpha * v
        if s.norm() / bn < tol:
            return x + alpha * p
        t = mv(s)
        omega = (t @ s) / (t @ t)
        x = x + alpha * p + omega * s
        r = s - omega * t
        if r.norm() / bn < tol:
            break
        rho = rho_new
    return x


# ---- matrix calculus (matrix_calculus.rs) -----------------------------------------------------------------------------
def jacobian(f, x: torch.Tensor) -> torch.Tensor:
    return torch.autograd.functional.jacobian(f, x)


def hessian(f, x: torch.Tensor) -> torch.Tensor:
    return torch.autograd.functional.hessian(f, x)


def condition_report(a: torch.Tensor) -> dict:
    """Numbers that tell whether solving with A is safe: 2-norm condition number, rank, smallest singular value and the
    forward-error bound ``cond * eps`` (numerical_stability.rs)."""
    s = torch.linalg.svdvals(a)
    eps = torch.finfo(a.dtype).eps
    return {"cond": float(s[0] / s[-1].clamp(min=1e-300)), "rank": int((s > s[0] * max(a.shape) * eps).sum()), "sigma_min": float(s[-1]),
            "forward_error_bound": float(s[0] / s[-1].clamp(min=1e-300) * eps)}
