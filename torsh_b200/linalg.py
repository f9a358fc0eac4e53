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
