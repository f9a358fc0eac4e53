"""Further special functions (``crates/torsh-special/src``): Bessel functions of integer order and spherical Bessel functions
(``bessel.rs``), Struve and Lommel functions (``lommel.rs``), Coulomb wave functions (``coulomb.rs``), Jacobi elliptic
functions (``elliptic.rs``), scaled / imaginary error functions, Dawson and Fresnel integrals, the Faddeeva function and
complex error function (``error_functions.rs``, ``complex/``), sine and cosine integrals (``exponential_integrals.rs``), complex
gamma, Riemann zeta, polylogarithm (``complex/``, ``advanced.rs``), Mathieu characteristic values and functions
(``mathieu.rs``), spheroidal characteristic values (``spheroidal.rs``), Jacobi polynomials, associated Legendre functions
and spherical harmonics (``orthogonal_polynomials.rs``), ``sinc`` / ``cospi`` style helpers (``trigonometric.rs``), constants
(``constants.rs``), tabulated evaluation (``lookup_tables.rs``), memoisation (``smart_caching.rs``), domain handling
(``error_handling.rs``) and accuracy reports (``visualization.rs``, ``numerical_accuracy_tests.rs``).

Everything is written on tensors (float64 internally) and runs on any device."""
from __future__ import annotations

import hashlib
import math
from collections import OrderedDict
from typing import Callable, Sequence

import torch

EULER_GAMMA, CATALAN, APERY, GOLDEN_RATIO, SQRT_PI, SQRT_2PI, LN_2PI = 0.5772156649015329, 0.915965594177219, 1.2020569031595942, 1.618033988749895, 1.7724538509055159, 2.5066282746310002, 1.8378770664093453
GLAISHER, KHINCHIN, TWIN_PRIME, OMEGA = 1.2824271291006226, 2.6854520010653062, 0.6601618158468696, 0.5671432904097838


def _d(x): return torch.as_tensor(x, dtype=torch.float64) if not isinstance(x, torch.Tensor) else x.double()


# ================================================================================================ domain handling
class SpecialFunctionError(ValueError):
    pass


def check_domain(name: str, x: torch.Tensor, lo: float | None = None, hi: float | None = None, mode: str = "nan", open_lo: bool = False, open_hi: bool = False) -> torch.Tensor:
    """Mask of the elements inside ``[lo, hi]``.  ``mode="raise"`` raises with the first offending value; ``"nan"`` leaves it to the
    caller to fill the outside with NaN."""
    ok = torch.ones_like(x, dtype=torch.bool)
    if lo is not None:
        ok &= (x > lo) if open_lo else (x >= lo)
    if hi is not None:
        ok &= (x < hi) if open_hi else (x <= hi)
    if mode == "raise" and not ok.all():
        bad = float(x[~ok].flatten()[0])
        raise SpecialFunctionError(f"{name}: argument {bad} outside the domain {'(' if open_lo else '['}{lo}, {hi}{')' if open_hi else ']'}")
    return ok


# ================================================================================================ Bessel functions
def _miller_j(x: torch.Tensor, nmax: int) -> torch.Tensor:
    """``J_0 .. J_nmax`` by backward recurrence normalised with ``J_0 + 2 sum J_{2k} = 1`` (no division by a value that can
    vanish).  Returns a tensor ``[nmax + 1, *x.shape]``."""
    x = x.clamp_min(1e-300)
    top = max(nmax, int(2 * float(x.max()))) + 60
    top += top % 2
    F = torch.zeros(top + 2, *x.shape, dtype=torch.float64, device=x.device)
    F[top] = 1e-250
    for k in range(top, 0, -1):
        F[k - 1] = 2 * k / x * F[k] - F[k + 1]
        big = F[k - 1].abs() > 1e200
        if big.any():
            F[k - 1:] = torch.where(big, F[k - 1:] * 1e-200, F[k - 1:])
    norm = F[0] + 2 * F[2:top + 1:2].sum(0)
    return F[:nmax + 1] / norm


def _hankel(nu: int, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``J_nu, Y_nu`` from Hankel's asymptotic expansion (for ``x >= 25`` the truncation error is below rounding)."""
    mu, term, P, Q = 4.0 * nu * nu, torch.ones_like(x), torch.ones_like(x), torch.zeros_like(x)
    for k in range(1, 26):
        term = term * (mu - (2 * k - 1) ** 2) / (k * 8 * x)
        if k % 2:
            Q = Q + (1 if k % 4 == 1 else -1) * term
        else:
            P = P + (1 if k % 4 == 0 else -1) * term
    chi = x - (nu / 2 + 0.25) * math.pi
    amp = torch.sqrt(2 / (math.pi * x))
    return amp * (P * torch.cos(chi) - Q * torch.sin(chi)), amp * (P * torch.sin(chi) + Q * torch.cos(chi))


def bessel_jy01(x) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``J_0, J_1, Y_0, Y_1`` for ``x > 0`` to double precision: Miller recurrence with Neumann series for ``Y`` up to 25, Hankel
    asymptotics beyond."""
    x = _d(x)
    big = x > 25
    xs = torch.where(big, torch.ones_like(x), x).clamp_min(1e-300)
    K = 60
    J = _miller_j(xs, 2 * K + 1)
    lg = torch.log(xs / 2) + EULER_GAMMA
    k = torch.arange(1, K + 1, dtype=torch.float64, device=x.device).reshape(-1, *[1] * x.dim())
    sgn = torch.where(k % 2 == 1, 1.0, -1.0)
    y0 = 2 / math.pi * lg * J[0] + 4 / math.pi * (sgn * J[2:2 * K + 1:2] / k).sum(0)
    dy0 = 2 / math.pi * (J[0] / xs - lg * J[1]) + 4 / math.pi * (sgn * (J[1:2 * K:2] - J[3:2 * K + 2:2]) / (2 * k)).sum(0)
    xb = torch.where(big, x, torch.full_like(x, 30.0))
    j0b, y0b = _hankel(0, xb)
    j1b, y1b = _hankel(1, xb)
    return torch.where(big, j0b, J[0]), torch.where(big, j1b, J[1]), torch.where(big, y0b, y0), torch.where(big, y1b, -dy0)


def _miller_i(n: int, x: torch.Tensor) -> torch.Tensor:
    """``I_n`` by backward recurrence normalised with the exact ``I_0`` (which never vanishes)."""
    x = x.clamp_min(1e-300)
    start = n + int(math.sqrt(60 * (n + 1))) + 2 * int(float(x.abs().max())) + 20
    fp, f, want = torch.zeros_like(x), torch.full_like(x, 1e-280), None
    for k in range(start, 0, -1):
        fp, f = f, 2 * k / x * f + fp
        big = f.abs() > 1e200
        if big.any():
            f, fp = torch.where(big, f * 1e-200, f), torch.where(big, fp * 1e-200, fp)
            if want is not None:
                want = torch.where(big, want * 1e-200, want)
        if k - 1 == n:
            want = f.clone()
    return want * torch.special.modified_bessel_i0(x) / f


def bessel_j(n: int, x) -> torch.Tensor:
    x = _d(x)
    if n < 0:
        return (-1) ** n * bessel_j(-n, x)
    ax = x.abs()
    j0, j1, _, _ = bessel_jy01(ax.clamp_min(1e-300))
    if n == 0:
        out = j0
    elif n == 1:
        out = j1
    else:
        fwd = ax > max(n, 25)                                                         # forward recurrence is stable while the order stays below the argument
        jm, j = j0, j1
        for k in range(1, n):
            jm, j = j, 2 * k / ax.clamp_min(1e-300) * j - jm
        back = _miller_j(torch.where(fwd, torch.ones_like(ax), ax), n)[n] if not fwd.all() else j
        out = torch.where(fwd, j, back)
    out = torch.where(ax == 0, torch.full_like(out, 1.0 if n == 0 else 0.0), out)
    return torch.where(x < 0, (-1) ** n * out, out)


def bessel_y(n: int, x) -> torch.Tensor:
    x = _d(x)
    if n < 0:
        return (-1) ** n * bessel_y(-n, x)
    _, _, ym, y = bessel_jy01(x)
    if n == 0:
        return ym
    for k in range(1, n):
        ym, y = y, 2 * k / x * y - ym
    return y


def bessel_i(n: int, x) -> torch.Tensor:
    x = _d(x); n = abs(n)
    if n == 0:
        return torch.special.modified_bessel_i0(x)
    if n == 1:
        return torch.special.modified_bessel_i1(x)
    out = _miller_i(n, x.abs())
    out = torch.where(x == 0, torch.zeros_like(out), out)
    return torch.where(x < 0, (-1) ** n * out, out)


def bessel_k(n: int, x) -> torch.Tensor:
    x = _d(x); n = abs(n)
    km, k = torch.special.modified_bessel_k0(x), torch.special.modified_bessel_k1(x)
    if n == 0:
        return km
    for j in range(1, n):
        km, k = k, 2 * j / x * k + km
    return k


def spherical_jn(n: int, x) -> torch.Tensor:
    x = _d(x)
    small = x.abs() < 1e-3 * (n + 1)
    xs = torch.where(small, torch.ones_like(x), x)
    # j_n = sqrt(pi / 2x) J_{n + 1/2}: upward recurrence where stable, series near the origin, Miller in between
    j0, j1 = torch.sin(xs) / xs, torch.sin(xs) / xs ** 2 - torch.cos(xs) / xs
    if n == 0:
        res = j0
    elif n == 1:
        res = j1
    else:
        up_m, up = j0, j1
        for k in range(1, n):
            up_m, up = up, (2 * k + 1) / xs * up - up_m
        start = n + int(math.sqrt(40 * (n + 1))) + int(float(xs.abs().max())) + 10
        fp, f, want = torch.zeros_like(xs), torch.full_like(xs, 1e-250), None
        for k in range(start, 0, -1):
            fm = (2 * k + 1) / xs * f - fp
            fp, f = f, fm
            big = f.abs() > 1e200
            f, fp = torch.where(big, f * 1e-200, f), torch.where(big, fp * 1e-200, fp)
            want = torch.where(big, want * 1e-200, want) if want is not None else None
            if k - 1 == n:
                want = f.clone()
        res = torch.where(xs.abs() > n + 1, up, want * j0 / f)
    dfact = math.prod(range(1, 2 * n + 2, 2))
    series = x ** n / dfact * (1 - x * x / (2 * (2 * n + 3)))
    return torch.where(small, series, res)


def spherical_yn(n: int, x) -> torch.Tensor:
    x = _d(x)
    ym, y = -torch.cos(x) / x, -torch.cos(x) / x ** 2 - torch.sin(x) / x
    if n == 0:
        return ym
    for k in range(1, n):
        ym, y = y, (2 * k + 1) / x * y - ym
    return y


# ================================================================================================ Struve, Lommel, Coulomb
def struve_h(nu: float, x, terms: int = 80) -> torch.Tensor:
    """Power series ``H_nu(x) = sum (-1)^k (x/2)^{2k+nu+1} / (Gamma(k+3/2) Gamma(k+nu+3/2))`` (accurate for ``|x|`` up to about 20 in
    float64)."""
    x = _d(x)
    k = torch.arange(terms, dtype=torch.float64, device=x.device)
    logc = -(torch.lgamma(k + 1.5) + torch.lgamma(k + nu + 1.5))
    h = (x / 2).unsqueeze(-1)
    t = torch.exp(logc + (2 * k + nu + 1) * torch.log(h.abs().clamp_min(1e-300))) * (1 - 2 * (k % 2))
    return t.sum(-1) * torch.where((x < 0) & (round(nu) % 2 == 0) if float(nu).is_integer() else torch.zeros_like(x, dtype=torch.bool), -torch.ones_like(x), torch.ones_like(x))


def lommel_s1(mu: float, nu: float, x, terms: int = 80) -> torch.Tensor:
    """``s_{mu,nu}(z) = z^{mu+1} sum_k (-1)^k z^{2k} / prod_{j<=k} ((mu + 2j + 1)^2 - nu^2)``: the particular solution of
    ``z^2 y'' + z y' + (z^2 - nu^2) y = z^{mu+1}``."""
    x = _d(x)
    term = x ** (mu + 1) / ((mu + 1) ** 2 - nu ** 2)
    total = term.clone()
    for k in range(1, terms):
        term = -term * x * x / ((mu + 2 * k + 1) ** 2 - nu ** 2)
        total = total + term
    return total


def coulomb_f(l: int, eta: float, rho, terms: int = 200) -> torch.Tensor:
    """Regular Coulomb wave function by its power series ``F_L = C_L(eta) rho^{L+1} sum A_k rho^{k-L-1}`` with
    ``(k + L)(k - L - 1) A_k = 2 eta A_{k-1} - A_{k-2}`` (for moderate ``rho``; float64)."""
    rho = _d(rho)
    lg = lambda z: _cgamma_log(torch.tensor(complex(z)))
    c = 2 ** l * math.exp(-math.pi * eta / 2) * abs(complex(torch.exp(lg(complex(l + 1, eta))))) / math.gamma(2 * l + 2)
    a_prev2, a_prev = 0.0, 1.0                                                        # A_{L+1} = 1, A_{L+2} = eta / (L + 1)
    total = torch.ones_like(rho)
    power = torch.ones_like(rho)
    for k in range(l + 2, l + 2 + terms):
        a = (2 * eta * a_prev - a_prev2) / ((k + l) * (k - l - 1))
        power = power * rho
        total = total + a * power
        a_prev2, a_prev = a_prev, a
    return c * rho ** (l + 1) * total


# ================================================================================================ Jacobi elliptic functions
def ellipj(u, m) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """``sn, cn, dn`` and the amplitude by the arithmetic-geometric mean (descending Landen) for ``0 <= m <= 1``."""
    u, m = torch.broadcast_tensors(_d(u), _d(m))
    a, b = [torch.ones_like(m)], torch.sqrt(1 - m)
    c = [torch.sqrt(m)]
    for _ in range(12):
        a.append((a[-1] + b) / 2); c.append((a[-2] - b) / 2); b = torch.sqrt(a[-2] * b)
    phi = 2 ** 12 * a[-1] * u
    for n in range(12, 0, -1):
        phi = (phi + torch.asin((c[n] / a[n]).clamp(-1, 1) * torch.sin(phi))) / 2
    sn, cn = torch.sin(phi), torch.cos(phi)
    dn = torch.sqrt(1 - m * sn * sn)
    one = m >= 1 - 1e-15                                                              # m = 1: hyperbolic limit
    sn, cn, dn = torch.where(one, torch.tanh(u), sn), torch.where(one, 1 / torch.cosh(u), cn), torch.where(one, 1 / torch.cosh(u), dn)
    return sn, cn, dn, torch.where(one, 2 * torch.atan(torch.exp(u)) - math.pi / 2, phi)


# ================================================================================================ error-function family
_W_N = 40
def _weideman_coeffs():
    n, m = _W_N, 2 * _W_N
    L = math.sqrt(n / math.sqrt(2))
    k = torch.arange(-m + 1, m, dtype=torch.float64)
    t = L * torch.tan(k * math.pi / m / 2)
    f = torch.cat([torch.zeros(1, dtype=torch.float64), torch.exp(-t * t) * (L * L + t * t)])
    a = torch.fft.fft(torch.fft.fftshift(f)).real / (2 * m)
    return L, a[1:n + 1].flip(0)
_W_L, _W_A = _weideman_coeffs()


def wofz(z) -> torch.Tensor:
    """Faddeeva function ``w(z) = exp(-z^2) erfc(-i z)`` (Weideman's rational approximation in the upper half plane, the
    reflection ``w(z) = 2 exp(-z^2) - w(-z)`` below)."""
    z = torch.as_tensor(z).to(torch.complex128)
    lower = z.imag < 0
    zz = torch.where(lower, -z, z)
    den = _W_L - 1j * zz
    Z = (_W_L + 1j * zz) / den
    p = torch.zeros_like(Z)
    for c in _W_A.to(z.device):
        p = p * Z + c
    w = 2 * p / den ** 2 + (1 / SQRT_PI) / den
    return torch.where(lower, 2 * torch.exp(-z * z) - w, w)


def erf_complex(z) -> torch.Tensor:
    z = torch.as_tensor(z).to(torch.complex128)
    neg = z.real < 0
    zz = torch.where(neg, -z, z)
    r = 1 - torch.exp(-zz * zz) * wofz(1j * zz)
    return torch.where(neg, -r, r)


def erfcx(x) -> torch.Tensor:
    """Scaled complementary error function ``exp(x^2) erfc(x)`` without overflow."""
    x = _d(x)
    return torch.where(x < 25, wofz(1j * x.to(torch.complex128)).real, 1 / (SQRT_PI * x) * (1 - 0.5 / x ** 2 + 0.75 / x ** 4 - 1.875 / x ** 6 + 6.5625 / x ** 8))


def erfi(x) -> torch.Tensor: x = _d(x); return (-1j * erf_complex(1j * x.to(torch.complex128))).real
def dawsn(x) -> torch.Tensor: x = _d(x); return SQRT_PI / 2 * wofz(x.to(torch.complex128)).imag
def voigt_profile(x, sigma: float, gamma: float) -> torch.Tensor: x = _d(x); return wofz((x + 1j * gamma) / (sigma * math.sqrt(2))).real / (sigma * SQRT_2PI)


def fresnel(x) -> tuple[torch.Tensor, torch.Tensor]:
    """``S(x) = int_0^x sin(pi t^2 / 2) dt`` and ``C(x)`` through the complex error function."""
    x = _d(x)
    e = erf_complex(SQRT_PI / 2 * (1 - 1j) * x.to(torch.complex128)) * (1 + 1j) / 2
    return e.imag, e.real


# ================================================================================================ sine / cosine integrals
_GL_X, _GL_W = None, None
def _gauss_legendre(n=256):
    global _GL_X, _GL_W
    if _GL_X is None:
        import numpy as np
        x, w = np.polynomial.legendre.leggauss(n)
        _GL_X, _GL_W = torch.tensor(x), torch.tensor(w)
    return _GL_X, _GL_W


def sici(x) -> tuple[torch.Tensor, torch.Tensor]:
    """``Si(x) = int_0^x sin t / t dt`` and ``Ci(x) = gamma + ln x + int_0^x (cos t - 1) / t dt`` by Gauss-Legendre quadrature on
    ``[0, x]`` (256 nodes: exact to rounding for ``|x|`` up to about 150)."""
    x = _d(x)
    gx, gw = _gauss_legendre()
    t = (x.unsqueeze(-1) / 2) * (gx.to(x.device) + 1)
    ts = torch.where(t == 0, torch.ones_like(t), t)
    si = ((torch.sin(ts) / ts) * gw.to(x.device)).sum(-1) * x / 2
    cin = (((torch.cos(ts) - 1) / ts) * gw.to(x.device)).sum(-1) * x / 2
    return si, EULER_GAMMA + torch.log(x.abs()) + cin


# ================================================================================================ complex gamma, zeta, polylogarithm
_LANCZOS = (0.99999999999980993, 676.5203681218851, -1259.1392167224028, 771.32342877765313, -176.61502916214059, 12.507343278686905, -0.13857109526572012, 9.9843695780195716e-6, 1.5056327351493116e-7)


def _cgamma_log(z: torch.Tensor) -> torch.Tensor:
    z = z.to(torch.complex128)
    refl = z.real < 0.5
    zz = torch.where(refl, 1 - z, z) - 1
    s = torch.full_like(zz, _LANCZOS[0])
    for i, c in enumerate(_LANCZOS[1:], 1):
        s = s + c / (zz + i)
    t = zz + 7.5
    lg = 0.5 * LN_2PI + (zz + 0.5) * torch.log(t) - t + torch.log(s)
    return torch.where(refl, math.log(math.pi) - torch.log(torch.sin(math.pi * z)) - lg, lg)


def loggamma_complex(z) -> torch.Tensor: return _cgamma_log(torch.as_tensor(z))
def gamma_complex(z) -> torch.Tensor: return torch.exp(_cgamma_log(torch.as_tensor(z)))


def zeta(s) -> torch.Tensor:
    """Riemann zeta for real ``s != 1``: Hurwitz series on the right, the functional equation on the left."""
    s = _d(s)
    right = s > 1
    sr = torch.where(right, s, 1 - s).clamp_min(1.0 + 1e-12)
    zr = torch.special.zeta(sr, torch.ones_like(sr))
    left = 2 ** s * math.pi ** (s - 1) * torch.sin(math.pi * s / 2) * torch.exp(torch.lgamma(1 - s)) * zr
    mid = (s > 0) & (s < 1)                                                           # Dirichlet eta series with Euler acceleration in the critical strip
    n = 60
    k = torch.arange(1, n + 1, dtype=torch.float64, device=s.device)
    binom = torch.tensor([math.comb(n, j) for j in range(n + 1)], dtype=torch.float64, device=s.device).cumsum(0)
    e = torch.cat([torch.full((n,), 2.0 ** n, dtype=torch.float64, device=s.device), 2.0 ** n - binom[:n]])
    kk = torch.arange(1, 2 * n + 1, dtype=torch.float64, device=s.device)
    sm = torch.where(mid, s, torch.full_like(s, 0.5))
    eta = ((-1) ** (kk - 1) * e / kk ** sm.unsqueeze(-1)).sum(-1) / 2.0 ** n
    zm = eta / (1 - 2 ** (1 - sm))
    out = torch.where(right, zr, torch.where(mid, zm, left))
    return torch.where(s == 0, torch.full_like(out, -0.5), out)


def polylog(s: float, z, terms: int = 500) -> torch.Tensor:
    """``Li_s(z) = sum z^k / k^s`` for ``|z| <= 1`` (``|z| < 1`` unless ``s > 1``); for ``-inf < z < -1`` not covered."""
    z = _d(z)
    k = torch.arange(1, terms + 1, dtype=torch.float64, device=z.device)
    return (z.unsqueeze(-1) ** k / k ** s).sum(-1)


# ================================================================================================ Mathieu and spheroidal characteristic values
def _mathieu_matrix(q: float, kind: str, n: int = 60) -> torch.Tensor:
    """Tridiagonal recurrence matrices of the four periodic classes: ``a_even`` (ce_{2r}), ``a_odd`` (ce_{2r+1}), ``b_even``
    (se_{2r+2}), ``b_odd`` (se_{2r+1})."""
    A = torch.zeros(n, n, dtype=torch.float64)
    if kind == "a_even":
        d = torch.arange(n, dtype=torch.float64) * 2
        A += torch.diag(d ** 2) + q * (torch.diag(torch.ones(n - 1), 1) + torch.diag(torch.ones(n - 1), -1))
        A[0, 1] = A[1, 0] = math.sqrt(2) * q
    elif kind in ("a_odd", "b_odd"):
        d = torch.arange(n, dtype=torch.float64) * 2 + 1
        A += torch.diag(d ** 2) + q * (torch.diag(torch.ones(n - 1), 1) + torch.diag(torch.ones(n - 1), -1))
        A[0, 0] += q if kind == "a_odd" else -q
    else:
        d = torch.arange(1, n + 1, dtype=torch.float64) * 2
        A += torch.diag(d ** 2) + q * (torch.diag(torch.ones(n - 1), 1) + torch.diag(torch.ones(n - 1), -1))
    return A


def mathieu_a(m: int, q: float) -> float:
    """Characteristic value of the even Mathieu function ``ce_m``."""
    return float(torch.linalg.eigvalsh(_mathieu_matrix(q, "a_even" if m % 2 == 0 else "a_odd"))[m // 2])


def mathieu_b(m: int, q: float) -> float:
    """Characteristic value of the odd Mathieu function ``se_m`` (``m >= 1``)."""
    return float(torch.linalg.eigvalsh(_mathieu_matrix(q, "b_even" if m % 2 == 0 else "b_odd"))[(m - 1) // 2])


def mathieu_cem(m: int, q: float, x) -> torch.Tensor:
    """Even Mathieu function ``ce_m(x, q)`` (``x`` in radians) normalised to ``int_0^{2 pi} ce^2 = pi``."""
    x = _d(x)
    kind = "a_even" if m % 2 == 0 else "a_odd"
    _, vec = torch.linalg.eigh(_mathieu_matrix(q, kind))
    v = vec[:, m // 2].clone()
    n = len(v)
    if kind == "a_even":
        v[0] /= math.sqrt(2)                                                          # undo the symmetrising scale of the constant term
        v = v / math.sqrt(2 * v[0] ** 2 + (v[1:] ** 2).sum())
        orders = torch.arange(n, dtype=torch.float64) * 2
    else:
        v = v / v.norm()
        orders = torch.arange(n, dtype=torch.float64) * 2 + 1
    val = (v * torch.cos(orders * x.unsqueeze(-1))).sum(-1)
    sign = torch.sign((v * 1.0).sum()) if q >= 0 else 1.0                             # convention: ce_m(0, q) > 0
    return val * sign


def spheroidal_cv(m: int, n: int, c: float, oblate: bool = False, size: int = 60) -> float:
    """Characteristic value ``lambda_{mn}(c)`` of the prolate (or oblate) angular spheroidal wave function from the tridiagonal
    recurrence of its Legendre expansion."""
    c2 = -c * c if oblate else c * c
    r0 = (n - m) % 2
    r = torch.arange(size, dtype=torch.float64) * 2 + r0
    beta = (m + r) * (m + r + 1) + (2 * (m + r) * (m + r + 1) - 2 * m * m - 1) * c2 / ((2 * m + 2 * r - 1) * (2 * m + 2 * r + 3))
    alpha = (2 * m + r + 2) * (2 * m + r + 1) * c2 / ((2 * m + 2 * r + 3) * (2 * m + 2 * r + 5))
    r2 = r + 2
    gamma = r2 * (r2 - 1) * c2 / ((2 * m + 2 * r2 - 3) * (2 * m + 2 * r2 - 1))
    off = torch.sqrt((alpha[:-1] * gamma[:-1]).clamp_min(0))                          # similar symmetric matrix: same spectrum
    A = torch.diag(beta) + torch.diag(off, 1) + torch.diag(off, -1)
    return float(torch.linalg.eigvalsh(A)[(n - m) // 2])


# ================================================================================================ polynomials and harmonics
def jacobi(n: int, alpha: float, beta: float, x) -> torch.Tensor:
    x = _d(x)
    p0, p1 = torch.ones_like(x), (alpha + 1) + (alpha + beta + 2) * (x - 1) / 2
    if n == 0:
        return p0
    for k in range(2, n + 1):
        a = 2 * k * (k + alpha + beta) * (2 * k + alpha + beta - 2)
        b = (2 * k + alpha + beta - 1) * ((2 * k + alpha + beta) * (2 * k + alpha + beta - 2) * x + alpha ** 2 - beta ** 2)
        c = 2 * (k + alpha - 1) * (k + beta - 1) * (2 * k + alpha + beta)
        p0, p1 = p1, (b * p1 - c * p0) / a
    return p1


def assoc_legendre(m: int, l: int, x) -> torch.Tensor:
    """``P_l^m(x)`` with the Condon-Shortley phase, ``0 <= m <= l``."""
    x = _d(x)
    pmm = (-1) ** m * math.prod(range(1, 2 * m, 2)) * (1 - x * x).clamp_min(0) ** (m / 2)
    if l == m:
        return pmm
    pm1 = x * (2 * m + 1) * pmm
    for k in range(m + 2, l + 1):
        pmm, pm1 = pm1, ((2 * k - 1) * x * pm1 - (k + m - 1) * pmm) / (k - m)
    return pm1


def sph_harm(m: int, l: int, azimuth, polar) -> torch.Tensor:
    """``Y_l^m`` at azimuth ``theta`` in ``[0, 2 pi)`` and polar angle ``phi`` in ``[0, pi]`` (the argument order of SciPy's ``sph_harm``)."""
    azimuth, polar = _d(azimuth), _d(polar)
    am = abs(m)
    norm = math.sqrt((2 * l + 1) / (4 * math.pi) * math.factorial(l - am) / math.factorial(l + am))
    y = norm * assoc_legendre(am, l, torch.cos(polar)) * torch.exp(1j * am * azimuth.to(torch.complex128))
    return (-1) ** am * y.conj() if m < 0 else y


def sinpi(x): x = _d(x); r = torch.remainder(x, 2.0); return torch.where(r == 1.0, torch.zeros_like(x), torch.sin(math.pi * torch.where(r > 1, r - 2, r))) * torch.where(torch.remainder(x, 1.0) == 0, torch.zeros_like(x), torch.ones_like(x))
def cospi(x): x = _d(x); r = torch.remainder(x, 2.0); return torch.where(torch.remainder(x, 1.0) == 0.5, torch.zeros_like(x), torch.cos(math.pi * r))
def sinc_pi(x): x = _d(x); return torch.where(x == 0, torch.ones_like(x), sinpi(x) / (math.pi * torch.where(x == 0, torch.ones_like(x), x)))
def versine(x): x = _d(x); return 2 * torch.sin(x / 2) ** 2
def haversine(x): return versine(x) / 2
def gudermannian(x): x = _d(x); return 2 * torch.atan(torch.tanh(x / 2))


# ================================================================================================ tables, caching, accuracy
class TabulatedFunction:
    """A function sampled once on a uniform grid and evaluated by cubic (Catmull-Rom) interpolation; outside the range the
    exact function is called."""

    def __init__(self, fn: Callable, lo: float, hi: float, points: int = 4096):
        self.fn, self.lo, self.hi, self.h = fn, lo, hi, (hi - lo) / (points - 1)
        self.table = fn(torch.linspace(lo - self.h, hi + self.h, points + 2, dtype=torch.float64))

    def __call__(self, x):
        x = _d(x)
        inside = (x >= self.lo) & (x <= self.hi)
        p = ((x.clamp(self.lo, self.hi) - self.lo) / self.h)
        i = p.floor().long().clamp(0, len(self.table) - 4)
        t = p - i
        tb = self.table.to(x.device)
        y0, y1, y2, y3 = tb[i], tb[i + 1], tb[i + 2], tb[i + 3]
        y = y1 + 0.5 * t * (y2 - y0 + t * (2 * y0 - 5 * y1 + 4 * y2 - y3 + t * (3 * (y1 - y2) + y3 - y0)))
        return torch.where(inside, y, self.fn(x)) if not inside.all() else y


class SmartCache:
    """Memoises expensive evaluations keyed by the function name, extra arguments and a digest of the tensor; least recently
    used entries leave first; hit statistics are kept."""

    def __init__(self, capacity: int = 64): self.capacity, self.store, self.hits, self.misses = capacity, OrderedDict(), 0, 0

    def __call__(self, fn: Callable, x: torch.Tensor, *args):
        key = (fn.__name__, args, tuple(x.shape), str(x.dtype), hashlib.blake2b(x.detach().cpu().contiguous().numpy().tobytes(), digest_size=16).hexdigest())
        if key in self.store:
            self.hits += 1; self.store.move_to_end(key)
            return self.store[key]
        self.misses += 1
        out = fn(*args, x) if args else fn(x)
        self.store[key] = out
        if len(self.store) > self.capacity:
            self.store.popitem(last=False)
        return out

    def hit_rate(self): return self.hits / max(self.hits + self.misses, 1)


def accuracy_report(fn: Callable, reference: Callable, lo: float, hi: float, points: int = 2001, bins: int = 10) -> dict:
    """Error of ``fn`` against a float64 reference over ``[lo, hi]``: worst absolute and relative errors with their locations, the
    error in units in the last place, and a per-interval profile with a text bar chart."""
    x = torch.linspace(lo, hi, points, dtype=torch.float64)
    y, r = _d(fn(x)), _d(reference(x))
    err = (y - r).abs()
    rel = err / r.abs().clamp_min(1e-300)
    ulp = err / (torch.finfo(torch.float64).eps * r.abs().clamp_min(1e-300))
    edges = torch.linspace(lo, hi, bins + 1)
    prof = [float(rel[(x >= edges[i]) & (x <= edges[i + 1])].max()) for i in range(bins)]
    top = max(max(prof), 1e-300)
    chart = "\n".join(f"[{float(edges[i]):>8.3g}, {float(edges[i + 1]):>8.3g}] {'#' * max(1, int(30 * (math.log10(max(p, 1e-17)) + 17) / (math.log10(top) + 17)))} {p:.2e}" for i, p in enumerate(prof))
    return {"max_abs": float(err.max()), "argmax_abs": float(x[err.argmax()]), "max_rel": float(rel.max()), "argmax_rel": float(x[rel.argmax()]), "median_ulp": float(ulp.median()), "max_ulp": float(ulp.max()), "profile": prof, "chart": chart}
