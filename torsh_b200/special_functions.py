"""Special functions beyond ``torch.special``, element-wise on tensors (float64 internally): complete and incomplete elliptic
integrals, Lambert W, exponential integrals, orthogonal polynomials by their recurrences, hypergeometric series, Airy
functions, the regularised incomplete beta function and the distribution functions built on it, and a few fast
approximations. Reference: crates/torsh-special/src/{elliptic,lambert_w,exponential_integrals,orthogonal_polynomials,
hypergeometric,airy,statistical,fast_approximations}.rs.
"""
from __future__ import annotations

import math

import torch

_EULER = 0.5772156649015329


def _f64(x):
    return torch.as_tensor(x, dtype=torch.float64)


# ---- elliptic integrals ------------------------------------------------------------------------------------------------
def ellipk(m):
    """Complete elliptic integral of the first kind K(m) (parameter m = k^2) by the arithmetic-geometric mean."""
    m = _f64(m)
    a, b = torch.ones_like(m), torch.sqrt(1 - m)
    for _ in range(40):
        a, b = 0.5 * (a + b), torch.sqrt(a * b)
    return math.pi / (2 * a)


def ellipe(m):
    """Complete elliptic integral of the second kind E(m) by the AGM with the c_n^2 sum."""
    m = _f64(m)
    a, b = torch.ones_like(m), torch.sqrt(1 - m)
    c2sum, pw = 0.5 * m, 0.5
    for _ in range(40):
        c = 0.5 * (a - b)
        a, b = 0.5 * (a + b), torch.sqrt(a * b)
        pw *= 2
        c2sum = c2sum + pw * c * c
    return math.pi / (2 * a) * (1 - c2sum)


def _rf(x, y, z):
    """Carlson's symmetric integral R_F by the duplication theorem."""
    for _ in range(60):
        lam = torch.sqrt(x * y) + torch.sqrt(y * z) + torch.sqrt(z * x)
        x, y, z = (x + lam) / 4, (y + lam) / 4, (z + lam) / 4
    return 1 / torch.sqrt((x + y + z) / 3)


def _rd(x, y, z):
    s, fac = torch.zeros_like(x), torch.ones_like(x)
    for _ in range(60):
        lam = torch.sqrt(x * y) + torch.sqrt(y * z) + torch.sqrt(z * x)
        s = s + fac / (torch.sqrt(z) * (z + lam))
        fac = fac / 4
        x, y, z = (x + lam) / 4, (y + lam) / 4, (z + lam) / 4
    mean = (x + y + 3 * z) / 5
    return 3 * s + fac / (mean * torch.sqrt(mean))


def ellipkinc(phi, m):
    """Incomplete elliptic integral of the first kind F(phi | m), |phi| <= pi / 2."""
    phi, m = _f64(phi), _f64(m)
    s, c = torch.sin(phi), torch.cos(phi)
    return s * _rf(c * c, 1 - m * s * s, torch.ones_like(s))


def ellipeinc(phi, m):
    phi, m = _f64(phi), _f64(m)
    s, c = torch.sin(phi), torch.cos(phi)
    one = torch.ones_like(s)
    return s * _rf(c * c, 1 - m * s * s, one) - m / 3 * s ** 3 * _rd(c * c, 1 - m * s * s, one)


# ---- Lambert W ---------------------------------------------------------------------------------------------------------
def lambertw(x, branch: int = 0):
    """Real branches W0 (x >= -1/e) and W-1 (-1/e <= x < 0) by Halley iteration."""
    x = _f64(x)
    if branch == 0:
        w = torch.where(x < 1, 0.6 * x.clamp(min=-0.36), torch.log(x.clamp(min=1e-300)) - torch.log(torch.log(x.clamp(min=1.5)) + 1e-300))
        w = torch.where(x < -0.25, -1 + torch.sqrt((2 * (math.e * x + 1)).clamp(min=0)), w)
    else:
        lx = torch.log((-x).clamp(min=1e-300))
        w = lx - torch.log(-lx)
        w = torch.where(x < -0.25, -1 - torch.sqrt((2 * (math.e * x + 1)).clamp(min=0)), w)
    for _ in range(50):
        ew = torch.exp(w)
        f = w * ew - x
        denom = ew * (w + 1) - (w + 2) * f / (2 * w + 2 + 1e-300)
        w = w - f / torch.where(denom.abs() < 1e-300, torch.full_like(denom, 1e-300), denom)
    bad = (x < -1 / math.e) | ((branch != 0) & (x >= 0))
    return torch.where(bad, torch.full_like(w, float("nan")), w)


# ---- exponential integrals ---------------------------------------------------------------------------------------------
def exp1(x):
    """E1(x) for x > 0: power series below 1, modified Lentz continued fraction above."""
    x = _f64(x)
    xs = x.clamp(max=1.0)
    series, term = -_EULER - torch.log(xs), torch.ones_like(xs)
    for k in range(1, 60):
        term = term * (-xs) / k
        series = series - term / k
    xl = x.clamp(min=1.0)
    b = xl + 1
    c, d = torch.full_like(xl, 1e300), 1 / b
    h = d
    for i in range(1, 200):
        an = -i * i
        b = b + 2
        d = 1 / (an * d + b)
        c = b + an / c
        h = h * c * d
    return torch.where(x <= 1, series, h * torch.exp(-xl))


def expi(x):
    """Ei(x) for x > 0 (series)."""
    x = _f64(x)
    s, term = _EULER + torch.log(x), torch.ones_like(x)
    for k in range(1, 200):
        term = term * x / k
        s = s + term / k
    return s


def expn(n: int, x):
    """E_n(x) for integer n >= 1 by the upward recurrence from E1."""
    x = _f64(x)
    e = exp1(x)
    for k in range(1, n):
        e = (torch.exp(-x) - x * e) / k
    return e


# ---- orthogonal polynomials ----------------------------------------------------------------------------------------------
def legendre(n: int, x):
    x = _f64(x)
    p0, p1 = torch.ones_like(x), x
    if n == 0:
        return p0
    for k in range(1, n):
        p0, p1 = p1, ((2 * k + 1) * x * p1 - k * p0) / (k + 1)
    return p1


def chebyshev_t(n: int, x):
    x = _f64(x)
    t0, t1 = torch.ones_like(x), x
    if n == 0:
        return t0
    for _ in range(1, n):
        t0, t1 = t1, 2 * x * t1 - t0
    return t1


def chebyshev_u(n: int, x):
    x = _f64(x)
    u0, u1 = torch.ones_like(x), 2 * x
    if n == 0:
        return u0
    for _ in range(1, n):
        u0, u1 = u1, 2 * x * u1 - u0
    return u1


def hermite(n: int, x):
    """Physicists' Hermite polynomial H_n."""
    x = _f64(x)
    h0, h1 = torch.ones_like(x), 2 * x
    if n == 0:
        return h0
    for k in range(1, n):
        h0, h1 = h1, 2 * x * h1 - 2 * k * h0
    return h1


def laguerre(n: int, x, alpha: float = 0.0):
    x = _f64(x)
    l0, l1 = torch.ones_like(x), 1 + alpha - x
    if n == 0:
        return l0
    for k in range(1, n):
        l0, l1 = l1, ((2 * k + 1 + alpha - x) * l1 - (k + alpha) * l0) / (k + 1)
    return l1


def gegenbauer(n: int, alpha: float, x):
    x = _f64(x)
    c0, c1 = torch.ones_like(x), 2 * alpha * x
    if n == 0:
        return c0
    for k in range(1, n):
        c0, c1 = c1, (2 * (k + alpha) * x * c1 - (k + 2 * alpha - 1) * c0) / (k + 1)
    return c1


# ---- hypergeometric ------------------------------------------------------------------------------------------------------
def hyp1f1(a: float, b: float, x, terms: int = 300):
    x = _f64(x)
    s, t = torch.ones_like(x), torch.ones_like(x)
    for k in range(terms):
        t = t * (a + k) / (b + k) * x / (k + 1)
        s = s + t
    return s


def hyp2f1(a: float, b: float, c: float, x, terms: int = 500):
    """Gauss series, |x| < 1."""
    x = _f64(x)
    s, t = torch.ones_like(x), torch.ones_like(x)
    for k in range(terms):
        t = t * (a + k) * (b + k) / (c + k) * x / (k + 1)
        s = s + t
    return s


# ---- Airy ------------------------------------------------------------------------------------------------------------------
def airy(x):
    """(Ai(x), Bi(x)) from the Maclaurin series for |x| <= 5 and the leading asymptotic forms beyond."""
    x = _f64(x)
    c1, c2 = 0.3550280538878172, 0.2588194037928068
    xs = x.clamp(-5.5, 5.5)
    f, g, tf, tg = torch.ones_like(xs), xs.clone(), torch.ones_like(xs), xs.clone()
    x3 = xs ** 3
    for k in range(1, 80):
        tf = tf * x3 / ((3 * k - 1) * (3 * k))
        tg = tg * x3 / ((3 * k) * (3 * k + 1))
        f, g = f + tf, g + tg
    ai_s, bi_s = c1 * f - c2 * g, math.sqrt(3) * (c1 * f + c2 * g)
    xp = x.clamp(min=5.0)
    z = 2 / 3 * xp ** 1.5
    ai_p = torch.exp(-z) / (2 * math.sqrt(math.pi) * xp ** 0.25) * (1 - 5 / (72 * z))
    bi_p = torch.exp(z) / (math.sqrt(math.pi) * xp ** 0.25) * (1 + 5 / (72 * z))
    xn = (-x).clamp(min=5.0)
    zn = 2 / 3 * xn ** 1.5
    ai_n = (torch.sin(zn + math.pi / 4) - 5 / (72 * zn) * torch.cos(zn + math.pi / 4)) / (math.sqrt(math.pi) * xn ** 0.25)
    bi_n = (torch.cos(zn + math.pi / 4) + 5 / (72 * zn) * torch.sin(zn + math.pi / 4)) / (math.sqrt(math.pi) * xn ** 0.25)
    ai = torch.where(x > 5.5, ai_p, torch.where(x < -5.5, ai_n, ai_s))
    bi = torch.where(x > 5.5, bi_p, torch.where(x < -5.5, bi_n, bi_s))
    return ai, bi


# ---- incomplete beta and distributions -------------------------------------------------------------------------------------
def betainc(a, b, x):
    """Regularised incomplete beta function I_x(a, b) by Lentz's continued fraction (with the symmetry transformation)."""
    a, b, x = torch.broadcast_tensors(_f64(a), _f64(b), _f64(x))
    x = x.clamp(0, 1)
    swap = x > (a + 1) / (a + b + 2)
    aa, bb, xx = torch.where(swap, b, a), torch.where(swap, a, b), torch.where(swap, 1 - x, x)
    lbeta = torch.lgamma(aa) + torch.lgamma(bb) - torch.lgamma(aa + bb)
    front = torch.exp(aa * torch.log(xx.clamp(min=1e-300)) + bb * torch.log((1 - xx).clamp(min=1e-300)) - lbeta) / aa
    tiny = 1e-300
    c, d = torch.ones_like(xx), 1 - (aa + bb) * xx / (aa + 1)
    d = 1 / torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
    h = d
    for m in range(1, 300):
        m2 = 2 * m
        num = m * (bb - m) * xx / ((aa + m2 - 1) * (aa + m2))
        d = 1 + num * d
        d = 1 / torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
        c = 1 + num / c
        c = torch.where(c.abs() < tiny, torch.full_like(c, tiny), c)
        h = h * d * c
        num = -(aa + m) * (aa + bb + m) * xx / ((aa + m2) * (aa + m2 + 1))
        d = 1 + num * d
        d = 1 / torch.where(d.abs() < tiny, torch.full_like(d, tiny), d)
        c = 1 + num / c
        c = torch.where(c.abs() < tiny, torch.full_like(c, tiny), c)
        h = h * d * c
    val = front * h
    val = torch.where(swap, 1 - val, val)
    return torch.where(x <= 0, torch.zeros_like(val), torch.where(x >= 1, torch.ones_like(val), val))


def norm_cdf(x):
    return 0.5 * torch.erfc(-_f64(x) / math.sqrt(2))


def norm_ppf(p):
    return math.sqrt(2) * torch.erfinv(2 * _f64(p) - 1)


def student_t_cdf(t, df):
    t, df = _f64(t), _f64(df)
    ib = betainc(df / 2, torch.full_like(df, 0.5), df / (df + t * t))
    return torch.where(t >= 0, 1 - 0.5 * ib, 0.5 * ib)


def chi2_cdf(x, k):
    return torch.special.gammainc(_f64(k) / 2, _f64(x) / 2)


def f_cdf(x, d1, d2):
    x, d1, d2 = _f64(x), _f64(d1), _f64(d2)
    return betainc(d1 / 2, d2 / 2, d1 * x / (d1 * x + d2))


def binom_cdf(k, n, p):
    k, n, p = _f64(k), _f64(n), _f64(p)
    return torch.where(k >= n, torch.ones_like(p), betainc(n - k, k + 1, 1 - p))


# ---- fast approximations -----------------------------------------------------------------------------------------------
def fast_tanh(x):
    """Rational (7, 6) approximation, |error| < 3e-5 on the real line after clamping."""
    x = x.clamp(-4.97, 4.97)
    x2 = x * x
    return x * (135135 + x2 * (17325 + x2 * (378 + x2))) / (135135 + x2 * (62370 + x2 * (3150 + 28 * x2)))


def fast_exp(x):
    """2^(x log2 e) with the fraction approximated by a degree-4 polynomial (relative error < 1e-4)."""
    y = x * 1.4426950408889634
    n = torch.floor(y)
    f = y - n
    p = 1 + f * (0.6931472 + f * (0.2402265 + f * (0.0555041 + f * 0.0096139 * 1.4)))
    return torch.ldexp(p, n.to(torch.int32))
