"""Time-series methods beyond :mod:`torsh_b200.series` (``crates/torsh-series/src``): stationarity and diagnostic tests,
LOESS-based STL, seasonal ARIMA with automatic order selection, nonlinear state estimation (extended / unscented Kalman,
particle filter), change points by PELT, causality (Granger, transfer entropy), mode decompositions (EMD, VMD),
imputation, outlier handling with an isolation forest, rolling statistics, feature extraction, time-aware
cross-validation, forecast metrics and neural forecasters.  Inputs are 1-D tensors unless stated; arithmetic is float64."""
from __future__ import annotations

import math
from typing import Callable, Sequence

import numpy as np
import torch
from torch import nn

from . import series as S


def _t(x) -> torch.Tensor: return torch.as_tensor(x, dtype=torch.float64)


def _ols(X: torch.Tensor, y: torch.Tensor):
    beta = torch.linalg.lstsq(X, y[:, None]).solution[:, 0]
    resid = y - X @ beta
    dof = max(len(y) - X.shape[1], 1)
    sigma2 = float(resid @ resid) / dof
    cov = sigma2 * torch.linalg.pinv(X.t() @ X)
    return beta, resid, cov, sigma2


# ================================================================================================ tests
_ADF_CRIT = {"c": {"1%": -3.43, "5%": -2.86, "10%": -2.57}, "ct": {"1%": -3.96, "5%": -3.41, "10%": -3.12}, "n": {"1%": -2.58, "5%": -1.95, "10%": -1.62}}


def adf_test(x, lags: int | None = None, regression: str = "c") -> dict:
    """Augmented Dickey-Fuller: t statistic of ``gamma`` in ``dy_t = a (+ b t) + gamma y_{t-1} + sum phi_i dy_{t-i}``; the
    series is called stationary when the statistic is below the 5 % asymptotic critical value."""
    x = _t(x)
    n = len(x)
    lags = int(12 * (n / 100) ** 0.25) if lags is None else lags
    lags = min(lags, n // 2 - 2)
    dy = x[1:] - x[:-1]
    rows = len(dy) - lags
    cols = [x[lags:-1]] + [dy[lags - i:len(dy) - i] for i in range(1, lags + 1)]
    if regression in ("c", "ct"):
        cols.append(torch.ones(rows, dtype=torch.float64))
    if regression == "ct":
        cols.append(torch.arange(rows, dtype=torch.float64))
    X = torch.stack(cols, 1)
    beta, _, cov, _ = _ols(X, dy[lags:])
    stat = float(beta[0] / cov[0, 0].sqrt())
    crit = _ADF_CRIT[regression]
    return {"statistic": stat, "lags": lags, "critical_values": crit, "stationary": stat < crit["5%"]}


_KPSS_CRIT = {"c": {"10%": 0.347, "5%": 0.463, "1%": 0.739}, "ct": {"10%": 0.119, "5%": 0.146, "1%": 0.216}}


def kpss_test(x, regression: str = "c", lags: int | None = None) -> dict:
    """KPSS (null: stationary): partial sums of residuals over a Bartlett long-run variance."""
    x = _t(x)
    n = len(x)
    X = torch.ones(n, 1, dtype=torch.float64) if regression == "c" else torch.stack([torch.ones(n, dtype=torch.float64), torch.arange(n, dtype=torch.float64)], 1)
    _, e, _, _ = _ols(X, x)
    lags = int(4 * (n / 100) ** 0.25) if lags is None else lags
    lrv = float(e @ e) / n + sum(2 * (1 - k / (lags + 1)) * float(e[k:] @ e[:-k]) / n for k in range(1, lags + 1))
    stat = float((e.cumsum(0) ** 2).sum()) / (n * n * lrv)
    crit = _KPSS_CRIT[regression]
    return {"statistic": stat, "lags": lags, "critical_values": crit, "stationary": stat < crit["5%"]}


def _chi2_sf(x: float, k: int) -> float:
    return float(torch.special.gammaincc(torch.tensor(k / 2, dtype=torch.float64), torch.tensor(x / 2, dtype=torch.float64)))


def ljung_box(x, lags: int = 10, fitted_params: int = 0) -> dict:
    x = _t(x)
    n = len(x)
    r = S.acf(x.float(), lags).double()[1:]
    q = float(n * (n + 2) * (r ** 2 / (n - torch.arange(1, lags + 1, dtype=torch.float64))).sum())
    p = _chi2_sf(q, max(lags - fitted_params, 1))
    return {"statistic": q, "p_value": p, "white_noise": p > 0.05}


def jarque_bera(x) -> dict:
    x = _t(x)
    n, z = len(x), (x - x.mean()) / x.std(unbiased=False)
    skew, kurt = float((z ** 3).mean()), float((z ** 4).mean())
    jb = n / 6 * (skew ** 2 + (kurt - 3) ** 2 / 4)
    return {"statistic": jb, "p_value": _chi2_sf(jb, 2), "skewness": skew, "kurtosis": kurt, "normal": _chi2_sf(jb, 2) > 0.05}


def residual_diagnostics(resid, lags: int = 10, fitted_params: int = 0) -> dict:
    r = _t(resid)
    half = len(r) // 2
    f = float(r[half:].var() / r[:half].var().clamp(min=1e-300))
    return {"mean": float(r.mean()), "ljung_box": ljung_box(r, lags, fitted_params), "jarque_bera": jarque_bera(r), "variance_ratio": f, "homoscedastic": 0.5 < f < 2.0}


def stationarity_suite(x) -> dict:
    a, k = adf_test(x), kpss_test(x)
    verdict = ("stationary" if a["stationary"] and k["stationary"] else "unit_root" if not a["stationary"] and not k["stationary"] else
               "trend_stationary" if not a["stationary"] else "difference_stationary")
    return {"adf": a, "kpss": k, "verdict": verdict, "suggested_differences": 0 if verdict == "stationary" else 1}


def granger_causality(y, x, lags: int = 2) -> dict:
    """F test: do ``lags`` past values of ``x`` improve an autoregression of ``y``?"""
    y, x = _t(y), _t(x)
    n = len(y) - lags
    own = [y[lags - i:len(y) - i] for i in range(1, lags + 1)]
    other = [x[lags - i:len(x) - i] for i in range(1, lags + 1)]
    one = torch.ones(n, dtype=torch.float64)
    _, r0, _, _ = _ols(torch.stack(own + [one], 1), y[lags:])
    _, r1, _, _ = _ols(torch.stack(own + other + [one], 1), y[lags:])
    rss0, rss1 = float(r0 @ r0), float(r1 @ r1)
    dof = n - 2 * lags - 1
    f = ((rss0 - rss1) / lags) / (rss1 / dof)
    from scipy import stats
    p = float(stats.f.sf(f, lags, dof))
    return {"f": f, "p_value": p, "causes": p < 0.05}


def transfer_entropy(source, target, bins: int = 4, lag: int = 1) -> float:
    """``TE(source -> target)`` in nats from quantile-binned symbols: ``I(target_t ; source_{t-lag} | target_{t-lag})``."""
    def sym(v):
        v = _t(v)
        edges = torch.quantile(v, torch.linspace(0, 1, bins + 1, dtype=torch.float64)[1:-1])
        return torch.bucketize(v, edges)
    s, t = sym(source), sym(target)
    a, b, c = t[lag:], t[:-lag], s[:-lag]
    def H(*cols):
        key = sum(col * bins ** i for i, col in enumerate(cols))
        p = torch.bincount(key).double()
        p = p[p > 0] / p.sum()
        return float(-(p * p.log()).sum())
    return H(a, b) + H(b, c) - H(b) - H(a, b, c)


# ================================================================================================ STL
def _loess(y: torch.Tensor, span: int, weights: torch.Tensor | None = None, degree: int = 1, at: torch.Tensor | None = None) -> torch.Tensor:
    """Local regression with tricube weights over the ``span`` nearest points of each position."""
    n = len(y)
    x = torch.arange(n, dtype=torch.float64)
    at = x if at is None else at
    span = min(max(span, degree + 2), n)
    d = (at[:, None] - x[None]).abs()
    h = d.kthvalue(span, dim=1).values.clamp(min=1e-12)[:, None]
    w = (1 - (d / h).clamp(max=1) ** 3) ** 3
    if weights is not None:
        w = w * weights[None]
    dx = x[None] - at[:, None]
    if degree == 0:
        return (w * y).sum(1) / w.sum(1).clamp(min=1e-300)
    s0, s1, s2 = w.sum(1), (w * dx).sum(1), (w * dx * dx).sum(1)
    t0, t1 = (w * y).sum(1), (w * dx * y).sum(1)
    det = (s0 * s2 - s1 * s1)
    safe = det.abs() > 1e-12
    return torch.where(safe, (s2 * t0 - s1 * t1) / torch.where(safe, det, torch.ones_like(det)), t0 / s0.clamp(min=1e-300))


def stl(x, period: int, seasonal: int = 7, trend: int | None = None, robust: bool = False, inner: int = 2, outer: int | None = None) -> dict:
    """Seasonal-trend decomposition by LOESS (Cleveland et al.): cycle-subseries smoothing, low-pass filtering of the
    seasonal, trend smoothing of the de-seasonalised series; ``robust`` re-weights by bisquare of the remainder."""
    x = _t(x)
    n = len(x)
    trend = trend or (int(math.ceil(1.5 * period / (1 - 1.5 / seasonal))) | 1)
    low = period | 1
    outer = (6 if robust else 0) if outer is None else outer
    tr, rw, seas = torch.zeros(n, dtype=torch.float64), torch.ones(n, dtype=torch.float64), torch.zeros(n, dtype=torch.float64)
    ma = lambda v, k: v.unfold(0, k, 1).mean(1)
    for o in range(outer + 1):
        for _ in range(inner):
            det = x - tr
            c = torch.zeros(n + 2 * period, dtype=torch.float64)
            for ph in range(period):
                sub, wsub = det[ph::period], rw[ph::period]
                at = torch.arange(-1, len(sub) + 1, dtype=torch.float64)
                c[ph::period][:len(at)] = _loess(sub, seasonal, wsub, 1, at)
            lp = _loess(ma(ma(ma(c, period), period), 3), low)
            seas = c[period:period + n] - lp
            tr = _loess(x - seas, trend, rw)
        if o < outer:
            r = (x - seas - tr).abs()
            h = 6 * r.median().clamp(min=1e-12)
            rw = (1 - (r / h).clamp(max=1) ** 2) ** 2
    return {"trend": tr, "seasonal": seas, "remainder": x - tr - seas, "weights": rw}


# ================================================================================================ seasonal ARIMA
class SARIMA:
    """``(p, d, q) x (P, D, Q)_s`` fitted by conditional sum of squares: the multiplied-out AR and MA polynomials give
    one-step residuals; parameters minimise their sum of squares with L-BFGS; AIC from the innovation variance."""

    def __init__(self, order=(1, 0, 0), seasonal_order=(0, 0, 0, 0)):
        self.order, self.sorder = order, seasonal_order

    @staticmethod
    def _poly(coefs: torch.Tensor, step: int, sign: float) -> torch.Tensor:
        out = torch.zeros(len(coefs) * step + 1, dtype=torch.float64)
        out[0] = 1.0
        for i, c in enumerate(coefs):
            out = out.index_add(0, torch.tensor([(i + 1) * step]), (sign * c)[None])
        return out

    @staticmethod
    def _mul(a, b):
        return torch.nn.functional.conv1d(a[None, None], b.flip(0)[None, None], padding=len(b) - 1)[0, 0]

    def _polys(self, th):
        p, _, q = self.order
        P, _, Q, s = self.sorder
        ar = self._mul(self._poly(th[:p], 1, -1.0), self._poly(th[p:p + P], max(s, 1), -1.0))
        ma = self._mul(self._poly(th[p + P:p + P + q], 1, 1.0), self._poly(th[p + P + q:p + P + q + Q], max(s, 1), 1.0))
        return ar, ma

    def _difference(self, x):
        _, d, _ = self.order
        _, D, _, s = self.sorder
        for _ in range(D):
            x = x[s:] - x[:-s]
        for _ in range(d):
            x = x[1:] - x[:-1]
        return x

    def _residuals(self, w, th):
        ar, ma = self._polys(th[:-1])
        z = w - th[-1]
        u = torch.nn.functional.conv1d(torch.nn.functional.pad(z, (len(ar) - 1, 0))[None, None], ar.flip(0)[None, None])[0, 0]
        e = []
        for t in range(len(z)):
            acc = u[t]
            for j in range(1, min(len(ma), t + 1)):
                acc = acc - ma[j] * e[t - j]
            e.append(acc)
        return torch.stack(e)

    def fit(self, x, iters: int = 60):
        self.x = _t(x)
        w = self._difference(self.x)
        k = self.order[0] + self.order[2] + self.sorder[0] + self.sorder[2]
        th = torch.zeros(k + 1, dtype=torch.float64)
        th[-1] = w.mean()
        th.requires_grad_(True)
        opt = torch.optim.LBFGS([th], lr=0.5, max_iter=iters, line_search_fn="strong_wolfe")
        burn = len(self._polys(th.detach()[:-1])[0]) - 1
        def closure():
            opt.zero_grad()
            e = self._residuals(w, th)
            loss = (e[burn:] ** 2).mean()
            loss.backward()
            return loss
        opt.step(closure)
        self.params = th.detach()
        e = self._residuals(w, self.params)
        self.residuals, self.sigma2 = e[burn:], float((e[burn:] ** 2).mean())
        n = len(e) - burn
        self.aic = n * math.log(self.sigma2) + 2 * (k + 1)
        self.bic = n * math.log(self.sigma2) + math.log(n) * (k + 1)
        self._w, self._e = w, e
        return self

    def forecast(self, steps: int) -> torch.Tensor:
        ar, ma = self._polys(self.params[:-1])
        mu = self.params[-1]
        z, e = list((self._w - mu).tolist()), list(self._e.tolist())
        for _ in range(steps):
            v = -sum(float(ar[j]) * z[-j] for j in range(1, len(ar)) if j <= len(z)) + sum(float(ma[j]) * e[-j] for j in range(1, len(ma)) if j <= len(e))
            z.append(v); e.append(0.0)
        w_f = torch.tensor(z[-steps:], dtype=torch.float64) + mu
        # undo the differences, regular ones first (they were applied last)
        _, d, _ = self.order
        _, D, _, s = self.sorder
        levels, cur = [self.x], self.x
        for _ in range(D):
            cur = cur[s:] - cur[:-s]; levels.append(cur)
        for _ in range(d):
            cur = cur[1:] - cur[:-1]; levels.append(cur)
        f = w_f
        for i in range(d):
            f = levels[-2 - i][-1] + f.cumsum(0)
        for i in range(D):
            base = levels[D - 1 - i].tolist()
            out = []
            for t in range(steps):
                prev = base[len(base) - s + t] if t < s else out[t - s]
                out.append(prev + float(f[t]))
            f = torch.tensor(out, dtype=torch.float64)
        return f


def auto_arima(x, max_p: int = 3, max_q: int = 3, max_d: int = 2, seasonal_period: int = 0, criterion: str = "aic") -> SARIMA:
    """Differencing order from repeated KPSS tests, then a grid over ``(p, q)`` (and seasonal ``(P, Q) <= 1`` when a period
    is given) picking the lowest information criterion."""
    x = _t(x)
    d, cur = 0, x
    while d < max_d and not kpss_test(cur)["stationary"]:
        cur, d = cur[1:] - cur[:-1], d + 1
    best = None
    seasonal_grid = [(0, 0)] if not seasonal_period else [(0, 0), (1, 0), (0, 1)]
    for p in range(max_p + 1):
        for q in range(max_q + 1):
            for P, Q in seasonal_grid:
                try:
                    m = SARIMA((p, d, q), (P, 1 if seasonal_period and (P or Q) else 0, Q, seasonal_period)).fit(x, iters=30)
                except Exception:
                    continue
                score = getattr(m, criterion)
                if math.isfinite(score) and (best is None or score < getattr(best, criterion)):
                    best = m
    return best


# ================================================================================================ nonlinear filters
class ExtendedKalmanFilter:
    """``x' = f(x) + w``, ``z = h(x) + v`` with Jacobians from autograd."""

    def __init__(self, f: Callable, h: Callable, Q, R, x0, P0):
        self.f, self.h, self.Q, self.R, self.x, self.P = f, h, _t(Q), _t(R), _t(x0), _t(P0)

    def step(self, z):
        F = torch.autograd.functional.jacobian(self.f, self.x)
        xp = self.f(self.x)
        Pp = F @ self.P @ F.t() + self.Q
        H = torch.autograd.functional.jacobian(self.h, xp)
        S_ = H @ Pp @ H.t() + self.R
        K = Pp @ H.t() @ torch.linalg.inv(S_)
        self.x = xp + K @ (_t(z) - self.h(xp))
        self.P = (torch.eye(len(self.x), dtype=torch.float64) - K @ H) @ Pp
        return self.x

    def filter(self, zs): return torch.stack([self.step(z) for z in zs])


class UnscentedKalmanFilter:
    """Scaled unscented transform with ``2n + 1`` sigma points (``alpha``, ``beta``, ``kappa``)."""

    def __init__(self, f, h, Q, R, x0, P0, alpha=1e-1, beta=2.0, kappa=0.0):
        self.f, self.h, self.Q, self.R, self.x, self.P = f, h, _t(Q), _t(R), _t(x0), _t(P0)
        n = len(self.x)
        lam = alpha ** 2 * (n + kappa) - n
        self.n, self.lam = n, lam
        self.wm = torch.full((2 * n + 1,), 1 / (2 * (n + lam)), dtype=torch.float64)
        self.wc = self.wm.clone()
        self.wm[0], self.wc[0] = lam / (n + lam), lam / (n + lam) + 1 - alpha ** 2 + beta

    def _sigma(self, x, P):
        L = torch.linalg.cholesky((self.n + self.lam) * (P + 1e-12 * torch.eye(self.n, dtype=torch.float64)))
        return torch.cat([x[None], x[None] + L.t(), x[None] - L.t()])

    def step(self, z):
        sp = torch.stack([self.f(s) for s in self._sigma(self.x, self.P)])
        xp = (self.wm[:, None] * sp).sum(0)
        dx = sp - xp
        Pp = (self.wc[:, None, None] * dx[:, :, None] * dx[:, None, :]).sum(0) + self.Q
        sp2 = self._sigma(xp, Pp)
        zs = torch.stack([self.h(s) for s in sp2])
        zp = (self.wm[:, None] * zs).sum(0)
        dz, dx2 = zs - zp, sp2 - xp
        S_ = (self.wc[:, None, None] * dz[:, :, None] * dz[:, None, :]).sum(0) + self.R
        C = (self.wc[:, None, None] * dx2[:, :, None] * dz[:, None, :]).sum(0)
        K = C @ torch.linalg.inv(S_)
        self.x = xp + K @ (_t(z) - zp)
        self.P = Pp - K @ S_ @ K.t()
        return self.x

    def filter(self, zs): return torch.stack([self.step(z) for z in zs])


class ParticleFilter:
    """Bootstrap filter: propagate with ``transition(particles, generator)``, weight by ``likelihood(z, particles)``, resample
    systematically when the effective sample size falls under half the particle count."""

    def __init__(self, transition, likelihood, particles: torch.Tensor, seed: int = 0):
        self.transition, self.likelihood, self.p = transition, likelihood, particles.double()
        self.w = torch.full((len(particles),), 1.0 / len(particles), dtype=torch.float64)
        self.gen, self.resamples = torch.Generator().manual_seed(seed), 0

    def step(self, z):
        self.p = self.transition(self.p, self.gen)
        self.w = self.w * self.likelihood(z, self.p).clamp(min=1e-300)
        self.w = self.w / self.w.sum()
        ess = 1 / float((self.w ** 2).sum())
        if ess < len(self.w) / 2:
            n = len(self.w)
            pos = (torch.rand((), generator=self.gen, dtype=torch.float64) + torch.arange(n, dtype=torch.float64)) / n
            idx = torch.searchsorted(self.w.cumsum(0), pos).clamp(max=n - 1)
            self.p, self.w, self.resamples = self.p[idx], torch.full((n,), 1.0 / n, dtype=torch.float64), self.resamples + 1
        return (self.w[:, None] * self.p.reshape(len(self.w), -1)).sum(0)

    def filter(self, zs): return torch.stack([self.step(z) for z in zs])


# ================================================================================================ change points
def pelt(x, penalty: float | None = None, min_size: int = 2, cost: str = "mean") -> list[int]:
    """Pruned exact linear time search for changes in mean (``cost='mean'``, squared error) or mean and variance
    (``'normal'``); returns the first index of every new segment."""
    x = _t(x)
    n = len(x)
    penalty = 2 * math.log(n) * float(x.var()) if penalty is None and cost == "mean" else (3 * math.log(n) if penalty is None else penalty)
    c1, c2 = torch.cat([torch.zeros(1, dtype=torch.float64), x.cumsum(0)]), torch.cat([torch.zeros(1, dtype=torch.float64), (x * x).cumsum(0)])
    def seg(a, b):
        m = b - a
        ss = float(c2[b] - c2[a] - (c1[b] - c1[a]) ** 2 / m)
        return ss if cost == "mean" else m * math.log(max(ss / m, 1e-12))
    F = [-penalty] + [math.inf] * n
    last, cand = [0] * (n + 1), [0]
    for t in range(min_size, n + 1):
        vals = [(F[s] + seg(s, t) + penalty, s) for s in cand if t - s >= min_size]
        if not vals:
            continue
        F[t], last[t] = min(vals)
        cand = [s for v, s in vals if v - penalty <= F[t]] + [t - min_size + 1]
    out, t = [], n
    while t > 0:
        t = last[t]
        if t > 0:
            out.append(t)
    return sorted(out)


# ================================================================================================ mode decompositions
def emd(x, max_imfs: int = 8, sift_iters: int = 50, tol: float = 0.05) -> list[torch.Tensor]:
    """Empirical mode decomposition: repeated sifting (subtract the mean of cubic-spline envelopes through the local
    maxima and minima) until the residue is monotone; returns the IMFs followed by the residue."""
    from scipy.interpolate import CubicSpline
    r, n, out = np.asarray(_t(x)), len(x), []
    t = np.arange(n)
    def extrema(v):
        d = np.diff(v)
        mx = np.nonzero((d[:-1] > 0) & (d[1:] <= 0))[0] + 1
        mn = np.nonzero((d[:-1] < 0) & (d[1:] >= 0))[0] + 1
        return mx, mn
    for _ in range(max_imfs):
        h = r.copy()
        for _ in range(sift_iters):
            mx, mn = extrema(h)
            if len(mx) < 3 or len(mn) < 3:
                break
            # mirror the end extrema so the envelopes do not swing at the boundaries
            pad = lambda idx: np.concatenate([[-idx[0]], idx, [2 * (n - 1) - idx[-1]]])
            padv = lambda idx: np.concatenate([[h[idx[0]]], h[idx], [h[idx[-1]]]])
            mean = (CubicSpline(pad(mx), padv(mx))(t) + CubicSpline(pad(mn), padv(mn))(t)) / 2
            new = h - mean
            sd = np.sum(mean ** 2) / max(np.sum(h ** 2), 1e-300)
            h = new
            if sd < tol ** 2:
                break
        mx, mn = extrema(h)
        if len(mx) + len(mn) < 4:
            break
        out.append(torch.from_numpy(h.copy()))
        r = r - h
        if len(extrema(r)[0]) + len(extrema(r)[1]) < 3:
            break
    return out + [torch.from_numpy(r)]


def vmd(x, k: int = 3, alpha: float = 2000.0, tau: float = 0.0, iters: int = 500, tol: float = 1e-7):
    """Variational mode decomposition (Dragomiretskiy & Zosso): ``k`` band-limited modes found by ADMM in the frequency
    domain on the mirrored signal.  Returns ``(modes [k, n], centre frequencies in cycles per sample)``."""
    f = np.asarray(_t(x))
    n = len(f)
    fm = np.concatenate([f[:n // 2][::-1], f, f[n // 2:][::-1]])
    T = len(fm)
    freqs = np.arange(T) / T - 0.5
    fh = np.fft.fftshift(np.fft.fft(fm))
    fh[:T // 2] = 0
    u = np.zeros((k, T), complex)
    omega = 0.5 / k * np.arange(k)
    lam = np.zeros(T, complex)
    for _ in range(iters):
        prev = u.copy()
        for i in range(k):
            rest = u.sum(0) - u[i]
            u[i] = (fh - rest - lam / 2) / (1 + alpha * (freqs - omega[i]) ** 2)
            p = np.abs(u[i, T // 2:]) ** 2
            omega[i] = (freqs[T // 2:] @ p) / max(p.sum(), 1e-300)
        lam = lam + tau * (u.sum(0) - fh)
        if sum(np.sum(np.abs(u[i] - prev[i]) ** 2) for i in range(k)) / T < tol:
            break
    full = np.zeros((k, T), complex)
    full[:, T // 2:] = u[:, T // 2:]
    full[:, 1:T // 2 + 1] = np.conj(u[:, T // 2:][:, ::-1])[:, :T // 2] if T % 2 == 0 else np.conj(u[:, T // 2 + 1:][:, ::-1])
    modes = np.real(np.fft.ifft(np.fft.ifftshift(full, axes=1), axis=1))[:, n // 2:n // 2 + n]
    order = np.argsort(omega)
    return torch.from_numpy(modes[order].copy()), torch.from_numpy(omega[order].copy())


# ================================================================================================ imputation / outliers
def impute(x, method: str = "linear", period: int | None = None) -> torch.Tensor:
    """Fills NaNs: ``mean``, ``ffill``, ``bfill``, ``linear``, ``spline`` (cubic through the observed points) or ``seasonal``
    (mean of the same phase, needs ``period``)."""
    x = _t(x).clone()
    miss = torch.isnan(x)
    if not miss.any():
        return x
    idx = torch.arange(len(x), dtype=torch.float64)
    ok = ~miss
    if method == "mean":
        x[miss] = x[ok].mean()
    elif method in ("ffill", "bfill"):
        src = torch.where(ok, torch.arange(len(x)), torch.full((len(x),), -1 if method == "ffill" else len(x)))
        src = src.cummax(0).values if method == "ffill" else src.flip(0).cummin(0).values.flip(0)
        fill = x[src.clamp(0, len(x) - 1)]
        x = torch.where(miss & (src >= 0) & (src < len(x)), fill, x)
        if torch.isnan(x).any():
            x = impute(x, "bfill" if method == "ffill" else "ffill")
    elif method == "linear":
        x[miss] = torch.from_numpy(np.interp(idx[miss].numpy(), idx[ok].numpy(), x[ok].numpy()))
    elif method == "spline":
        from scipy.interpolate import CubicSpline
        x[miss] = torch.from_numpy(CubicSpline(idx[ok].numpy(), x[ok].numpy())(idx[miss].numpy()))
    elif method == "seasonal":
        for ph in range(period):
            sl = slice(ph, None, period)
            v = x[sl]
            v[torch.isnan(v)] = v[~torch.isnan(v)].mean() if (~torch.isnan(v)).any() else x[ok].mean()
            x[sl] = v
    else:
        raise ValueError(f"unknown imputation method {method!r}")
    return x


class IsolationForest:
    """Random axis-aligned isolation trees on ``[n, d]`` data; the score ``2^(-E[path] / c(psi))`` is near 1 for points that
    isolate quickly."""

    def __init__(self, trees: int = 100, sample_size: int = 256, seed: int = 0):
        self.trees, self.psi, self.rng, self.forest = trees, sample_size, np.random.default_rng(seed), []

    @staticmethod
    def _c(n): return 2 * (math.log(n - 1) + 0.5772156649) - 2 * (n - 1) / n if n > 2 else (1.0 if n == 2 else 0.0)

    def _grow(self, X, depth, limit):
        if depth >= limit or len(X) <= 1:
            return ("leaf", len(X))
        f = self.rng.integers(X.shape[1])
        lo, hi = X[:, f].min(), X[:, f].max()
        if lo == hi:
            return ("leaf", len(X))
        s = self.rng.uniform(lo, hi)
        m = X[:, f] < s
        return ("node", f, s, self._grow(X[m], depth + 1, limit), self._grow(X[~m], depth + 1, limit))

    def fit(self, X):
        X = np.asarray(_t(X)).reshape(len(X), -1)
        psi = min(self.psi, len(X))
        self.psi_eff = psi
        self.forest = [self._grow(X[self.rng.choice(len(X), psi, replace=False)], 0, math.ceil(math.log2(psi))) for _ in range(self.trees)]
        return self

    def _path(self, x, node, depth):
        while node[0] == "node":
            node, depth = (node[3] if x[node[1]] < node[2] else node[4]), depth + 1
        return depth + self._c(node[1])

    def score(self, X) -> torch.Tensor:
        X = np.asarray(_t(X)).reshape(len(X), -1)
        e = np.array([[self._path(x, t, 0) for t in self.forest] for x in X]).mean(1)
        return torch.from_numpy(2 ** (-e / self._c(self.psi_eff)))


def detect_outliers(x, method: str = "hampel", window: int = 7, threshold: float = 3.0) -> torch.Tensor:
    """Boolean mask: ``hampel`` (rolling median / MAD), ``zscore``, ``iqr`` or ``isolation_forest`` (on value and first difference)."""
    x = _t(x)
    if method == "hampel":
        pad = torch.nn.functional.pad(x[None, None], (window // 2, window // 2), mode="replicate")[0, 0].unfold(0, window, 1)
        med = pad.median(1).values
        mad = 1.4826 * (pad - med[:, None]).abs().median(1).values
        return (x - med).abs() > threshold * mad.clamp(min=1e-12)
    if method == "zscore":
        return ((x - x.mean()) / x.std()).abs() > threshold
    if method == "iqr":
        q1, q3 = torch.quantile(x, 0.25), torch.quantile(x, 0.75)
        return (x < q1 - 1.5 * (q3 - q1)) | (x > q3 + 1.5 * (q3 - q1))
    feats = torch.stack([x, torch.cat([torch.zeros(1, dtype=torch.float64), x[1:] - x[:-1]])], 1)
    return IsolationForest(seed=0).fit(feats).score(feats) > 0.65


def treat_outliers(x, mask, how: str = "interpolate") -> torch.Tensor:
    x = _t(x).clone()
    if how == "clip":
        lo, hi = x[~mask].min(), x[~mask].max()
        return x.clamp(lo, hi)
    x[mask] = float("nan")
    return impute(x, "linear" if how == "interpolate" else "mean")


# ================================================================================================ rolling / features / CV / metrics
def rolling(x, window: int, stat: str = "mean") -> torch.Tensor:
    """Trailing window statistics (``mean``, ``std``, ``min``, ``max``, ``median``, ``sum``); the first ``window - 1`` are NaN."""
    x = _t(x)
    w = x.unfold(0, window, 1)
    v = {"mean": lambda: w.mean(1), "std": lambda: w.std(1), "min": lambda: w.amin(1), "max": lambda: w.amax(1), "median": lambda: w.median(1).values, "sum": lambda: w.sum(1)}[stat]()
    return torch.cat([torch.full((window - 1,), float("nan"), dtype=torch.float64), v])


def ewm(x, alpha: float) -> torch.Tensor:
    x, out = _t(x), []
    acc = x[0]
    for v in x:
        acc = alpha * v + (1 - alpha) * acc
        out.append(acc)
    return torch.stack(out)


def extract_features(x, period: int | None = None) -> dict:
    """Summary features in the style of tsfeatures: moments, trend and seasonal strength (from STL), autocorrelation,
    spectral entropy, crossing points, flat spots."""
    x = _t(x)
    n = len(x)
    z = (x - x.mean()) / x.std().clamp(min=1e-12)
    period = period or int(S.dominant_period(x.float()))
    out = {"mean": float(x.mean()), "std": float(x.std()), "skewness": float((z ** 3).mean()), "kurtosis": float((z ** 4).mean()),
           "acf1": float(S.acf(x.float(), 1)[1]), "spectral_entropy": float(S.spectral_entropy(x.float())),
           "crossing_points": int(((x[:-1] > x.median()) != (x[1:] > x.median())).sum()), "linear_slope": float(np.polyfit(np.arange(n), x.numpy(), 1)[0]), "period": period}
    if 2 <= period <= n // 2:
        d = stl(x, period)
        rv = d["remainder"].var()
        out["trend_strength"] = float((1 - rv / (d["trend"] + d["remainder"]).var().clamp(min=1e-300)).clamp(min=0))
        out["seasonal_strength"] = float((1 - rv / (d["seasonal"] + d["remainder"]).var().clamp(min=1e-300)).clamp(min=0))
    return out


class TimeSeriesCV:
    """Splitters that never train on the future: ``expanding`` (growing train window), ``sliding`` (fixed window),
    ``blocked`` (disjoint consecutive blocks, each split inside its block), with an optional ``gap`` between train and test
    (purging) and an ``embargo`` after each test fold that later training folds skip."""

    def __init__(self, n_splits: int = 5, test_size: int | None = None, mode: str = "expanding", train_size: int | None = None, gap: int = 0, embargo: int = 0):
        self.k, self.test_size, self.mode, self.train_size, self.gap, self.embargo = n_splits, test_size, mode, train_size, gap, embargo

    def split(self, n: int):
        if self.mode == "blocked":
            block = n // self.k
            for i in range(self.k):
                lo, hi = i * block, (i + 1) * block
                cut = lo + int(0.8 * block)
                yield list(range(lo, cut - self.gap)), list(range(cut, hi))
            return
        ts = self.test_size or n // (self.k + 1)
        for i in range(self.k):
            test_lo = n - (self.k - i) * ts
            train_hi = test_lo - self.gap
            train_lo = 0 if self.mode == "expanding" else max(0, train_hi - (self.train_size or ts * 2))
            train = [t for t in range(train_lo, train_hi)]
            if self.embargo:                                                  # drop training points that fall right after an earlier test fold
                banned = set()
                for j in range(i):
                    e_lo = n - (self.k - j) * ts + ts
                    banned |= set(range(e_lo, e_lo + self.embargo))
                train = [t for t in train if t not in banned]
            yield train, list(range(test_lo, test_lo + ts))

    def score(self, x, fit_forecast: Callable[[torch.Tensor, int], torch.Tensor], metric: Callable | None = None) -> list[float]:
        x, metric = _t(x), metric or (lambda a, f: float((a - f).abs().mean()))
        return [metric(x[te], fit_forecast(x[tr], len(te))) for tr, te in self.split(len(x))]


def forecast_metrics(actual, forecast, train=None, period: int = 1) -> dict:
    a, f = _t(actual), _t(forecast)
    e = a - f
    out = {"mae": float(e.abs().mean()), "rmse": float((e ** 2).mean().sqrt()), "mape": float((e.abs() / a.abs().clamp(min=1e-12)).mean() * 100),
           "smape": float((2 * e.abs() / (a.abs() + f.abs()).clamp(min=1e-12)).mean() * 100), "bias": float(e.mean())}
    if train is not None:
        tr = _t(train)
        scale = (tr[period:] - tr[:-period]).abs().mean().clamp(min=1e-12)
        out["mase"] = float(e.abs().mean() / scale)
    return out


# ================================================================================================ neural forecasters
class _WindowForecaster(nn.Module):
    def fit(self, x, epochs: int = 200, lr: float = 1e-2, seed: int = 0):
        torch.manual_seed(seed)
        x = torch.as_tensor(x, dtype=torch.float32)
        self.mu, self.sd = x.mean(), x.std().clamp(min=1e-6)
        z = (x - self.mu) / self.sd
        w = z.unfold(0, self.window + self.horizon, 1)
        xs, ys = w[:, :self.window], w[:, self.window:]
        opt = torch.optim.Adam(self.parameters(), lr)
        for _ in range(epochs):
            opt.zero_grad()
            loss = nn.functional.mse_loss(self(xs), ys)
            loss.backward()
            opt.step()
        self.train_loss = float(loss.detach())
        self._tail = z[-self.window:]
        return self

    @torch.no_grad()
    def forecast(self, steps: int) -> torch.Tensor:
        hist, out = self._tail.clone(), []
        while len(out) < steps:
            nxt = self(hist[None])[0]
            out += nxt.tolist()
            hist = torch.cat([hist, nxt])[-self.window:]
        return torch.tensor(out[:steps]) * self.sd + self.mu


class LSTMForecaster(_WindowForecaster):
    def __init__(self, window: int = 24, horizon: int = 1, hidden: int = 32, cell: str = "lstm"):
        super().__init__()
        self.window, self.horizon = window, horizon
        self.rnn = (nn.LSTM if cell == "lstm" else nn.GRU)(1, hidden, batch_first=True)
        self.head = nn.Linear(hidden, horizon)

    def forward(self, x): return self.head(self.rnn(x[..., None])[0][:, -1])


class GRUForecaster(LSTMForecaster):
    def __init__(self, window=24, horizon=1, hidden=32): super().__init__(window, horizon, hidden, "gru")


class CNNForecaster(_WindowForecaster):
    """Dilated causal convolutions (receptive field doubles per layer) and a linear head."""

    def __init__(self, window: int = 24, horizon: int = 1, channels: int = 16, layers: int = 3):
        super().__init__()
        self.window, self.horizon = window, horizon
        self.convs = nn.ModuleList(nn.Conv1d(1 if i == 0 else channels, channels, 2, dilation=2 ** i) for i in range(layers))
        self.head = nn.Linear(channels, horizon)

    def forward(self, x):
        h = x[:, None]
        for i, c in enumerate(self.convs):
            h = torch.relu(c(nn.functional.pad(h, (2 ** i, 0))))
        return self.head(h[:, :, -1])


class TransformerForecaster(_WindowForecaster):
    def __init__(self, window: int = 24, horizon: int = 1, dim: int = 32, heads: int = 4, layers: int = 2):
        super().__init__()
        self.window, self.horizon = window, horizon
        self.inp, self.pos = nn.Linear(1, dim), nn.Parameter(0.02 * torch.randn(window, dim))
        self.enc = nn.TransformerEncoder(nn.TransformerEncoderLayer(dim, heads, 2 * dim, dropout=0.0, batch_first=True), layers)
        self.head = nn.Linear(dim, horizon)

    def forward(self, x): return self.head(self.enc(self.inp(x[..., None]) + self.pos)[:, -1])


# ================================================================================================ dynamic linear models
class DynamicLinearModel:
    """Structural time-series model in state-space form (``crates/torsh-series/src/state_space/dlm.rs``): the state stacks a
    polynomial trend block (order 1 = local level, 2 = local linear trend), optional seasonal dummies of period ``s`` and
    regression coefficients; ``y_t = F_t' x_t + v_t``, ``x_t = G x_{t-1} + w_t``.  Kalman filter, Rauch-Tung-Striebel smoother,
    forecasts with intervals, the exact Gaussian log-likelihood and maximum-likelihood variances."""

    def __init__(self, trend_order: int = 1, seasonal_period: int | None = None, regressors: int = 0, obs_var: float = 1.0, level_var: float = 0.1, slope_var: float = 0.01, seasonal_var: float = 0.01, reg_var: float = 0.0):
        self.order, self.s, self.k = trend_order, seasonal_period, regressors
        self.vars = {"obs": obs_var, "level": level_var, "slope": slope_var, "seasonal": seasonal_var, "reg": reg_var}
        self.n = trend_order + ((seasonal_period - 1) if seasonal_period else 0) + regressors

    def _matrices(self, v: dict | None = None):
        v = v or self.vars
        G, W, F = torch.zeros(self.n, self.n, dtype=torch.float64), torch.zeros(self.n, dtype=torch.float64), torch.zeros(self.n, dtype=torch.float64)
        for i in range(self.order):
            G[i, i:self.order] = 1.0
        F[0] = 1.0
        W = W.clone(); W[0] = v["level"]
        Wd = [W[0]] + ([v["slope"]] * (self.order - 1))
        pos = self.order
        if self.s:
            m = self.s - 1
            G[pos, pos:pos + m] = -1.0
            for i in range(1, m):
                G[pos + i, pos + i - 1] = 1.0
            F[pos] = 1.0
            Wd += [v["seasonal"]] + [0.0] * (m - 1)
            pos += m
        for i in range(self.k):
            G[pos + i, pos + i] = 1.0
            Wd.append(v["reg"])
        Wm = torch.diag(torch.stack([torch.as_tensor(w, dtype=torch.float64) for w in Wd]))
        return G, Wm, F

    def filter(self, y: torch.Tensor, X: torch.Tensor | None = None, variances: dict | None = None, m0: torch.Tensor | None = None, c0: float = 1e6) -> dict:
        v = variances or self.vars
        G, W, F0 = self._matrices(v)
        y = y.double()
        m, C = (m0.double() if m0 is not None else torch.zeros(self.n, dtype=torch.float64)), torch.eye(self.n, dtype=torch.float64) * c0
        ms, Cs, as_, Rs, ll, preds, pvars = [], [], [], [], 0.0, [], []
        for t in range(len(y)):
            F = F0.clone()
            if self.k:
                F[self.n - self.k:] = X[t].double()
            a, R = G @ m, G @ C @ G.T + W
            f, q = F @ a, F @ R @ F + v["obs"]
            preds.append(f); pvars.append(q)
            if not torch.isnan(y[t]):
                e = y[t] - f
                A = R @ F / q
                m, C = a + A * e, R - torch.outer(A, A) * q
                ll = ll - 0.5 * (torch.log(2 * math.pi * q) + e * e / q)
            else:
                m, C = a, R
            ms.append(m); Cs.append(C); as_.append(a); Rs.append(R)
        return {"m": torch.stack(ms), "C": torch.stack(Cs), "a": torch.stack(as_), "R": torch.stack(Rs), "loglik": ll, "pred": torch.stack(preds), "pred_var": torch.stack(pvars), "G": G, "F": F0}

    def smooth(self, filt: dict) -> dict:
        m, C, a, R, G = filt["m"], filt["C"], filt["a"], filt["R"], filt["G"]
        sm, sC = [m[-1]], [C[-1]]
        for t in range(len(m) - 2, -1, -1):
            B = C[t] @ G.T @ torch.linalg.inv(R[t + 1])
            sm.insert(0, m[t] + B @ (sm[0] - a[t + 1])); sC.insert(0, C[t] + B @ (sC[0] - R[t + 1]) @ B.T)
        s = torch.stack(sm)
        out = {"state": s, "cov": torch.stack(sC), "level": s[:, 0]}
        if self.order > 1:
            out["slope"] = s[:, 1]
        if self.s:
            out["seasonal"] = s[:, self.order]
        return out

    def forecast(self, filt: dict, steps: int, X_future: torch.Tensor | None = None, z: float = 1.96) -> dict:
        G, W, F0 = self._matrices()
        m, C = filt["m"][-1], filt["C"][-1]
        mean, var = [], []
        for h in range(steps):
            m, C = G @ m, G @ C @ G.T + W
            F = F0.clone()
            if self.k:
                F[self.n - self.k:] = X_future[h].double()
            mean.append(F @ m); var.append(F @ C @ F + self.vars["obs"])
        mean, sd = torch.stack(mean), torch.stack(var).sqrt()
        return {"mean": mean, "lower": mean - z * sd, "upper": mean + z * sd, "std": sd}

    def fit(self, y: torch.Tensor, X: torch.Tensor | None = None, steps: int = 60, burn_in: int | None = None) -> dict:
        """Maximum-likelihood variances (log-parameterised, L-BFGS); the first ``burn_in`` observations, which only resolve the
        diffuse prior, are left out of the likelihood."""
        names = ["obs", "level"] + (["slope"] if self.order > 1 else []) + (["seasonal"] if self.s else [])
        scale = float(torch.nan_to_num(y.double()).var()) or 1.0
        theta = torch.tensor([math.log(max(self.vars[n], 1e-8) * 1.0) for n in names], dtype=torch.float64, requires_grad=True)
        burn = self.n if burn_in is None else burn_in
        opt = torch.optim.LBFGS([theta], max_iter=steps, line_search_fn="strong_wolfe")
        def nll():
            v = {**self.vars, **{n: torch.exp(theta[i]) for i, n in enumerate(names)}}
            G, W, F0 = self._matrices(v)
            m, C, ll = torch.zeros(self.n, dtype=torch.float64), torch.eye(self.n, dtype=torch.float64) * 1e6, 0.0
            yy = y.double()
            for t in range(len(yy)):
                F = F0.clone()
                if self.k:
                    F[self.n - self.k:] = X[t].double()
                a, R = G @ m, G @ C @ G.T + W
                f, q = F @ a, F @ R @ F + v["obs"]
                e = yy[t] - f
                A = R @ F / q
                m, C = a + A * e, R - torch.outer(A, A) * q
                if t >= burn:
                    ll = ll - 0.5 * (torch.log(2 * math.pi * q) + e * e / q)
            return -ll
        def closure():
            opt.zero_grad(); l = nll(); l.backward(); return l
        opt.step(closure)
        for i, n in enumerate(names):
            self.vars[n] = float(torch.exp(theta[i].detach()))
        return {"variances": dict(self.vars), "neg_loglik": float(nll().detach()), "signal_to_noise": self.vars["level"] / self.vars["obs"], "data_variance": scale}
