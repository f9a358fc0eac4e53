"""Class-style time-series models (``crates/torsh-series/src/{timeseries,multivariate,forecasting,decomposition,
frequency,imputation,validation,anomaly,detection}.rs``).

New here: a ``TimeSeries`` container, vector autoregression with impulse responses and variance decomposition, the
Johansen cointegration test and the vector error-correction model built on it, Engle-Granger and Phillips-Perron tests,
X-11 style decomposition with Henderson filters, chained-equation imputation, continuous wavelet analysis, Welch spectral
density and magnitude-squared coherence, multi-level wavelet decomposition, conditional transfer entropy, purged /
combinatorial / blocked / nested cross-validation and a recurrent forecaster used as an anomaly detector.  The remaining
classes give the estimator interface (``fit`` / ``forecast`` / ``decompose`` / ``detect``) over the function-style
implementations in ``series`` and ``series_ext``.  Everything runs on whatever device the input tensor lives on; the
estimation algebra is float64."""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass, field

import torch
from torch import nn

from . import series as _s
from . import series_ext as _e

__all__ = [
    "TimeSeries", "VAR", "JohansenResult", "johansen_test", "VECM", "EngleGrangerResult", "engle_granger",
    "PPResult", "phillips_perron", "henderson_weights", "X11Decomposition", "AdditiveDecomposition",
    "MultiplicativeDecomposition", "STLDecomposition", "MSTLDecomposition", "SSA", "MICEImputer", "TimeSeriesImputer",
    "ARIMA", "AutoARIMA", "SimpleExpSmoothing", "DoubleExpSmoothing", "HoltWinters", "PELT", "BinarySegmentation",
    "ChangePointDetector", "CWTAnalyzer", "PSDEstimator", "CoherenceAnalyzer", "FFTAnalyzer", "PeriodogramAnalyzer",
    "WaveletDecomposer", "WaveletPacketDecomposer", "ConditionalTransferEntropy", "TransferEntropyEstimator",
    "GrangerCausality", "StationarityTestSuite", "ResidualDiagnostics", "RollingStatistics", "OutlierDetector",
    "StatisticalDetector", "WindowDetector", "LSTMAnomaly", "BlockedTimeSeriesCV", "PurgedTimeSeriesCV",
    "CombinatorialPurgedCV", "NestedTimeSeriesCV", "ScoredTimeSeriesCV", "ForecastMetrics",
]


def _t(x) -> torch.Tensor:
    return torch.as_tensor(x, dtype=torch.float64) if not isinstance(x, torch.Tensor) else x.to(torch.float64)


# ================================================================================================ container
@dataclass
class TimeSeries:
    """Values ``(T,)`` or ``(T, k)`` with optional timestamps (seconds) and column names
    (``crates/torsh-series/src/timeseries.rs``)."""
    values: torch.Tensor
    timestamps: torch.Tensor | None = None
    names: list[str] | None = None
    frequency: float | None = None

    def __post_init__(self):
        self.values = torch.as_tensor(self.values)
        if self.timestamps is not None:
            self.timestamps = torch.as_tensor(self.timestamps, dtype=torch.float64)
            if len(self.timestamps) != len(self.values):
                raise ValueError("timestamps and values differ in length")

    def __len__(self): return len(self.values)
    @property
    def num_features(self) -> int: return 1 if self.values.dim() == 1 else self.values.shape[1]

    def slice(self, start: int, stop: int) -> "TimeSeries":
        return TimeSeries(self.values[start:stop], None if self.timestamps is None else self.timestamps[start:stop], self.names, self.frequency)

    def split(self, fraction: float) -> tuple["TimeSeries", "TimeSeries"]:
        k = int(len(self) * fraction)
        return self.slice(0, k), self.slice(k, len(self))

    def windows(self, size: int, horizon: int = 1, stride: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
        """Supervised pairs ``(inputs (N, size, ...), targets (N, horizon, ...))``."""
        v = self.values
        idx = range(0, len(v) - size - horizon + 1, stride)
        return torch.stack([v[i:i + size] for i in idx]), torch.stack([v[i + size:i + size + horizon] for i in idx])

    def resample(self, step: float, how: str = "mean") -> "TimeSeries":
        """Buckets of width ``step`` seconds aggregated by ``mean``, ``sum``, ``last`` or ``max``; empty buckets give NaN."""
        if self.timestamps is None:
            raise ValueError("resample needs timestamps")
        t0 = float(self.timestamps[0])
        bucket = ((self.timestamps - t0) / step).floor().long()
        nb = int(bucket.max()) + 1
        v = self.values.to(torch.float64).reshape(len(self), -1)
        out = torch.full((nb, v.shape[1]), float("nan"), dtype=torch.float64)
        for b in range(nb):
            sel = v[bucket == b]
            if len(sel):
                out[b] = {"mean": sel.mean(0), "sum": sel.sum(0), "last": sel[-1], "max": sel.max(0).values}[how]
        out = out.squeeze(1) if self.values.dim() == 1 else out
        return TimeSeries(out, t0 + step * torch.arange(nb, dtype=torch.float64), self.names, 1.0 / step)

    def lag(self, k: int) -> "TimeSeries":
        v = self.values.to(torch.float64)
        pad = torch.full_like(v[:k], float("nan"))
        return TimeSeries(torch.cat([pad, v[:-k]]) if k else v, self.timestamps, self.names, self.frequency)

    def diff(self, d: int = 1) -> "TimeSeries":
        v = self.values
        for _ in range(d):
            v = v[1:] - v[:-1]
        return TimeSeries(v, None if self.timestamps is None else self.timestamps[d:], self.names, self.frequency)


# ================================================================================================ multivariate
def _lagmat(y: torch.Tensor, p: int, const: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    T = len(y)
    cols = [y[p - l:T - l] for l in range(1, p + 1)]
    X = torch.cat(cols, 1)
    if const:
        X = torch.cat([torch.ones(T - p, 1, dtype=y.dtype, device=y.device), X], 1)
    return X, y[p:]


class VAR:
    """Vector autoregression ``y_t = c + A_1 y_{t-1} + ... + A_p y_{t-p} + u_t`` by equation-wise least squares
    (``crates/torsh-series/src/multivariate.rs``).  After ``fit``: ``coefs`` is ``(p, k, k)``, ``intercept`` ``(k,)``,
    ``sigma_u`` the residual covariance with the ``T - kp - 1`` degrees-of-freedom correction."""

    def __init__(self, lags: int = 1):
        self.p = lags

    def fit(self, y) -> "VAR":
        y = _t(y)
        X, Y = _lagmat(y, self.p)
        B = torch.linalg.lstsq(X, Y).solution
        self.k = y.shape[1]
        self.intercept = B[0]
        self.coefs = B[1:].reshape(self.p, self.k, self.k).transpose(1, 2)
        self.resid = Y - X @ B
        self.nobs = len(Y)
        self.sigma_u = self.resid.T @ self.resid / (self.nobs - self.k * self.p - 1)
        self.sigma_ml = self.resid.T @ self.resid / self.nobs
        self._tail = y[-self.p:]
        return self

    def information_criteria(self) -> dict:
        ld = float(torch.logdet(self.sigma_ml))
        m = self.k * (self.k * self.p + 1)
        T = self.nobs
        return {"aic": ld + 2 * m / T, "bic": ld + math.log(T) * m / T, "hqic": ld + 2 * math.log(math.log(T)) * m / T}

    @classmethod
    def select_order(cls, y, max_lags: int = 8, criterion: str = "aic") -> int:
        """Lag with the lowest criterion; every candidate is fitted on the same ``T - max_lags`` rows."""
        y = _t(y)
        best, arg = float("inf"), 1
        for p in range(1, max_lags + 1):
            m = cls(p).fit(y[max_lags - p:])
            v = m.information_criteria()[criterion]
            if v < best:
                best, arg = v, p
        return arg

    def forecast(self, steps: int, history=None) -> torch.Tensor:
        hist = list(self._tail if history is None else _t(history)[-self.p:])
        out = []
        for _ in range(steps):
            nxt = self.intercept + sum(self.coefs[l] @ hist[-1 - l] for l in range(self.p))
            out.append(nxt)
            hist.append(nxt)
        return torch.stack(out)

    def ma_representation(self, horizon: int) -> torch.Tensor:
        """``Phi_0 .. Phi_horizon`` with ``Phi_0 = I`` and ``Phi_i = sum_j Phi_{i-j} A_j``."""
        phi = [torch.eye(self.k, dtype=torch.float64)]
        for i in range(1, horizon + 1):
            phi.append(sum(phi[i - j] @ self.coefs[j - 1] for j in range(1, min(i, self.p) + 1)))
        return torch.stack(phi)

    def impulse_response(self, horizon: int = 10, orthogonal: bool = True) -> torch.Tensor:
        """``(horizon + 1, k, k)``: response of variable ``i`` to a shock in ``j``; orthogonalised by the Cholesky factor."""
        phi = self.ma_representation(horizon)
        return phi @ torch.linalg.cholesky(self.sigma_u) if orthogonal else phi

    def fevd(self, horizon: int = 10) -> torch.Tensor:
        """Forecast-error variance decomposition ``(horizon, k, k)``: rows sum to one."""
        theta = self.impulse_response(horizon - 1) ** 2
        cum = theta.cumsum(0)
        return cum / cum.sum(2, keepdim=True)

    def is_stable(self) -> bool:
        k, p = self.k, self.p
        comp = torch.zeros(k * p, k * p, dtype=torch.float64)
        comp[:k] = torch.cat(list(self.coefs), 1)
        if p > 1:
            comp[k:, :-k] = torch.eye(k * (p - 1), dtype=torch.float64)
        return bool(torch.linalg.eigvals(comp).abs().max() < 1)

    def test_causality(self, y, caused: int, causing: int) -> dict:
        """Wald F-test that every lag of ``causing`` has a zero coefficient in the equation of ``caused``."""
        y = _t(y)
        X, Y = _lagmat(y, self.p)
        keep = [0] + [1 + l * self.k + j for l in range(self.p) for j in range(self.k) if j != causing]
        full = Y[:, caused] - X @ torch.linalg.lstsq(X, Y[:, caused:caused + 1]).solution[:, 0]
        Xr = X[:, keep]
        restr = Y[:, caused] - Xr @ torch.linalg.lstsq(Xr, Y[:, caused:caused + 1]).solution[:, 0]
        df2 = len(Y) - X.shape[1]
        f = float(((restr ** 2).sum() - (full ** 2).sum()) / self.p / ((full ** 2).sum() / df2))
        from scipy import stats
        return {"f": f, "df": (self.p, df2), "p_value": float(stats.f.sf(f, self.p, df2))}



# Osterwald-Lenum / MacKinnon-Haug-Michelis 5 % critical values of the trace and maximum-eigenvalue statistics, constant
# restricted to the levels (the "constant" case), indexed by the number of common trends ``k - r`` (1..6).
_JOH_TRACE_95 = [3.8415, 15.4943, 29.7961, 47.8545, 69.8189, 95.7542]
_JOH_MAXEIG_95 = [3.8415, 14.2639, 21.1314, 27.5858, 33.8777, 40.0763]


@dataclass
class JohansenResult:
    eigenvalues: torch.Tensor
    eigenvectors: torch.Tensor          # columns = cointegrating vectors, normalised beta' S11 beta = I
    trace_stat: torch.Tensor
    max_eig_stat: torch.Tensor
    trace_crit_95: list
    max_eig_crit_95: list
    rank: int


def _joh_moments(y: torch.Tensor, k_ar_diff: int):
    dy = y[1:] - y[:-1]
    T = len(dy) - k_ar_diff
    Z0 = dy[k_ar_diff:]
    Z1 = y[k_ar_diff:-1]
    cols = [dy[k_ar_diff - l:len(dy) - l] for l in range(1, k_ar_diff + 1)]
    Z2 = torch.cat(cols + [torch.ones(T, 1, dtype=y.dtype)], 1)
    P = Z2 @ torch.linalg.pinv(Z2)
    R0, R1 = Z0 - P @ Z0, Z1 - P @ Z1
    return Z0, Z1, Z2, R0, R1, T


def johansen_test(y, k_ar_diff: int = 1) -> JohansenResult:
    """Reduced-rank regression of ``dy_t`` on ``y_{t-1}`` after partialling out a constant and ``k_ar_diff`` lagged
    differences; eigenvalues of ``S11^-1 S10 S00^-1 S01`` give the trace ``-T sum log(1 - lambda_i)`` and maximum-eigenvalue
    statistics; the rank is the first hypothesis the trace test does not reject at 5 %."""
    y = _t(y)
    k = y.shape[1]
    _, _, _, R0, R1, T = _joh_moments(y, k_ar_diff)
    S00, S11, S01 = R0.T @ R0 / T, R1.T @ R1 / T, R0.T @ R1 / T
    L = torch.linalg.cholesky(S11)
    Li = torch.linalg.inv(L)
    M = Li @ S01.T @ torch.linalg.solve(S00, S01) @ Li.T
    w, V = torch.linalg.eigh((M + M.T) / 2)
    order = torch.argsort(w, descending=True)
    w, V = w[order].clamp(0, 1 - 1e-12), V[:, order]
    beta = Li.T @ V
    logs = torch.log1p(-w)
    trace = torch.stack([-T * logs[r:].sum() for r in range(k)])
    maxeig = -T * logs
    tc = [_JOH_TRACE_95[k - r - 1] if k - r <= 6 else float("nan") for r in range(k)]
    mc = [_JOH_MAXEIG_95[k - r - 1] if k - r <= 6 else float("nan") for r in range(k)]
    rank = next((r for r in range(k) if not float(trace[r]) > tc[r]), k)
    return JohansenResult(w, beta, trace, maxeig, tc, mc, rank)


class VECM:
    """``dy_t = alpha beta' y_{t-1} + sum_i Gamma_i dy_{t-i} + c + u_t`` with ``beta`` from the Johansen eigenvectors and the
    rest by least squares given ``beta``."""

    def __init__(self, k_ar_diff: int = 1, coint_rank: int | None = None):
        self.k_ar_diff, self.rank = k_ar_diff, coint_rank

    def fit(self, y) -> "VECM":
        y = _t(y)
        jo = johansen_test(y, self.k_ar_diff)
        r = self.rank if self.rank is not None else max(jo.rank, 1)
        self.johansen, self.rank = jo, r
        beta = jo.eigenvectors[:, :r]
        self.beta = beta @ torch.linalg.inv(beta[:r])             # identified: the first r rows are the identity
        Z0, Z1, Z2, _, _, T = _joh_moments(y, self.k_ar_diff)
        X = torch.cat([Z1 @ self.beta, Z2], 1)
        B = torch.linalg.lstsq(X, Z0).solution
        k = y.shape[1]
        self.alpha = B[:r].T
        self.gamma = B[r:r + k * self.k_ar_diff].reshape(self.k_ar_diff, k, k).transpose(1, 2)
        self.const = B[-1]
        self.resid = Z0 - X @ B
        self.sigma_u = self.resid.T @ self.resid / T
        self._tail = y[-(self.k_ar_diff + 1):]
        return self

    def forecast(self, steps: int) -> torch.Tensor:
        hist = list(self._tail)
        out = []
        for _ in range(steps):
            dy = self.alpha @ (self.beta.T @ hist[-1]) + self.const
            for i in range(self.k_ar_diff):
                dy = dy + self.gamma[i] @ (hist[-1 - i] - hist[-2 - i])
            hist.append(hist[-1] + dy)
            out.append(hist[-1])
        return torch.stack(out)

    def to_var(self) -> torch.Tensor:
        """Level VAR matrices ``A_1 .. A_{p}`` with ``p = k_ar_diff + 1``."""
        k = self.alpha.shape[0]
        pi = self.alpha @ self.beta.T
        g = list(self.gamma)
        A = [torch.eye(k, dtype=torch.float64) + pi + (g[0] if g else 0)]
        for i in range(1, self.k_ar_diff):
            A.append(g[i] - g[i - 1])
        if g:
            A.append(-g[-1])
        return torch.stack(A)


@dataclass
class EngleGrangerResult:
    statistic: float
    critical_values: dict
    cointegrated: bool
    beta: torch.Tensor
    residuals: torch.Tensor


def engle_granger(y, x, lags: int = 1) -> EngleGrangerResult:
    """Two-step test: regress ``y`` on ``x`` and a constant, then an augmented Dickey-Fuller regression without constant
    on the residuals; critical values from MacKinnon's response surface for ``N = 1 + columns(x)`` variables."""
    y, x = _t(y), _t(x).reshape(len(y), -1)
    X = torch.cat([torch.ones(len(y), 1, dtype=torch.float64), x], 1)
    b = torch.linalg.lstsq(X, y[:, None]).solution[:, 0]
    e = y - X @ b
    de = e[1:] - e[:-1]
    cols = [e[lags:-1]] + [de[lags - l:len(de) - l] for l in range(1, lags + 1)]
    Z = torch.stack(cols, 1)
    t_y = de[lags:]
    coef = torch.linalg.lstsq(Z, t_y[:, None]).solution[:, 0]
    r = t_y - Z @ coef
    s2 = (r ** 2).sum() / (len(t_y) - Z.shape[1])
    se = torch.sqrt(s2 * torch.linalg.inv(Z.T @ Z)[0, 0])
    stat = float(coef[0] / se)
    n = x.shape[1] + 1
    T = len(t_y)
    surf = {2: {"1%": (-3.9001, -10.534, -30.03), "5%": (-3.3377, -5.967, -8.98), "10%": (-3.0462, -4.069, -5.73)},
            3: {"1%": (-4.2981, -13.790, -46.37), "5%": (-3.7429, -8.352, -13.41), "10%": (-3.4518, -6.241, -2.79)},
            4: {"1%": (-4.6493, -17.188, -59.20), "5%": (-4.1000, -10.745, -21.57), "10%": (-3.8110, -8.317, -5.19)}}[min(max(n, 2), 4)]
    crit = {k: a + b1 / T + b2 / T ** 2 for k, (a, b1, b2) in surf.items()}
    return EngleGrangerResult(stat, crit, stat < crit["5%"], b, e)


@dataclass
class PPResult:
    statistic: float
    rho_statistic: float
    critical_values: dict
    stationary: bool


def phillips_perron(x, lags: int | None = None) -> PPResult:
    """Dickey-Fuller regression with constant whose t-statistic is corrected non-parametrically with a Bartlett-kernel
    long-run variance (``Z_t`` and ``Z_rho``)."""
    x = _t(x)
    y, y1 = x[1:], x[:-1]
    T = len(y)
    X = torch.stack([torch.ones(T, dtype=torch.float64), y1], 1)
    XtXi = torch.linalg.inv(X.T @ X)
    b = XtXi @ X.T @ y
    u = y - X @ b
    s2 = float((u ** 2).sum() / (T - 2))
    se = math.sqrt(s2 * float(XtXi[1, 1]))
    q = lags if lags is not None else int(math.ceil(12 * (T / 100) ** 0.25))
    g0 = float((u ** 2).sum() / T)
    lam2 = g0 + 2 * sum((1 - j / (q + 1)) * float((u[j:] * u[:-j]).sum() / T) for j in range(1, q + 1))
    t_rho = float((b[1] - 1) / se)
    z_t = math.sqrt(g0 / lam2) * t_rho - 0.5 * (lam2 - g0) / math.sqrt(lam2) * T * se / math.sqrt(s2)
    z_rho = T * float(b[1] - 1) - 0.5 * T ** 2 * se ** 2 / s2 * (lam2 - g0)
    crit = {"1%": -3.43035 - 6.5393 / T - 16.786 / T ** 2, "5%": -2.86154 - 2.8903 / T - 4.234 / T ** 2, "10%": -2.56677 - 1.5384 / T - 2.809 / T ** 2}
    return PPResult(z_t, z_rho, crit, z_t < crit["5%"])


# ================================================================================================ decomposition
def henderson_weights(length: int) -> torch.Tensor:
    """Symmetric Henderson trend filter of odd ``length`` (closed form); reproduces cubic polynomials."""
    if length % 2 == 0:
        raise ValueError("Henderson filters have odd length")
    m = (length - 1) // 2
    n = m + 2
    j = torch.arange(-m, m + 1, dtype=torch.float64)
    num = 315 * ((n - 1) ** 2 - j ** 2) * (n ** 2 - j ** 2) * ((n + 1) ** 2 - j ** 2) * (3 * n ** 2 - 16 - 11 * j ** 2)
    den = 8 * n * (n ** 2 - 1) * (4 * n ** 2 - 1) * (4 * n ** 2 - 9) * (4 * n ** 2 - 25)
    return num / den


def _sym_filter(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Centred filter; at the ends the weights that fall off the series are dropped and the rest renormalised."""
    m = (len(w) - 1) // 2
    n = len(x)
    pad = torch.nn.functional.pad(x[None, None], (m, m))[0, 0]
    ones = torch.nn.functional.pad(torch.ones_like(x)[None, None], (m, m))[0, 0]
    k = w.flip(0)[None, None]
    num = torch.nn.functional.conv1d(pad[None, None], k)[0, 0]
    den = torch.nn.functional.conv1d(ones[None, None], k)[0, 0]
    return (num / den)[:n]


def _centered_ma(x: torch.Tensor, period: int) -> torch.Tensor:
    if period % 2:
        w = torch.full((period,), 1.0 / period, dtype=torch.float64)
    else:
        w = torch.full((period + 1,), 1.0 / period, dtype=torch.float64)
        w[0] = w[-1] = 0.5 / period
    return _sym_filter(x, w)


def _seasonal_ma(x: torch.Tensor, period: int, terms: int) -> torch.Tensor:
    """``3 x terms`` moving average along every phase of the season."""
    inner = torch.full((terms,), 1.0 / terms, dtype=torch.float64)
    w = torch.nn.functional.conv1d(torch.nn.functional.pad(inner[None, None], (2, 2)), torch.full((1, 1, 3), 1 / 3, dtype=torch.float64))[0, 0]
    out = torch.empty_like(x)
    for ph in range(period):
        out[ph::period] = _sym_filter(x[ph::period], w)
    return out


class X11Decomposition:
    """The X-11 iteration (``crates/torsh-series/src/decomposition.rs``): centred ``2 x period`` trend, ``3x3`` seasonal
    averages normalised by their own centred average, Henderson trend on the adjusted series, ``3x5`` seasonal averages,
    final Henderson trend.  ``mode`` is ``additive`` or ``multiplicative``."""

    def __init__(self, period: int, mode: str = "additive", henderson: int | None = None):
        self.period, self.mode = period, mode
        self.h = henderson or (13 if period >= 12 else 5 if period <= 4 else 2 * (period // 2) + 1)

    def decompose(self, x) -> dict:
        x = _t(x)
        mul = self.mode == "multiplicative"
        sub = (lambda a, b: a / b) if mul else (lambda a, b: a - b)
        hw = henderson_weights(self.h)
        trend = _centered_ma(x, self.period)
        si = sub(x, trend)
        seas = _seasonal_ma(si, self.period, 3)
        seas = sub(seas, _centered_ma(seas, self.period))
        adj = sub(x, seas)
        trend = _sym_filter(adj, hw)
        si = sub(x, trend)
        seas = _seasonal_ma(si, self.period, 5)
        seas = sub(seas, _centered_ma(seas, self.period))
        adj = sub(x, seas)
        trend = _sym_filter(adj, hw)
        irregular = sub(adj, trend)
        return {"trend": trend, "seasonal": seas, "irregular": irregular, "adjusted": adj}


class AdditiveDecomposition:
    def __init__(self, period: int): self.period = period
    def decompose(self, x) -> dict:
        d = _s.seasonal_decompose(_t(x), self.period)
        return {"trend": d.trend, "seasonal": d.seasonal, "residual": d.residual}


class MultiplicativeDecomposition:
    """``x = trend * seasonal * residual`` for positive series: additive decomposition of the logarithm."""
    def __init__(self, period: int): self.period = period
    def decompose(self, x) -> dict:
        x = _t(x)
        if bool((x <= 0).any()):
            raise ValueError("multiplicative decomposition needs a positive series")
        d = _s.seasonal_decompose(x.log(), self.period)
        return {"trend": d.trend.exp(), "seasonal": d.seasonal.exp(), "residual": d.residual.exp()}


class STLDecomposition:
    def __init__(self, period: int, seasonal: int = 7, trend: int | None = None, robust: bool = False):
        self.kw = dict(period=period, seasonal=seasonal, trend=trend, robust=robust)
    def decompose(self, x) -> dict: return _e.stl(x, **self.kw)


class MSTLDecomposition:
    def __init__(self, periods: list[int]): self.periods = list(periods)
    def decompose(self, x) -> dict:
        trend, seas, rem = _s.mstl(_t(x), self.periods)
        return {"trend": trend, "seasonal": dict(zip(sorted(self.periods), seas)), "residual": rem}


class SSA:
    """Singular-spectrum analysis with explicit components: ``fit`` keeps the elementary series, ``reconstruct`` sums a
    group, ``forecast`` uses the linear recurrence of the leading subspace."""

    def __init__(self, window: int): self.L = window

    def fit(self, x) -> "SSA":
        x = _t(x)
        n, L = len(x), self.L
        K = n - L + 1
        H = torch.stack([x[i:i + K] for i in range(L)])
        U, S, Vh = torch.linalg.svd(H, full_matrices=False)
        self.U, self.S, self.x = U, S, x
        comps = []
        cnt = torch.zeros(n, dtype=torch.float64)
        for i in range(L):
            cnt[i:i + K] += 1
        for r in range(len(S)):
            M = S[r] * U[:, r:r + 1] @ Vh[r:r + 1]
            s = torch.zeros(n, dtype=torch.float64)
            for i in range(L):
                s[i:i + K] += M[i]
            comps.append(s / cnt)
        self.components = torch.stack(comps)
        return self

    def explained(self) -> torch.Tensor: return self.S ** 2 / (self.S ** 2).sum()
    def reconstruct(self, group) -> torch.Tensor: return self.components[list(group)].sum(0)

    def forecast(self, steps: int, rank: int) -> torch.Tensor:
        U = self.U[:, :rank]
        pi = U[-1]
        nu2 = float((pi ** 2).sum())
        R = (U[:-1] @ pi) / (1 - nu2)
        series = list(self.reconstruct(range(rank)))
        for _ in range(steps):
            series.append(sum(R[j] * series[len(series) - self.L + 1 + j] for j in range(self.L - 1)))
        return torch.stack(series[-steps:])


# ================================================================================================ imputation
class MICEImputer:
    """Multivariate imputation by chained equations (``crates/torsh-series/src/imputation.rs``): every column with gaps is
    regressed (ridge) on the others, cycling ``iters`` times from a column-mean start; ``sample=True`` adds residual noise
    so that repeated runs give multiple imputations."""

    def __init__(self, iters: int = 10, ridge: float = 1e-6, sample: bool = False, seed: int = 0):
        self.iters, self.ridge, self.sample, self.gen = iters, ridge, sample, torch.Generator().manual_seed(seed)

    def fit_transform(self, X) -> torch.Tensor:
        X = _t(X).clone()
        miss = torch.isnan(X)
        means = torch.nanmean(X, 0)
        X[miss] = means.expand_as(X)[miss]
        order = sorted((j for j in range(X.shape[1]) if miss[:, j].any()), key=lambda j: int(miss[:, j].sum()))
        for _ in range(self.iters):
            for j in order:
                obs = ~miss[:, j]
                others = [c for c in range(X.shape[1]) if c != j]
                A = torch.cat([torch.ones(len(X), 1, dtype=torch.float64), X[:, others]], 1)
                G = A[obs].T @ A[obs] + self.ridge * torch.eye(A.shape[1], dtype=torch.float64)
                w = torch.linalg.solve(G, A[obs].T @ X[obs, j])
                pred = A[~obs] @ w
                if self.sample:
                    sd = (X[obs, j] - A[obs] @ w).std()
                    pred = pred + sd * torch.randn(pred.shape, generator=self.gen, dtype=torch.float64)
                X[~obs, j] = pred
        return X


class TimeSeriesImputer:
    def __init__(self, method: str = "linear", period: int | None = None): self.method, self.period = method, period
    def fit_transform(self, x) -> torch.Tensor:
        x = _t(x)
        if x.dim() == 2:
            return torch.stack([_e.impute(x[:, j], self.method, self.period) for j in range(x.shape[1])], 1)
        return _e.impute(x, self.method, self.period)


# ================================================================================================ forecasting facades
class ARIMA:
    def __init__(self, p: int = 1, d: int = 0, q: int = 0, seasonal_order=(0, 0, 0, 0)):
        self.model = _e.SARIMA((p, d, q), seasonal_order)
    def fit(self, x) -> "ARIMA":
        self.model.fit(_t(x))
        return self
    def forecast(self, steps: int) -> torch.Tensor: return self.model.forecast(steps)
    def __getattr__(self, name): return getattr(self.__dict__["model"], name)


class AutoARIMA:
    def __init__(self, max_p: int = 3, max_q: int = 3, max_d: int = 2, seasonal_period: int = 0, criterion: str = "aic"):
        self.kw = dict(max_p=max_p, max_q=max_q, max_d=max_d, seasonal_period=seasonal_period, criterion=criterion)
    def fit(self, x) -> "AutoARIMA":
        self.model = _e.auto_arima(x, **self.kw)
        self.order = self.model.order
        return self
    def forecast(self, steps: int) -> torch.Tensor: return self.model.forecast(steps)


def _golden(f, lo=0.01, hi=0.99, iters=40):
    g = (math.sqrt(5) - 1) / 2
    a, b = lo, hi
    c, d = b - g * (b - a), a + g * (b - a)
    fc, fd = f(c), f(d)
    for _ in range(iters):
        if fc < fd:
            b, d, fd = d, c, fc
            c = b - g * (b - a)
            fc = f(c)
        else:
            a, c, fc = c, d, fd
            d = a + g * (b - a)
            fd = f(d)
    return (a + b) / 2


class SimpleExpSmoothing:
    """Level-only smoothing; ``alpha=None`` picks it by minimising the one-step squared error."""
    def __init__(self, alpha: float | None = None): self.alpha = alpha

    def _run(self, x, a):
        level, sse = float(x[0]), 0.0
        for v in x[1:].tolist():
            sse += (v - level) ** 2
            level += a * (v - level)
        return level, sse

    def fit(self, x) -> "SimpleExpSmoothing":
        x = _t(x)
        if self.alpha is None:
            self.alpha = _golden(lambda a: self._run(x, a)[1])
        self.level, self.sse = self._run(x, self.alpha)
        return self

    def forecast(self, steps: int) -> torch.Tensor: return torch.full((steps,), self.level, dtype=torch.float64)


class DoubleExpSmoothing:
    """Holt's linear trend, optionally damped by ``phi``."""
    def __init__(self, alpha: float = 0.5, beta: float = 0.1, phi: float = 1.0): self.alpha, self.beta, self.phi = alpha, beta, phi

    def fit(self, x) -> "DoubleExpSmoothing":
        x = _t(x).tolist()
        level, trend, sse = x[0], x[1] - x[0], 0.0
        for v in x[1:]:
            pred = level + self.phi * trend
            sse += (v - pred) ** 2
            new = self.alpha * v + (1 - self.alpha) * pred
            trend = self.beta * (new - level) + (1 - self.beta) * self.phi * trend
            level = new
        self.level, self.trend, self.sse = level, trend, sse
        return self

    def forecast(self, steps: int) -> torch.Tensor:
        damp = torch.cumsum(torch.tensor([self.phi ** h for h in range(1, steps + 1)], dtype=torch.float64), 0)
        return self.level + damp * self.trend


class HoltWinters:
    """Triple exponential smoothing, additive or multiplicative season; ``fit(optimize=True)`` tunes the three smoothing
    constants by coordinate-wise golden-section search on the one-step squared error."""

    def __init__(self, period: int, alpha: float = 0.3, beta: float = 0.05, gamma: float = 0.1, seasonal: str = "additive"):
        self.period, self.alpha, self.beta, self.gamma, self.seasonal = period, alpha, beta, gamma, seasonal

    def _run(self, x, a, b, g):
        m, mul = self.period, self.seasonal == "multiplicative"
        mean0 = sum(x[:m]) / m
        trend = (sum(x[m:2 * m]) - sum(x[:m])) / m / m
        line = [mean0 + (i - (m - 1) / 2) * trend for i in range(m)]          # the first season's trend line
        season = [(v / l if mul else v - l) for v, l in zip(x[:m], line)]
        level = line[0] - trend                                                # level just before the first sample
        sse, fitted = 0.0, []
        for t, v in enumerate(x):
            s = season[t % m]
            pred = (level + trend) * s if mul else level + trend + s
            fitted.append(pred)
            sse += (v - pred) ** 2
            new = a * (v / s if mul else v - s) + (1 - a) * (level + trend)
            trend = b * (new - level) + (1 - b) * trend
            season[t % m] = g * (v / new if mul else v - new) + (1 - g) * s
            level = new
        return level, trend, season, sse, fitted

    def fit(self, x, optimize: bool = False) -> "HoltWinters":
        xs = _t(x).tolist()
        if optimize:
            p = [self.alpha, self.beta, self.gamma]
            for _ in range(3):
                for i in range(3):
                    p[i] = _golden(lambda v: self._run(xs, *(p[:i] + [v] + p[i + 1:]))[3], 0.001, 0.999, 25)
            self.alpha, self.beta, self.gamma = p
        self.level, self.trend, self.season, self.sse, fitted = self._run(xs, self.alpha, self.beta, self.gamma)
        self.fitted, self.n = torch.tensor(fitted, dtype=torch.float64), len(xs)
        return self

    def forecast(self, steps: int) -> torch.Tensor:
        mul = self.seasonal == "multiplicative"
        out = []
        for h in range(1, steps + 1):
            s = self.season[(self.n + h - 1) % self.period]
            base = self.level + h * self.trend
            out.append(base * s if mul else base + s)
        return torch.tensor(out, dtype=torch.float64)


# ================================================================================================ change points
class PELT:
    def __init__(self, penalty: float | None = None, min_size: int = 2, cost: str = "mean"): self.kw = dict(penalty=penalty, min_size=min_size, cost=cost)
    def detect(self, x) -> list[int]: return _e.pelt(x, **self.kw)


class BinarySegmentation:
    def __init__(self, max_changes: int = 5, penalty: float | None = None): self.max_changes, self.penalty = max_changes, penalty
    def detect(self, x) -> list[int]: return sorted(_s.binary_segmentation(_t(x), self.max_changes, penalty=self.penalty))


class ChangePointDetector:
    """``method`` in ``pelt``, ``binseg``, ``cusum``; ``detect`` returns the change indices and per-segment means."""
    def __init__(self, method: str = "pelt", **kw): self.method, self.kw = method, kw

    def detect(self, x) -> dict:
        x = _t(x)
        if self.method == "pelt":
            cps = PELT(**self.kw).detect(x)
        elif self.method == "binseg":
            cps = BinarySegmentation(**self.kw).detect(x)
        else:
            cps = list(_s.cusum(x, **self.kw))
        cps = [int(c) for c in cps]
        edges = [0] + cps + [len(x)]
        return {"change_points": cps, "segment_means": [float(x[a:b].mean()) for a, b in zip(edges[:-1], edges[1:]) if b > a]}


# ================================================================================================ frequency domain
class FFTAnalyzer:
    def __init__(self, fs: float = 1.0, window: str | None = "hann", detrend: bool = True): self.fs, self.window, self.detrend = fs, window, detrend

    def analyze(self, x) -> dict:
        x = _t(x)
        if self.detrend:
            x = x - x.mean()
        w = torch.hann_window(len(x), periodic=False, dtype=torch.float64) if self.window == "hann" else torch.ones(len(x), dtype=torch.float64)
        spec = torch.fft.rfft(x * w)
        freqs = torch.fft.rfftfreq(len(x), 1 / self.fs).to(torch.float64)
        amp = spec.abs() * 2 / w.sum()
        k = int(torch.argmax(amp[1:])) + 1
        return {"freqs": freqs, "amplitude": amp, "phase": torch.angle(spec), "dominant_frequency": float(freqs[k]), "dominant_amplitude": float(amp[k])}


class PeriodogramAnalyzer:
    def __init__(self, fs: float = 1.0): self.fs = fs
    def analyze(self, x) -> dict:
        f, p = _s.periodogram(_t(x).float(), self.fs)
        return {"freqs": f, "power": p, "dominant_period": _s.dominant_period(_t(x).float()), "spectral_entropy": _s.spectral_entropy(_t(x).float())}


def _segments(x: torch.Tensor, nperseg: int, noverlap: int, win: torch.Tensor) -> torch.Tensor:
    step = nperseg - noverlap
    segs = x.unfold(0, nperseg, step)
    segs = segs - segs.mean(1, keepdim=True)
    return torch.fft.rfft(segs * win, dim=1)


class PSDEstimator:
    """Welch's averaged, Hann-windowed, mean-detrended periodogram with one-sided density scaling."""
    def __init__(self, fs: float = 1.0, nperseg: int = 256, noverlap: int | None = None):
        self.fs, self.nperseg, self.noverlap = fs, nperseg, nperseg // 2 if noverlap is None else noverlap

    def estimate(self, x) -> tuple[torch.Tensor, torch.Tensor]:
        x = _t(x)
        n = min(self.nperseg, len(x))
        win = torch.hann_window(n, periodic=True, dtype=torch.float64)
        S = _segments(x, n, min(self.noverlap, n - 1), win)
        p = (S.abs() ** 2).mean(0) / (self.fs * (win ** 2).sum())
        p[1:-1 if n % 2 == 0 else None] *= 2
        return torch.fft.rfftfreq(n, 1 / self.fs).to(torch.float64), p


class CoherenceAnalyzer:
    """Magnitude-squared coherence ``|Pxy|^2 / (Pxx Pyy)`` from Welch cross- and auto-spectra; also the phase lag."""
    def __init__(self, fs: float = 1.0, nperseg: int = 256, noverlap: int | None = None):
        self.fs, self.nperseg, self.noverlap = fs, nperseg, nperseg // 2 if noverlap is None else noverlap

    def analyze(self, x, y) -> dict:
        x, y = _t(x), _t(y)
        n = min(self.nperseg, len(x))
        win = torch.hann_window(n, periodic=True, dtype=torch.float64)
        X, Y = _segments(x, n, self.noverlap, win), _segments(y, n, self.noverlap, win)
        pxy = (X.conj() * Y).mean(0)
        pxx, pyy = (X.abs() ** 2).mean(0), (Y.abs() ** 2).mean(0)
        return {"freqs": torch.fft.rfftfreq(n, 1 / self.fs).to(torch.float64), "coherence": pxy.abs() ** 2 / (pxx * pyy).clamp(min=1e-300), "phase": torch.angle(pxy)}


class CWTAnalyzer:
    """Continuous wavelet transform with the analytic Morlet wavelet (``omega0``), computed in the frequency domain for all
    scales at once; ``scale_to_frequency`` uses the Fourier factor of Torrence and Compo."""
    def __init__(self, omega0: float = 6.0, fs: float = 1.0): self.w0, self.fs = omega0, fs

    def scale_to_frequency(self, scales) -> torch.Tensor:
        return (self.w0 + math.sqrt(2 + self.w0 ** 2)) / (4 * math.pi * _t(scales)) * self.fs

    def frequency_to_scale(self, freqs) -> torch.Tensor:
        return (self.w0 + math.sqrt(2 + self.w0 ** 2)) / (4 * math.pi * _t(freqs)) * self.fs

    def transform(self, x, scales) -> torch.Tensor:
        x, s = _t(x), _t(scales)
        n = len(x)
        xf = torch.fft.fft(x - x.mean())
        om = 2 * math.pi * torch.fft.fftfreq(n).to(torch.float64)
        arg = s[:, None] * om[None]
        psi = math.pi ** -0.25 * torch.exp(-0.5 * (arg - self.w0) ** 2) * (om[None] > 0)
        psi = psi * torch.sqrt(2 * math.pi * s)[:, None]
        return torch.fft.ifft(xf[None] * psi, dim=1)

    def analyze(self, x, scales) -> dict:
        W = self.transform(x, scales)
        power = W.abs() ** 2
        glob = power.mean(1)
        return {"coefficients": W, "power": power, "global_spectrum": glob, "frequencies": self.scale_to_frequency(scales),
                "dominant_frequency": float(self.scale_to_frequency(scales)[int(torch.argmax(glob / _t(scales)))])}


_WAVELETS = {
    "haar": [1 / math.sqrt(2), 1 / math.sqrt(2)],
    "db2": [0.48296291314469025, 0.836516303737469, 0.22414386804185735, -0.12940952255092145],
    "db4": [0.23037781330885523, 0.7148465705525415, 0.6308807679295904, -0.02798376941698385, -0.18703481171888114,
            0.030841381835986965, 0.032883011666982945, -0.010597401784997278],
}


class WaveletDecomposer:
    """Multi-level orthogonal wavelet transform with periodic extension (exact reconstruction for lengths divisible by
    ``2 ** level``): ``decompose`` returns ``[approx_L, detail_L, ..., detail_1]``."""
    def __init__(self, wavelet: str = "db2", level: int = 3):
        h = torch.tensor(_WAVELETS[wavelet], dtype=torch.float64)
        self.h, self.level = h, level
        self.g = h.flip(0) * torch.tensor([(-1.0) ** k for k in range(len(h))], dtype=torch.float64)

    def _analysis(self, x, f):
        n, L = len(x), len(f)
        idx = (2 * torch.arange(n // 2)[:, None] + torch.arange(L)[None]) % n
        return (x[idx] * f[None]).sum(1)

    def _synthesis(self, a, d):
        n, L = 2 * len(a), len(self.h)
        out = torch.zeros(n, dtype=torch.float64)
        idx = (2 * torch.arange(len(a))[:, None] + torch.arange(L)[None]) % n
        out.index_add_(0, idx.reshape(-1), (a[:, None] * self.h[None] + d[:, None] * self.g[None]).reshape(-1))
        return out

    def decompose(self, x) -> list[torch.Tensor]:
        a, out = _t(x), []
        for _ in range(self.level):
            out.append(self._analysis(a, self.g))
            a = self._analysis(a, self.h)
        return [a] + out[::-1]

    def reconstruct(self, coeffs) -> torch.Tensor:
        a = coeffs[0]
        for d in coeffs[1:]:
            a = self._synthesis(a, d)
        return a

    def denoise(self, x, threshold: float | None = None) -> torch.Tensor:
        """Soft thresholding of the details with the universal threshold ``sigma sqrt(2 log n)`` (sigma from the finest MAD)."""
        c = self.decompose(x)
        if threshold is None:
            sigma = float(c[-1].abs().median()) / 0.6745
            threshold = sigma * math.sqrt(2 * math.log(len(_t(x))))
        return self.reconstruct([c[0]] + [torch.sign(d) * (d.abs() - threshold).clamp(min=0) for d in c[1:]])

    def energy_by_level(self, x) -> torch.Tensor:
        c = self.decompose(x)
        e = torch.stack([(v ** 2).sum() for v in c])
        return e / e.sum()


class WaveletPacketDecomposer:
    """Full binary tree of ``WaveletDecomposer`` steps; leaves keyed by their path of ``a`` / ``d``; ``best_basis`` prunes
    by Shannon entropy."""
    def __init__(self, wavelet: str = "db2", level: int = 3): self.w, self.level = WaveletDecomposer(wavelet, 1), level

    def decompose(self, x) -> dict[str, torch.Tensor]:
        nodes = {"": _t(x)}
        for _ in range(self.level):
            nodes = {k + s: v for k, n in nodes.items() for s, v in (("a", self.w._analysis(n, self.w.h)), ("d", self.w._analysis(n, self.w.g)))}
        return nodes

    def reconstruct(self, leaves: dict[str, torch.Tensor]) -> torch.Tensor:
        nodes = dict(leaves)
        while "" not in nodes:
            depth = max(len(k) for k in nodes)
            for k in [k for k in nodes if len(k) == depth and k.endswith("a")]:
                nodes[k[:-1]] = self.w._synthesis(nodes.pop(k), nodes.pop(k[:-1] + "d"))
        return nodes[""]

    @staticmethod
    def _entropy(v):
        p = v ** 2
        p = p[p > 0]
        return float(-(p * p.log()).sum())

    def best_basis(self, x) -> dict[str, torch.Tensor]:
        def rec(path, node, depth):
            if depth == self.level:
                return {path: node}, self._entropy(node)
            a, d = self.w._analysis(node, self.w.h), self.w._analysis(node, self.w.g)
            la, ea = rec(path + "a", a, depth + 1)
            ld, ed = rec(path + "d", d, depth + 1)
            own = self._entropy(node)
            return ({path: node}, own) if own <= ea + ed else ({**la, **ld}, ea + ed)
        return rec("", _t(x), 0)[0]


# ================================================================================================ causality and diagnostics
def _discretise(x: torch.Tensor, bins: int) -> torch.Tensor:
    q = torch.quantile(x, torch.linspace(0, 1, bins + 1, dtype=torch.float64)[1:-1])
    return torch.bucketize(x, q)


def _joint_entropy(*cols) -> float:
    code = torch.zeros_like(cols[0])
    for c in cols:
        code = code * (int(c.max()) + 1) + c
    p = torch.unique(code, return_counts=True)[1].double()
    p = p / p.sum()
    return float(-(p * p.log()).sum())


class ConditionalTransferEntropy:
    """``TE(X -> Y | Z) = H(Y+, Y, Z) + H(Y, X, Z) - H(Y+, Y, X, Z) - H(Y, Z)`` on quantile-binned series; removes the
    part of the coupling that a common driver ``Z`` explains."""
    def __init__(self, bins: int = 4, lag: int = 1): self.bins, self.lag = bins, lag

    def estimate(self, source, target, condition) -> float:
        x, y, z = (_discretise(_t(v), self.bins) for v in (source, target, condition))
        l = self.lag
        yp, y0, x0, z0 = y[l:], y[:-l], x[:-l], z[:-l]
        return _joint_entropy(yp, y0, z0) + _joint_entropy(y0, x0, z0) - _joint_entropy(yp, y0, x0, z0) - _joint_entropy(y0, z0)


class TransferEntropyEstimator:
    def __init__(self, bins: int = 4, lag: int = 1): self.bins, self.lag = bins, lag
    def estimate(self, source, target) -> float: return _e.transfer_entropy(source, target, bins=self.bins, lag=self.lag)
    def net_flow(self, a, b) -> float: return self.estimate(a, b) - self.estimate(b, a)


class GrangerCausality:
    def __init__(self, lags: int = 2): self.lags = lags
    def test(self, y, x) -> dict: return _e.granger_causality(y, x, self.lags)


class StationarityTestSuite:
    def run(self, x) -> dict:
        out = _e.stationarity_suite(x)
        pp = phillips_perron(x)
        out["pp"] = {"statistic": pp.statistic, "stationary": pp.stationary}
        return out


class ResidualDiagnostics:
    def __init__(self, lags: int = 10, fitted_params: int = 0): self.lags, self.fp = lags, fitted_params
    def run(self, resid) -> dict: return _e.residual_diagnostics(resid, self.lags, self.fp)


class RollingStatistics:
    def __init__(self, window: int): self.window = window
    def __getattr__(self, stat):
        if stat.startswith("_"):
            raise AttributeError(stat)
        return lambda x: _e.rolling(x, self.window, stat)
    def zscore(self, x) -> torch.Tensor:
        x = _t(x)
        return (x - _e.rolling(x, self.window, "mean")) / _e.rolling(x, self.window, "std").clamp(min=1e-12)


# ================================================================================================ anomaly detection
class OutlierDetector:
    def __init__(self, method: str = "hampel", window: int = 7, threshold: float = 3.0): self.kw = dict(method=method, window=window, threshold=threshold)
    def detect(self, x) -> torch.Tensor: return _e.detect_outliers(x, **self.kw)
    def treat(self, x, how: str = "interpolate") -> torch.Tensor: return _e.treat_outliers(x, self.detect(x), how)


class StatisticalDetector:
    """Global ``zscore``, ``iqr`` or ``mad`` rule."""
    def __init__(self, method: str = "zscore", threshold: float = 3.0): self.method, self.threshold = method, threshold

    def scores(self, x) -> torch.Tensor:
        x = _t(x)
        if self.method == "zscore":
            return (x - x.mean()).abs() / x.std().clamp(min=1e-12)
        if self.method == "mad":
            med = x.median()
            return 0.6745 * (x - med).abs() / (x - med).abs().median().clamp(min=1e-12)
        q1, q3 = torch.quantile(x, 0.25), torch.quantile(x, 0.75)
        return torch.maximum(q1 - x, x - q3).clamp(min=0) / (q3 - q1).clamp(min=1e-12)

    def detect(self, x) -> torch.Tensor:
        return self.scores(x) > (self.threshold if self.method != "iqr" else self.threshold / 2)


class WindowDetector:
    """Flags points whose distance from the trailing-window mean exceeds ``threshold`` trailing standard deviations
    (the window excludes the point itself)."""
    def __init__(self, window: int = 20, threshold: float = 3.0): self.window, self.threshold = window, threshold

    def detect(self, x) -> torch.Tensor:
        x = _t(x)
        out = torch.zeros(len(x), dtype=torch.bool)
        c1 = torch.cat([torch.zeros(1, dtype=torch.float64), x.cumsum(0)])
        c2 = torch.cat([torch.zeros(1, dtype=torch.float64), (x ** 2).cumsum(0)])
        w = self.window
        i = torch.arange(w, len(x))
        mean = (c1[i] - c1[i - w]) / w
        var = ((c2[i] - c2[i - w]) / w - mean ** 2).clamp(min=0) * w / (w - 1)
        out[w:] = (x[w:] - mean).abs() > self.threshold * var.sqrt().clamp(min=1e-12)
        return out


class LSTMAnomaly(nn.Module):
    """One-step-ahead recurrent forecaster; points whose forecast error exceeds ``threshold`` robust standard deviations
    of the training errors are anomalies (``crates/torsh-series/src/anomaly.rs``)."""

    def __init__(self, window: int = 16, hidden: int = 32, threshold: float = 4.0):
        super().__init__()
        self.window, self.threshold = window, threshold
        self.lstm = nn.LSTM(1, hidden, batch_first=True)
        self.head = nn.Linear(hidden, 1)
        self.register_buffer("center", torch.zeros(()))
        self.register_buffer("scale", torch.ones(()))
        self.register_buffer("err_scale", torch.ones(()))

    def forward(self, w: torch.Tensor) -> torch.Tensor:
        return self.head(self.lstm(w.unsqueeze(-1))[0][:, -1]).squeeze(-1)

    def _pairs(self, x):
        z = (x.float() - self.center) / self.scale
        W = z.unfold(0, self.window, 1)[:-1]
        return W, z[self.window:]

    def fit(self, x, epochs: int = 60, lr: float = 1e-2) -> "LSTMAnomaly":
        x = torch.as_tensor(x).float()
        self.center, self.scale = x.median(), (x - x.median()).abs().median().clamp(min=1e-6) * 1.4826
        W, y = self._pairs(x)
        opt = torch.optim.Adam(self.parameters(), lr=lr)
        for _ in range(epochs):
            opt.zero_grad()
            loss = torch.nn.functional.huber_loss(self(W), y)
            loss.backward()
            opt.step()
        with torch.no_grad():
            err = (self(W) - y).abs()
            self.err_scale = (err.median() * 1.4826).clamp(min=1e-6)
        return self

    @torch.no_grad()
    def scores(self, x) -> torch.Tensor:
        W, y = self._pairs(torch.as_tensor(x).float())
        s = torch.zeros(len(x))
        s[self.window:] = (self(W) - y).abs() / self.err_scale
        return s

    def detect(self, x) -> torch.Tensor: return self.scores(x) > self.threshold


# ================================================================================================ validation
class BlockedTimeSeriesCV:
    """Non-overlapping blocks, each split into its own train head and test tail, with ``gap`` samples between them."""
    def __init__(self, n_splits: int = 5, test_fraction: float = 0.2, gap: int = 0): self.n, self.f, self.gap = n_splits, test_fraction, gap

    def split(self, n: int):
        size = n // self.n
        for b in range(self.n):
            lo, hi = b * size, (b + 1) * size if b < self.n - 1 else n
            cut = hi - max(1, int((hi - lo) * self.f))
            yield list(range(lo, cut - self.gap)), list(range(cut, hi))


class PurgedTimeSeriesCV:
    """K contiguous test folds; training drops every sample whose label window ``[i, i + label_horizon]`` overlaps the
    test fold (purging) and the ``embargo`` samples that follow it."""
    def __init__(self, n_splits: int = 5, label_horizon: int = 0, embargo: int = 0): self.n, self.h, self.embargo = n_splits, label_horizon, embargo

    def _train_for(self, n: int, tests: list[tuple[int, int]]) -> list[int]:
        keep = [True] * n
        for lo, hi in tests:
            for i in range(max(0, lo - self.h), min(n, hi + self.embargo)):
                keep[i] = False
        return [i for i in range(n) if keep[i]]

    def folds(self, n: int) -> list[tuple[int, int]]:
        edges = [round(i * n / self.n) for i in range(self.n + 1)]
        return list(zip(edges[:-1], edges[1:]))

    def split(self, n: int):
        for lo, hi in self.folds(n):
            yield self._train_for(n, [(lo, hi)]), list(range(lo, hi))


class CombinatorialPurgedCV(PurgedTimeSeriesCV):
    """Every choice of ``n_test_groups`` out of ``n_splits`` groups is a test set: ``C(n, k)`` splits which recombine into
    ``C(n, k) k / n`` full back-test paths."""
    def __init__(self, n_splits: int = 6, n_test_groups: int = 2, label_horizon: int = 0, embargo: int = 0):
        super().__init__(n_splits, label_horizon, embargo)
        self.k = n_test_groups

    def split(self, n: int):
        folds = self.folds(n)
        for combo in itertools.combinations(range(self.n), self.k):
            tests = [folds[c] for c in combo]
            yield self._train_for(n, tests), [i for lo, hi in tests for i in range(lo, hi)]

    def num_paths(self) -> int: return math.comb(self.n, self.k) * self.k // self.n


class NestedTimeSeriesCV:
    """Outer expanding-window folds for the error estimate; inside every outer training part an inner expanding-window
    search picks the hyper-parameter."""
    def __init__(self, outer_splits: int = 3, inner_splits: int = 3): self.outer, self.inner = outer_splits, inner_splits

    def run(self, x, candidates: list, fit_forecast, metric=None) -> dict:
        x = _t(x)
        metric = metric or (lambda a, f: float(((a - f) ** 2).mean()))
        outer = _e.TimeSeriesCV(self.outer)
        chosen, scores = [], []
        for tr, te in outer.split(len(x)):
            xtr = x[tr]
            inner = _e.TimeSeriesCV(self.inner)
            best, arg = float("inf"), candidates[0]
            for c in candidates:
                s = sum(metric(xtr[ite], fit_forecast(xtr[itr], len(ite), c)) for itr, ite in inner.split(len(xtr))) / self.inner
                if s < best:
                    best, arg = s, c
            chosen.append(arg)
            scores.append(metric(x[te], fit_forecast(xtr, len(te), arg)))
        return {"chosen": chosen, "scores": scores, "mean_score": sum(scores) / len(scores)}


class ScoredTimeSeriesCV:
    def __init__(self, n_splits: int = 5, **kw): self.cv = _e.TimeSeriesCV(n_splits, **kw)
    def score(self, x, fit_forecast, metric=None) -> dict:
        s = self.cv.score(x, fit_forecast, metric)
        t = torch.tensor(s, dtype=torch.float64)
        return {"scores": s, "mean": float(t.mean()), "std": float(t.std()) if len(s) > 1 else 0.0}


@dataclass
class ForecastMetrics:
    values: dict = field(default_factory=dict)
    @classmethod
    def compute(cls, actual, forecast, train=None, period: int = 1) -> "ForecastMetrics":
        return cls(_e.forecast_metrics(actual, forecast, train, period))
    def __getitem__(self, k): return self.values[k]
