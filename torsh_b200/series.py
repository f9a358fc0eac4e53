"""Time series (``crates/torsh-series``): moving-average / STL-style decomposition, singular spectrum analysis, a linear
Kalman filter + RTS smoother, exponential smoothing (Holt-Winters), AR fitting and forecasting, and anomaly scores."""
from __future__ import annotations

from dataclasses import dataclass

import torch


def moving_average(x: torch.Tensor, window: int) -> torch.Tensor:
    pad_l, pad_r = (window - 1) // 2, window // 2
    xp = torch.cat([x[:1].expand(pad_l), x, x[-1:].expand(pad_r)])
    return torch.nn.functional.avg_pool1d(xp.reshape(1, 1, -1), window, 1).reshape(-1)


@dataclass
class Decomposition:
    trend: torch.Tensor
    seasonal: torch.Tensor
    residual: torch.Tensor


def seasonal_decompose(x: torch.Tensor, period: int, iters: int = 2) -> Decomposition:
    """Additive trend / seasonal / residual split; ``iters`` inner passes refine trend and seasonal alternately."""
    seasonal = torch.zeros_like(x)
    for _ in range(iters):
        trend = moving_average(x - seasonal, period if period % 2 else period + 1)
        det = x - trend
        means = torch.stack([det[i::period].mean() for i in range(period)])
        means = means - means.mean()
        seasonal = means.repeat(x.numel() // period + 1)[: x.numel()]
    return Decomposition(trend, seasonal, x - trend - seasonal)


def mstl(x: torch.Tensor, periods: list[int]) -> tuple[torch.Tensor, list[torch.Tensor], torch.Tensor]:
    seas, rem = [], x
    for p in sorted(periods):
        d = seasonal_decompose(rem, p)
        seas.append(d.seasonal)
        rem = rem - d.seasonal
    trend = moving_average(rem, max(periods) | 1)
    return trend, seas, rem - trend


def ssa(x: torch.Tensor, window: int, rank: int) -> torch.Tensor:
    """Rank-``rank`` singular-spectrum reconstruction (Hankel embedding, SVD, anti-diagonal averaging)."""
    n = x.numel()
    k = n - window + 1
    traj = x.unfold(0, window, 1).t()                       # [window, k]
    u, s, vh = torch.linalg.svd(traj, full_matrices=False)
    low = (u[:, :rank] * s[:rank]) @ vh[:rank]
    out, cnt = torch.zeros(n, dtype=x.dtype), torch.zeros(n, dtype=x.dtype)
    idx = torch.arange(window)[:, None] + torch.arange(k)[None]
    out.index_add_(0, idx.reshape(-1), low.reshape(-1))
    cnt.index_add_(0, idx.reshape(-1), torch.ones(window * k, dtype=x.dtype))
    return out / cnt


class KalmanFilter:
    """x' = F x + w (cov Q);  z = H x + v (cov R)."""

    def __init__(self, F, H, Q, R, x0=None, P0=None):
        self.F, self.H, self.Q, self.R = F, H, Q, R
        n = F.shape[0]
        self.x = torch.zeros(n, dtype=F.dtype) if x0 is None else x0
        self.P = torch.eye(n, dtype=F.dtype) if P0 is None else P0

    def predict(self):
        self.x = self.F @ self.x
        self.P = self.F @ self.P @ self.F.T + self.Q
        return self.x

    def update(self, z):
        S = self.H @ self.P @ self.H.T + self.R
        K = torch.linalg.solve(S, self.H @ self.P).T
        self.x = self.x + K @ (z - self.H @ self.x)
        self.P = (torch.eye(self.P.shape[0], dtype=self.P.dtype) - K @ self.H) @ self.P
        return self.x

    def filter(self, zs: torch.Tensor):
        xs, Ps, xp, Pp = [], [], [], []
        for z in zs:
            self.predict(); xp.append(self.x.clone()); Pp.append(self.P.clone())
            self.update(z); xs.append(self.x.clone()); Ps.append(self.P.clone())
        self._hist = (xs, Ps, xp, Pp)
        return torch.stack(xs)

    def smooth(self) -> torch.Tensor:
        xs, Ps, xp, Pp = self._hist
        out = [xs[-1]]
        for t in range(len(xs) - 2, -1, -1):
            C = Ps[t] @ self.F.T @ torch.linalg.inv(Pp[t + 1])
            out.append(xs[t] + C @ (out[-1] - xp[t + 1]))
        return torch.stack(out[::-1])


def holt_winters(x: torch.Tensor, period: int, alpha=0.3, beta=0.05, gamma=0.1, horizon: int = 0) -> torch.Tensor:
    level, trend = x[:period].mean(), (x[period:2 * period].mean() - x[:period].mean()) / period
    season = (x[:period] - level).clone()
    fitted = []
    for t in range(x.numel()):
        s = season[t % period]
        fitted.append(level + trend + s)
        new_level = alpha * (x[t] - s) + (1 - alpha) * (level + trend)
        trend = beta * (new_level - level) + (1 - beta) * trend
        season[t % period] = gamma * (x[t] - new_level) + (1 - gamma) * s
        level = new_level
    fc = [level + (h + 1) * trend + season[(x.numel() + h) % period] for h in range(horizon)]
    return torch.stack(fitted + fc)


def fit_ar(x: torch.Tensor, order: int) -> torch.Tensor:
    """Least-squares AR coefficients ``[c, a_1..a_p]`` with ``x_t = c + Σ a_i x_{t-i}``."""
    lags = torch.stack([x[order - i - 1: x.numel() - i - 1] for i in range(order)], 1)
    A = torch.cat([torch.ones(lags.shape[0], 1, dtype=x.dtype), lags], 1)
    return torch.linalg.lstsq(A, x[order:, None]).solution[:, 0]


def forecast_ar(x: torch.Tensor, coef: torch.Tensor, steps: int) -> torch.Tensor:
    p = coef.numel() - 1
    hist = x[-p:].tolist()
    out = []
    for _ in range(steps):
        v = coef[0].item() + sum(coef[i + 1].item() * hist[-i - 1] for i in range(p))
        out.append(v); hist.append(v)
    return torch.tensor(out, dtype=x.dtype)


def anomaly_zscore(x: torch.Tensor, period: int, thresh: float = 3.0) -> torch.Tensor:
    r = seasonal_decompose(x, period).residual
    return ((r - r.median()).abs() / (1.4826 * (r - r.median()).abs().median() + 1e-12)) > thresh


# ---- utilities (crates/torsh-series/src/utils) ------------------------------------------------------------------------
def difference(x: torch.Tensor, d: int = 1, season: int = 1) -> torch.Tensor:
    for _ in range(d):
        x = x[season:] - x[:-season]
    return x


def undifference(dx: torch.Tensor, head: torch.Tensor, season: int = 1) -> torch.Tensor:
    """Inverts one differencing step given the first ``season`` values of the original series."""
    out = list(head.tolist())
    for v in dx.tolist():
        out.append(v + out[-season])
    return torch.tensor(out, dtype=dx.dtype)


def acf(x: torch.Tensor, nlags: int) -> torch.Tensor:
    x = x.double() - x.double().mean()
    c0 = (x * x).sum()
    return torch.stack([(x[k:] * x[:len(x) - k]).sum() / c0 for k in range(nlags + 1)])


def pacf(x: torch.Tensor, nlags: int) -> torch.Tensor:
    """Partial autocorrelations by the Durbin-Levinson recursion."""
    r = acf(x, nlags)
    out, phi = [1.0], torch.zeros(0, dtype=torch.float64)
    for k in range(1, nlags + 1):
        num = r[k] - (phi * r[1:k].flip(0)).sum() if k > 1 else r[1]
        den = 1 - (phi * r[1:k]).sum() if k > 1 else torch.tensor(1.0, dtype=torch.float64)
        a = num / den
        phi = torch.cat([phi - a * phi.flip(0), a.reshape(1)]) if k > 1 else a.reshape(1)
        out.append(float(a))
    return torch.tensor(out, dtype=torch.float64)


# ---- frequency domain (frequency/) ---------------------------------------------------------------------------------------
def periodogram(x: torch.Tensor, fs: float = 1.0):
    x = x.double() - x.double().mean()
    spec = torch.fft.rfft(x).abs() ** 2 / (fs * len(x))
    spec[1:-1 if len(x) % 2 == 0 else None] *= 2
    return torch.fft.rfftfreq(len(x), 1 / fs).double(), spec


def dominant_period(x: torch.Tensor) -> float:
    f, p = periodogram(x)
    k = int(p[1:].argmax()) + 1
    return float(1 / f[k])


def spectral_entropy(x: torch.Tensor) -> float:
    _, p = periodogram(x)
    q = p[1:] / p[1:].sum()
    return float(-(q * torch.log(q.clamp(min=1e-300))).sum() / torch.log(torch.tensor(float(len(q)))))


# ---- change points (changepoint/) --------------------------------------------------------------------------------------
def cusum(x: torch.Tensor, threshold: float = 5.0, drift: float = 0.0):
    """Two-sided CUSUM on the standardised series; returns the indices where an alarm is raised (statistic reset after each)."""
    z = (x.double() - x.double().mean()) / x.double().std().clamp(min=1e-12)
    hi = lo = 0.0
    alarms = []
    for i, v in enumerate(z.tolist()):
        hi, lo = max(0.0, hi + v - drift), max(0.0, lo - v - drift)
        if hi > threshold or lo > threshold:
            alarms.append(i)
            hi = lo = 0.0
    return alarms


def binary_segmentation(x: torch.Tensor, max_changes: int = 5, min_size: int = 5, penalty: float | None = None):
    """Mean-shift change points by recursive splitting on the largest reduction of the squared error; a split is kept when
    the reduction exceeds ``penalty`` (default: 2 * variance * log n, the BIC-type penalty)."""
    x = x.double()
    n = len(x)
    pen = penalty if penalty is not None else 2 * float(x.var()) * torch.log(torch.tensor(float(n))).item() * 0.5
    cs, cs2 = torch.cat([torch.zeros(1, dtype=torch.float64), x.cumsum(0)]), torch.cat([torch.zeros(1, dtype=torch.float64), (x * x).cumsum(0)])
    sse = lambda a, b: float(cs2[b] - cs2[a] - (cs[b] - cs[a]) ** 2 / (b - a))
    segs, found = [(0, n)], []
    while len(found) < max_changes:
        best = None
        for a, b in segs:
            if b - a < 2 * min_size:
                continue
            base = sse(a, b)
            for t in range(a + min_size, b - min_size + 1):
                gain = base - sse(a, t) - sse(t, b)
                if best is None or gain > best[0]:
                    best = (gain, t, (a, b))
        if best is None or best[0] <= pen:
            break
        _, t, (a, b) = best
        found.append(t)
        segs.remove((a, b))
        segs += [(a, t), (t, b)]
    return sorted(found)


# ---- forecasting (forecast/) ---------------------------------------------------------------------------------------------
def seasonal_naive(x: torch.Tensor, horizon: int, season: int = 1) -> torch.Tensor:
    return torch.stack([x[len(x) - season + (h % season)] for h in range(horizon)])


def simple_exp_smoothing(x: torch.Tensor, alpha: float, horizon: int = 1) -> torch.Tensor:
    level = x[0]
    for v in x[1:]:
        level = alpha * v + (1 - alpha) * level
    return level.repeat(horizon)


def theta_forecast(x: torch.Tensor, horizon: int, alpha: float = 0.5) -> torch.Tensor:
    """Classical Theta method: average of the linear trend extrapolation (theta = 0) and simple exponential smoothing of
    the theta = 2 line."""
    n = len(x)
    t = torch.arange(n, dtype=x.dtype)
    slope = ((t - t.mean()) * (x - x.mean())).sum() / ((t - t.mean()) ** 2).sum()
    intercept = x.mean() - slope * t.mean()
    theta2 = 2 * x - (intercept + slope * t)
    ses = simple_exp_smoothing(theta2, alpha, 1)[0]
    h = torch.arange(n, n + horizon, dtype=x.dtype)
    return 0.5 * (intercept + slope * h) + 0.5 * (ses + 0 * h)


@dataclass
class ArimaModel:
    order: tuple
    const: float
    ar: torch.Tensor
    ma: torch.Tensor
    sigma2: float
    history: torch.Tensor
    residuals: torch.Tensor


def fit_arima(x: torch.Tensor, order=(1, 0, 0)) -> ArimaModel:
    """ARIMA(p, d, q) by the Hannan-Rissanen two-stage regression: a long autoregression estimates the innovations, then
    the differenced series is regressed on its own lags and the lagged innovations."""
    p, d, q = order
    x = x.double()
    y = difference(x, d) if d else x
    m = max(p, q)
    if q:
        L = min(max(10, 2 * (p + q)), len(y) // 3)
        A = torch.stack([y[L - k - 1:len(y) - k - 1] for k in range(L)], 1)
        A = torch.cat([torch.ones(len(A), 1, dtype=torch.float64), A], 1)
        coef = torch.linalg.lstsq(A, y[L:, None]).solution[:, 0]
        e = torch.cat([torch.zeros(L, dtype=torch.float64), y[L:] - A @ coef])
        start = L + m
    else:
        e, start = torch.zeros_like(y), m
    cols = [torch.ones(len(y) - start, dtype=torch.float64)]
    cols += [y[start - k:len(y) - k] for k in range(1, p + 1)]
    cols += [e[start - k:len(y) - k] for k in range(1, q + 1)]
    X = torch.stack(cols, 1)
    beta = torch.linalg.lstsq(X, y[start:, None]).solution[:, 0]
    res = y[start:] - X @ beta
    full_res = torch.cat([e[:start] if q else torch.zeros(start, dtype=torch.float64), res])
    return ArimaModel(order, float(beta[0]), beta[1:1 + p], beta[1 + p:], float(res.var()), x, full_res)


def forecast_arima(model: ArimaModel, horizon: int) -> torch.Tensor:
    p, d, q = model.order
    y = (difference(model.history, d) if d else model.history).tolist()
    e = model.residuals.tolist()
    out = []
    for _ in range(horizon):
        v = model.const + sum(float(model.ar[k]) * y[-k - 1] for k in range(p)) + sum(float(model.ma[k]) * e[-k - 1] for k in range(q))
        y.append(v)
        e.append(0.0)
        out.append(v)
    f = torch.tensor(out, dtype=torch.float64)
    for _ in range(d):                                   # integrate back, one differencing level at a time
        hist = model.history if d == 1 else difference(model.history, d - 1)
        f = hist[-1] + f.cumsum(0)
        d -= 1
    return f


# ---- anomalies ---------------------------------------------------------------------------------------------------------
def anomaly_iqr(x: torch.Tensor, k: float = 1.5) -> torch.Tensor:
    q1, q3 = torch.quantile(x.double(), torch.tensor([0.25, 0.75], dtype=torch.float64))
    return (x < q1 - k * (q3 - q1)) | (x > q3 + k * (q3 - q1))


def anomaly_seasonal_residual(x: torch.Tensor, period: int, z: float = 3.0) -> torch.Tensor:
    """Points whose residual after trend + seasonal removal is more than ``z`` robust standard deviations from zero."""
    r = seasonal_decompose(x, period).residual
    mad = (r - r.median()).abs().median() * 1.4826
    return (r - r.median()).abs() > z * mad.clamp(min=1e-12)
