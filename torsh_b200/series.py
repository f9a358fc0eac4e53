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
