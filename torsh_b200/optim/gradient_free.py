"""Optimizers that need no gradients (``crates/torsh-optim/src``: evolutionary, Bayesian and gradient-free modules):
Nelder-Mead simplex, a (μ/μ_w, λ) evolution strategy with step-size adaptation, random search and Bayesian optimisation
with a Gaussian-process surrogate and expected improvement. They minimise ``f(x)`` for a flat tensor ``x``; use
``torch.nn.utils.parameters_to_vector`` / ``vector_to_parameters`` to drive a module's parameters."""
from __future__ import annotations

import math

import torch


class RandomSearch:
    def __init__(self, x0: torch.Tensor, sigma: float = 0.5, seed: int = 0):
        self.best_x, self.best_f, self.sigma = x0.clone().float(), math.inf, sigma
        self.gen = torch.Generator().manual_seed(seed)

    def step(self, f, samples: int = 16) -> float:
        if self.best_f == math.inf:
            self.best_f = float(f(self.best_x))
        for _ in range(samples):
            x = self.best_x + self.sigma * torch.randn(self.best_x.shape, generator=self.gen)
            v = float(f(x))
            if v < self.best_f:
                self.best_x, self.best_f = x, v
        return self.best_f


class NelderMead:
    """Downhill simplex with the standard coefficients (reflection 1, expansion 2, contraction ½, shrink ½)."""

    def __init__(self, x0: torch.Tensor, step: float = 0.5):
        x0 = x0.clone().float().reshape(-1)
        n = x0.numel()
        self.simplex = [x0] + [x0 + step * torch.eye(n)[i] for i in range(n)]
        self.values: list[float] | None = None

    @property
    def best_x(self) -> torch.Tensor:
        return self.simplex[0]

    def step(self, f) -> float:
        if self.values is None:
            self.values = [float(f(x)) for x in self.simplex]
        order = sorted(range(len(self.simplex)), key=lambda i: self.values[i])
        self.simplex, self.values = [self.simplex[i] for i in order], [self.values[i] for i in order]
        centroid = torch.stack(self.simplex[:-1]).mean(0)
        worst = self.simplex[-1]
        xr = centroid + (centroid - worst)
        fr = float(f(xr))
        if fr < self.values[0]:
            xe = centroid + 2 * (centroid - worst)
            fe = float(f(xe))
            self.simplex[-1], self.values[-1] = (xe, fe) if fe < fr else (xr, fr)
        elif fr < self.values[-2]:
            self.simplex[-1], self.values[-1] = xr, fr
        else:
            xc = centroid + 0.5 * (worst - centroid)
            fc = float(f(xc))
            if fc < self.values[-1]:
                self.simplex[-1], self.values[-1] = xc, fc
            else:
                best = self.simplex[0]
                self.simplex = [best] + [best + 0.5 * (x - best) for x in self.simplex[1:]]
                self.values = [self.values[0]] + [float(f(x)) for x in self.simplex[1:]]
        i = min(range(len(self.values)), key=lambda j: self.values[j])
        self.simplex[0], self.simplex[i] = self.simplex[i], self.simplex[0]
        self.values[0], self.values[i] = self.values[i], self.values[0]
        return self.values[0]


class EvolutionStrategy:
    """(μ/μ_w, λ)-ES: λ Gaussian offspring around the mean, the best μ recombined with log weights, and the global step
    size adapted by the 1/5th-style success rule (grows when the best offspring beats the parent mean, shrinks otherwise)."""

    def __init__(self, x0: torch.Tensor, sigma: float = 0.5, population: int | None = None, seed: int = 0):
        self.mean, self.sigma = x0.clone().float().reshape(-1), sigma
        n = self.mean.numel()
        self.lam = population or 4 + int(3 * math.log(n + 1)) * 2
        self.mu = self.lam // 2
        w = torch.tensor([math.log(self.mu + 0.5) - math.log(i + 1) for i in range(self.mu)])
        self.w = w / w.sum()
        self.gen = torch.Generator().manual_seed(seed)
        self.best_x, self.best_f = self.mean.clone(), math.inf

    def step(self, f) -> float:
        z = torch.randn(self.lam, self.mean.numel(), generator=self.gen)
        xs = self.mean + self.sigma * z
        vals = torch.tensor([float(f(x)) for x in xs])
        order = vals.argsort()
        parent = float(f(self.mean))
        self.mean = (self.w[:, None] * xs[order[: self.mu]]).sum(0)
        self.sigma *= 1.2 if float(vals[order[0]]) < parent else 0.82
        if float(vals[order[0]]) < self.best_f:
            self.best_f, self.best_x = float(vals[order[0]]), xs[order[0]].clone()
        return self.best_f


class BayesianOptimizer:
    """Gaussian-process surrogate (RBF kernel, fixed length scale relative to the box) with expected improvement maximised
    over random candidates inside ``bounds`` (``[(lo, hi), ...]``)."""

    def __init__(self, bounds, length_scale: float = 0.2, noise: float = 1e-6, candidates: int = 512, seed: int = 0):
        self.lo = torch.tensor([b[0] for b in bounds], dtype=torch.float64)
        self.hi = torch.tensor([b[1] for b in bounds], dtype=torch.float64)
        self.ls, self.noise, self.ncand = length_scale, noise, candidates
        self.gen = torch.Generator().manual_seed(seed)
        self.X: list[torch.Tensor] = []
        self.y: list[float] = []

    def _unit(self, x):
        return (x - self.lo) / (self.hi - self.lo)

    def _k(self, a, b):
        return torch.exp(-0.5 * torch.cdist(a, b).pow(2) / self.ls ** 2)

    def suggest(self) -> torch.Tensor:
        d = self.lo.numel()
        cand = torch.rand(self.ncand, d, generator=self.gen, dtype=torch.float64)
        if len(self.X) < 2:
            return self.lo + cand[0] * (self.hi - self.lo)
        X = torch.stack([self._unit(x) for x in self.X])
        y = torch.tensor(self.y, dtype=torch.float64)
        mu0, sd0 = y.mean(), y.std().clamp(min=1e-9)
        yn = (y - mu0) / sd0
        K = self._k(X, X) + self.noise * torch.eye(len(X), dtype=torch.float64)
        L = torch.linalg.cholesky(K)
        alpha = torch.cholesky_solve(yn[:, None], L)
        Ks = self._k(cand, X)
        mean = (Ks @ alpha)[:, 0]
        v = torch.linalg.solve_triangular(L, Ks.t(), upper=False)
        var = (1.0 - (v * v).sum(0)).clamp(min=1e-12)
        sd = var.sqrt()
        best = yn.min()
        zed = (best - mean) / sd
        normal = torch.distributions.Normal(0.0, 1.0)
        ei = (best - mean) * normal.cdf(zed) + sd * torch.exp(normal.log_prob(zed))
        return self.lo + cand[ei.argmax()] * (self.hi - self.lo)

    def observe(self, x: torch.Tensor, value: float):
        self.X.append(x.double())
        self.y.append(float(value))

    def step(self, f) -> float:
        x = self.suggest()
        self.observe(x, float(f(x.float())))
        return min(self.y)

    @property
    def best_x(self) -> torch.Tensor:
        return self.X[min(range(len(self.y)), key=lambda i: self.y[i])].float()
