"""Further optimizers and optimizer tooling (``crates/torsh-optim/src``): names of the reference that differ only in spelling,
``AdvancedAdam``, ``ScheduleFreeAdamW``, ``Sophia`` (``adam.rs``, ``schedule_free.rs``, ``sophia.rs``); population
methods — CMA-ES, OpenAI-ES, particle swarm (``evolutionary_strategies.rs``, ``gradient_free.rs``); Gaussian-process regression
for Bayesian search (``bayesian_optimization.rs``); test functions, benchmarks and stress tests (``benchmarks.rs``,
``stress_tests.rs``, ``numerical_stability_tests.rs``); convergence tracking (``convergence.rs``); optimizers that react to carbon
intensity or a power budget (``green_optimizers.rs``), checkpoint-and-rollback and eligibility-trace wrappers
(``checkpointing.rs``, ``neuromorphic.rs``); builders and a task matcher (``builders.rs``, ``meta_learning.rs``)."""
from __future__ import annotations

import copy
import math
import time
from typing import Callable, Iterable, Sequence

import torch
from torch.optim import Optimizer

AdaDelta, AdaGrad, AdaMax = torch.optim.Adadelta, torch.optim.Adagrad, torch.optim.Adamax


# ================================================================================================ gradient-based
class AdvancedAdam(Optimizer):
    """Adam with the usual refinements as switches: decoupled weight decay, AMSGrad's running maximum, gradient
    centralisation (zero-mean gradients per output row of matrices), per-step clipping of the update and a warm-up of the
    second-moment bias correction."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False, centralize=False, max_update: float | None = None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad, centralize=centralize, max_update=max_update))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                if g["centralize"] and grad.dim() > 1:
                    grad = grad - grad.mean(tuple(range(1, grad.dim())), keepdim=True)
                st = self.state[p]
                if not st:
                    st.update(step=0, m=torch.zeros_like(p), v=torch.zeros_like(p), vmax=torch.zeros_like(p))
                st["step"] += 1
                st["m"].mul_(b1).add_(grad, alpha=1 - b1); st["v"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                v = st["v"]
                if g["amsgrad"]:
                    torch.maximum(st["vmax"], v, out=st["vmax"]); v = st["vmax"]
                upd = (st["m"] / (1 - b1 ** st["step"])) / ((v / (1 - b2 ** st["step"])).sqrt() + g["eps"])
                if g["max_update"] is not None:
                    upd.clamp_(-g["max_update"], g["max_update"])
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(upd, alpha=-g["lr"])
        return loss


class ScheduleFreeAdamW(Optimizer):
    """Schedule-free AdamW: gradients are taken at the interpolation ``y = (1 - beta1) z + beta1 x`` of the fast iterate ``z`` and
    the running average ``x``; no learning-rate schedule is needed.  The parameters hold ``y`` while training; ``eval_mode()`` swaps
    in the average ``x`` and ``train_mode()`` swaps back."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, warmup_steps=0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, warmup_steps=warmup_steps, k=0, lr_sum=0.0))
        self._training = True

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            g["k"] += 1
            sched = min(1.0, g["k"] / max(g["warmup_steps"], 1)) if g["warmup_steps"] else 1.0
            lr = g["lr"] * sched * math.sqrt(1 - b2 ** g["k"])
            g["lr_sum"] += lr ** 2
            ck = lr ** 2 / g["lr_sum"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st.update(z=p.detach().clone(), v=torch.zeros_like(p))
                st["v"].mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                d = p.grad / (st["v"].sqrt() + g["eps"]) + g["weight_decay"] * p
                p.lerp_(st["z"], ck)                                                # y moves toward z by c: x <- (1 - c) x + c z, expressed on y
                p.add_(d, alpha=lr * (b1 * (1 - ck) - 1))
                st["z"].sub_(d, alpha=lr)
        return loss

    @torch.no_grad()
    def _swap(self, to_average: bool):
        for g in self.param_groups:
            b1 = g["betas"][0]
            for p in g["params"]:
                st = self.state.get(p)
                if st:
                    p.lerp_(st["z"], 1 - 1 / b1) if to_average else p.lerp_(st["z"], 1 - b1)

    def eval_mode(self):
        if self._training:
            self._swap(True); self._training = False
    def train_mode(self):
        if not self._training:
            self._swap(False); self._training = True


def Sophia(params, **kw):
    """The reference's name for the Sophia-G optimizer."""
    from .extra import SophiaG
    return SophiaG(params, **kw)


# ================================================================================================ population methods
class CMAES:
    """Covariance matrix adaptation evolution strategy (rank-one and rank-mu updates, cumulative step-size adaptation) for
    ``minimise f(x)``, ``x`` in ``R^n``.  ``ask`` samples a population, ``tell`` ranks it and updates mean, step size and covariance."""

    def __init__(self, x0: torch.Tensor, sigma: float = 0.5, population: int | None = None, seed: int = 0):
        self.n = n = x0.numel()
        self.mean, self.sigma, self.g = x0.detach().double().flatten().clone(), sigma, torch.Generator().manual_seed(seed)
        self.lam = population or 4 + int(3 * math.log(n))
        self.mu = self.lam // 2
        w = math.log(self.mu + 0.5) - torch.log(torch.arange(1, self.mu + 1, dtype=torch.float64))
        self.w = w / w.sum()
        self.mueff = float(1 / (self.w ** 2).sum())
        self.cc, self.cs = (4 + self.mueff / n) / (n + 4 + 2 * self.mueff / n), (self.mueff + 2) / (n + self.mueff + 5)
        self.c1 = 2 / ((n + 1.3) ** 2 + self.mueff)
        self.cmu = min(1 - self.c1, 2 * (self.mueff - 2 + 1 / self.mueff) / ((n + 2) ** 2 + self.mueff))
        self.damps = 1 + 2 * max(0.0, math.sqrt((self.mueff - 1) / (n + 1)) - 1) + self.cs
        self.pc, self.ps, self.C = torch.zeros(n, dtype=torch.float64), torch.zeros(n, dtype=torch.float64), torch.eye(n, dtype=torch.float64)
        self.chi = math.sqrt(n) * (1 - 1 / (4 * n) + 1 / (21 * n * n))
        self.generation, self.best = 0, (math.inf, None)

    def ask(self) -> torch.Tensor:
        evals, vecs = torch.linalg.eigh(self.C)
        self._B, self._D = vecs, evals.clamp_min(1e-20).sqrt()
        self._z = torch.randn(self.lam, self.n, generator=self.g, dtype=torch.float64)
        self._y = (self._z * self._D) @ self._B.T
        return self.mean + self.sigma * self._y

    def tell(self, xs: torch.Tensor, fitness: torch.Tensor):
        order = fitness.argsort()
        if float(fitness[order[0]]) < self.best[0]:
            self.best = (float(fitness[order[0]]), xs[order[0]].clone())
        y = self._y[order[: self.mu]]
        yw = (self.w[:, None] * y).sum(0)
        self.mean = self.mean + self.sigma * yw
        inv_sqrt = self._B @ torch.diag(1 / self._D) @ self._B.T
        self.ps = (1 - self.cs) * self.ps + math.sqrt(self.cs * (2 - self.cs) * self.mueff) * (inv_sqrt @ yw)
        self.generation += 1
        hsig = float(self.ps.norm()) / math.sqrt(1 - (1 - self.cs) ** (2 * self.generation)) / self.chi < 1.4 + 2 / (self.n + 1)
        self.pc = (1 - self.cc) * self.pc + (math.sqrt(self.cc * (2 - self.cc) * self.mueff) * yw if hsig else 0)
        rank_mu = (self.w[:, None, None] * (y[:, :, None] * y[:, None, :])).sum(0)
        self.C = (1 - self.c1 - self.cmu) * self.C + self.c1 * (torch.outer(self.pc, self.pc) + (0 if hsig else self.cc * (2 - self.cc)) * self.C) + self.cmu * rank_mu
        self.C = (self.C + self.C.T) / 2
        self.sigma *= math.exp(self.cs / self.damps * (float(self.ps.norm()) / self.chi - 1))

    def minimize(self, f: Callable[[torch.Tensor], float], generations: int = 200, tol: float = 1e-12) -> dict:
        for _ in range(generations):
            xs = self.ask()
            self.tell(xs, torch.tensor([float(f(x)) for x in xs], dtype=torch.float64))
            if self.best[0] < tol or self.sigma < 1e-14:
                break
        return {"x": self.best[1], "value": self.best[0], "generations": self.generation, "sigma": self.sigma}


class OpenAIES:
    """Evolution strategy with antithetic Gaussian perturbations and rank-shaped returns; the search gradient feeds Adam."""

    def __init__(self, x0: torch.Tensor, sigma: float = 0.1, population: int = 50, lr: float = 0.05, seed: int = 0):
        self.x = x0.detach().double().clone().requires_grad_(True)
        self.sigma, self.pop, self.g, self.opt = sigma, population // 2 * 2, torch.Generator().manual_seed(seed), torch.optim.Adam([self.x], lr=lr)

    def step(self, f: Callable[[torch.Tensor], float]) -> float:
        eps = torch.randn(self.pop // 2, self.x.numel(), generator=self.g, dtype=torch.float64)
        eps = torch.cat([eps, -eps])
        vals = torch.tensor([float(f((self.x.detach() + self.sigma * e.view_as(self.x)))) for e in eps], dtype=torch.float64)
        ranks = vals.argsort().argsort().double() / (len(vals) - 1) - 0.5           # shaped: invariant to the scale of f
        self.x.grad = ((ranks[:, None] * eps).mean(0) / self.sigma).view_as(self.x)
        self.opt.step()
        return float(vals.min())

    def minimize(self, f, iterations: int = 200) -> dict:
        hist = [self.step(f) for _ in range(iterations)]
        return {"x": self.x.detach().clone(), "value": float(f(self.x.detach())), "history": hist}


class ParticleSwarmOptimizer:
    def __init__(self, dim: int, particles: int = 30, bounds: tuple[float, float] = (-5.0, 5.0), inertia: float = 0.7, cognitive: float = 1.5, social: float = 1.5, seed: int = 0):
        self.g = torch.Generator().manual_seed(seed)
        lo, hi = bounds
        self.bounds, self.w, self.c1, self.c2 = bounds, inertia, cognitive, social
        self.x = lo + (hi - lo) * torch.rand(particles, dim, generator=self.g, dtype=torch.float64)
        self.v = torch.zeros_like(self.x)
        self.pbest, self.pval = self.x.clone(), torch.full((particles,), math.inf, dtype=torch.float64)
        self.gbest, self.gval = self.x[0].clone(), math.inf

    def step(self, f: Callable[[torch.Tensor], float]):
        vals = torch.tensor([float(f(p)) for p in self.x], dtype=torch.float64)
        better = vals < self.pval
        self.pbest[better], self.pval[better] = self.x[better], vals[better]
        i = int(self.pval.argmin())
        if float(self.pval[i]) < self.gval:
            self.gval, self.gbest = float(self.pval[i]), self.pbest[i].clone()
        r1, r2 = torch.rand(self.x.shape, generator=self.g, dtype=torch.float64), torch.rand(self.x.shape, generator=self.g, dtype=torch.float64)
        self.v = self.w * self.v + self.c1 * r1 * (self.pbest - self.x) + self.c2 * r2 * (self.gbest - self.x)
        self.x = (self.x + self.v).clamp(*self.bounds)

    def minimize(self, f, iterations: int = 100) -> dict:
        for _ in range(iterations):
            self.step(f)
        return {"x": self.gbest, "value": self.gval}


# ================================================================================================ Gaussian process
class GaussianProcess:
    """Exact GP regression with an RBF kernel and observation noise: posterior mean and variance, log marginal likelihood
    and expected improvement for minimisation."""

    def __init__(self, length_scale: float = 1.0, signal_var: float = 1.0, noise_var: float = 1e-6): self.ls, self.sv, self.nv = length_scale, signal_var, noise_var
    def _k(self, a, b): return self.sv * torch.exp(-0.5 * torch.cdist(a / self.ls, b / self.ls) ** 2)

    def fit(self, x: torch.Tensor, y: torch.Tensor) -> "GaussianProcess":
        self.x, self.ymean = x.double(), float(y.double().mean())
        self.y = y.double() - self.ymean
        K = self._k(self.x, self.x) + self.nv * torch.eye(len(x), dtype=torch.float64)
        self.L = torch.linalg.cholesky(K)
        self.alpha = torch.cholesky_solve(self.y[:, None], self.L)[:, 0]
        return self

    def predict(self, xs: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        ks = self._k(xs.double(), self.x)
        v = torch.linalg.solve_triangular(self.L, ks.T, upper=False)
        return ks @ self.alpha + self.ymean, (self.sv - (v * v).sum(0)).clamp_min(1e-12)

    def log_marginal_likelihood(self) -> float: return float(-0.5 * self.y @ self.alpha - torch.log(self.L.diag()).sum() - 0.5 * len(self.y) * math.log(2 * math.pi))

    def expected_improvement(self, xs: torch.Tensor, xi: float = 0.0) -> torch.Tensor:
        mu, var = self.predict(xs)
        sd, best = var.sqrt(), float((self.y + self.ymean).min())
        z = (best - mu - xi) / sd
        n = torch.distributions.Normal(0.0, 1.0)
        return (best - mu - xi) * n.cdf(z) + sd * torch.exp(n.log_prob(z))


# ================================================================================================ test functions, benchmarks, stress
class Sphere:
    minimum, bounds = 0.0, (-5.12, 5.12)
    def __call__(self, x): return (x ** 2).sum()
    def optimum(self, n): return torch.zeros(n)


class Rosenbrock:
    minimum, bounds = 0.0, (-2.0, 2.0)
    def __call__(self, x): return (100 * (x[1:] - x[:-1] ** 2) ** 2 + (1 - x[:-1]) ** 2).sum()
    def optimum(self, n): return torch.ones(n)


class Rastrigin:
    minimum, bounds = 0.0, (-5.12, 5.12)
    def __call__(self, x): return 10 * x.numel() + (x ** 2 - 10 * torch.cos(2 * math.pi * x)).sum()
    def optimum(self, n): return torch.zeros(n)


class Branin:
    minimum, bounds = 0.39788735772973816, (-5.0, 15.0)
    def __call__(self, x):
        a, b, c, r, s, t = 1.0, 5.1 / (4 * math.pi ** 2), 5 / math.pi, 6.0, 10.0, 1 / (8 * math.pi)
        return a * (x[1] - b * x[0] ** 2 + c * x[0] - r) ** 2 + s * (1 - t) * torch.cos(x[0]) + s
    def optimum(self, n=2): return torch.tensor([math.pi, 2.275])


class ConvergenceTracker:
    """Loss history with the usual stopping rules: patience without relative improvement, gradient-norm floor, divergence."""

    def __init__(self, patience: int = 20, min_delta: float = 1e-6, grad_tol: float = 0.0, diverge_factor: float = 1e6): self.patience, self.min_delta, self.grad_tol, self.div, self.losses, self.best, self.since = patience, min_delta, grad_tol, diverge_factor, [], math.inf, 0

    def update(self, loss: float, grad_norm: float | None = None) -> str | None:
        self.losses.append(loss)
        if not math.isfinite(loss) or (len(self.losses) > 1 and loss > self.div * max(abs(self.losses[0]), 1e-12)):
            return "diverged"
        if not math.isfinite(self.best) or loss < self.best - self.min_delta * max(abs(self.best), 1.0):
            self.best, self.since = loss, 0
        else:
            self.since += 1
        if grad_norm is not None and grad_norm < self.grad_tol:
            return "gradient_tolerance"
        return "stalled" if self.since >= self.patience else None

    def rate(self, window: int = 20) -> float:
        """Mean log-reduction per step over the last ``window`` steps (positive: converging)."""
        h = [l for l in self.losses[-window:] if l > 0]
        return (math.log(h[0]) - math.log(h[-1])) / (len(h) - 1) if len(h) > 1 else 0.0


class OptimizerBenchmarks:
    """Runs optimizers on the test functions from the same start and reports the final value, the steps needed to reach a
    tolerance and the wall time."""

    def __init__(self, functions: dict | None = None, dim: int = 4, steps: int = 500, tol: float = 1e-4): self.functions, self.dim, self.steps, self.tol = functions or {"sphere": Sphere(), "rosenbrock": Rosenbrock()}, dim, steps, tol

    def run(self, optimizers: dict[str, Callable[[list], Optimizer]], seed: int = 0) -> dict:
        out = {}
        for fname, f in self.functions.items():
            g = torch.Generator().manual_seed(seed)
            lo, hi = f.bounds
            x0 = lo + (hi - lo) * torch.rand(self.dim, generator=g, dtype=torch.float64)
            row = {}
            for oname, make in optimizers.items():
                x = x0.clone().requires_grad_(True)
                opt, reached, t0 = make([x]), None, time.perf_counter()
                for i in range(self.steps):
                    def closure():
                        opt.zero_grad(); l = f(x); l.backward(); return l
                    l = opt.step(closure)
                    if reached is None and float(f(x.detach())) - f.minimum < self.tol:
                        reached = i + 1
                row[oname] = {"final": float(f(x.detach())) - f.minimum, "steps_to_tolerance": reached, "seconds": time.perf_counter() - t0}
            out[fname] = {**row, "winner": min(row, key=lambda k: (row[k]["steps_to_tolerance"] or math.inf, row[k]["final"]))}
        return out


class OptimizerStressTester:
    """Hostile conditions: an ill-conditioned quadratic, noisy gradients, a gradient spike, non-finite gradients, a huge
    learning rate.  Each test reports whether the iterate stayed finite and how far it got."""

    def __init__(self, make: Callable[[list], Optimizer], steps: int = 200): self.make, self.steps = make, steps

    def _run(self, grad_fn, x0):
        x = x0.clone().requires_grad_(True)
        opt = self.make([x])
        for i in range(self.steps):
            opt.zero_grad(); x.grad = grad_fn(x.detach(), i); opt.step()
            if not torch.isfinite(x).all():
                return x.detach(), False
        return x.detach(), True

    def run(self) -> dict:
        g = torch.Generator().manual_seed(0)
        d = torch.tensor([1.0, 10.0, 100.0, 1000.0], dtype=torch.float64)
        x0 = torch.ones(4, dtype=torch.float64)
        tests = {"ill_conditioned": lambda x, i: d * x, "noisy": lambda x, i: x + 0.5 * torch.randn(4, generator=g, dtype=torch.float64), "spike": lambda x, i: x * (1e6 if i == 50 else 1.0),
                 "non_finite": lambda x, i: torch.full_like(x, float("nan")) if i == 30 else x}
        out = {}
        for name, fn in tests.items():
            x, finite = self._run(fn, x0)
            out[name] = {"finite": finite, "distance": float(x.norm()) if finite else math.inf}
        out["passed"] = [k for k, v in out.items() if isinstance(v, dict) and v["finite"] and v["distance"] < 1.0]
        return out


# ================================================================================================ wrappers
class CarbonConsciousOptimizer:
    """Defers optional work when the grid is dirty: above ``threshold`` gCO2/kWh only every ``defer_factor``-th step is applied
    (gradients keep accumulating, so no information is lost); the estimated emissions per step are tallied."""

    def __init__(self, base: Optimizer, intensity: Callable[[], float], threshold: float = 400.0, defer_factor: int = 4, joules_per_step: float = 100.0):
        self.base, self.intensity, self.threshold, self.defer, self.jps, self.steps, self.applied, self.grams = base, intensity, threshold, defer_factor, joules_per_step, 0, 0, 0.0

    def step(self) -> bool:
        self.steps += 1
        ci = self.intensity()
        if ci > self.threshold and self.steps % self.defer:
            return False
        self.base.step(); self.base.zero_grad(); self.applied += 1
        self.grams += self.jps / 3.6e6 * ci
        return True
    def zero_grad(self): pass                                                       # cleared only after an applied step
    def report(self) -> dict: return {"steps": self.steps, "applied": self.applied, "grams_co2": self.grams}


class PowerCappedOptimizer:
    """Keeps a moving average of measured power under ``cap_watts`` by inserting a pause proportional to the overshoot before a
    step (a duty-cycle control; no device setting is changed)."""

    def __init__(self, base: Optimizer, power: Callable[[], float], cap_watts: float, gain: float = 0.01, sleep: Callable[[float], None] = time.sleep, alpha: float = 0.3):
        self.base, self.power, self.cap, self.gain, self.sleep, self.alpha, self.avg, self.paused = base, power, cap_watts, gain, sleep, alpha, None, 0.0
    def step(self):
        w = self.power()
        self.avg = w if self.avg is None else (1 - self.alpha) * self.avg + self.alpha * w
        if self.avg > self.cap:
            pause = self.gain * (self.avg - self.cap) / self.cap
            self.sleep(pause); self.paused += pause
        self.base.step()
    def zero_grad(self, *a, **k): self.base.zero_grad(*a, **k)


class CheckpointingOptimizer:
    """Snapshots parameters and optimizer state every ``every`` steps (keeping the last ``keep``) and can roll back, e.g. after a
    loss spike."""

    def __init__(self, base: Optimizer, every: int = 100, keep: int = 3): self.base, self.every, self.keep, self.n, self.snapshots = base, every, keep, 0, []
    def step(self, closure=None):
        out = self.base.step(closure) if closure else self.base.step()
        self.n += 1
        if self.n % self.every == 0:
            self.snapshots.append((self.n, [[p.detach().clone() for p in g["params"]] for g in self.base.param_groups], copy.deepcopy(self.base.state_dict())))
            self.snapshots = self.snapshots[-self.keep:]
        return out
    def zero_grad(self, *a, **k): self.base.zero_grad(*a, **k)
    @torch.no_grad()
    def rollback(self, back: int = 1) -> int:
        step, params, state = self.snapshots[-back]
        for g, saved in zip(self.base.param_groups, params):
            for p, s in zip(g["params"], saved):
                p.copy_(s)
        self.base.load_state_dict(state)
        self.snapshots, self.n = self.snapshots[: len(self.snapshots) - back + 1], step
        return step


class TemporalCreditOptimizer(Optimizer):
    """Eligibility traces: each parameter keeps a decaying trace of its gradients; a scalar reward (or error) signal delivered
    later scales the trace into an update, assigning credit to gradients from the recent past."""

    def __init__(self, params, lr=0.01, trace_decay=0.9): super().__init__(params, dict(lr=lr, trace_decay=trace_decay))
    @torch.no_grad()
    def accumulate(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    st = self.state[p]
                    st["trace"] = st.get("trace", torch.zeros_like(p)) * g["trace_decay"] + p.grad
    @torch.no_grad()
    def step(self, reward: float = 1.0):
        for g in self.param_groups:
            for p in g["params"]:
                if "trace" in self.state[p]:
                    p.add_(self.state[p]["trace"], alpha=g["lr"] * reward)


def LowPrecisionOptimizer(params, **kw):
    from .advanced import LowPrecisionAdam
    return LowPrecisionAdam(params, **kw)


# ================================================================================================ builders and matching
class ParamGroupBuilder:
    def __init__(self): self.groups = []
    def group(self, params: Iterable, **options): self.groups.append({"params": list(params), **options}); return self
    def no_decay_for(self, model: torch.nn.Module, weight_decay: float, patterns=("bias", "norm", "ln", "bn")):
        decay, no = [], []
        for n, p in model.named_parameters():
            (no if p.dim() < 2 or any(k in n.lower() for k in patterns) else decay).append(p)
        self.groups += [{"params": decay, "weight_decay": weight_decay}, {"params": no, "weight_decay": 0.0}]
        return self
    def build(self) -> list[dict]: return [g for g in self.groups if g["params"]]


_REGISTRY = {"sgd": torch.optim.SGD, "adam": torch.optim.Adam, "adamw": torch.optim.AdamW, "rmsprop": torch.optim.RMSprop, "adagrad": torch.optim.Adagrad, "adadelta": torch.optim.Adadelta, "adamax": torch.optim.Adamax, "nadam": torch.optim.NAdam,
             "radam": torch.optim.RAdam, "advanced_adam": AdvancedAdam, "schedule_free_adamw": ScheduleFreeAdamW}


class OptimizerBuilder:
    """``OptimizerBuilder("adamw").lr(3e-4).weight_decay(0.1).betas((0.9, 0.95)).build(params)``; unknown names also look in this
    package's optimizers."""

    def __init__(self, name: str): self.name, self.kw = name.lower(), {}
    def __getattr__(self, key):
        if key.startswith("_"):
            raise AttributeError(key)
        def setter(v): self.kw[key] = v; return self
        return setter
    def build(self, params):
        if self.name in _REGISTRY:
            return _REGISTRY[self.name](params, **self.kw)
        import torsh_b200.optim as O
        for n in dir(O):
            if n.lower() == self.name and isinstance(getattr(O, n), type):
                return getattr(O, n)(params, **self.kw)
        raise ValueError(f"unknown optimizer {self.name!r}")


class TaskMatcher:
    """Remembers which optimizer configuration worked for tasks described by a few numbers (log parameters, log data size,
    sparsity, noise) and proposes the configuration of the most similar remembered task."""

    def __init__(self): self.memory = []
    @staticmethod
    def _vec(c: dict) -> torch.Tensor: return torch.tensor([math.log10(max(c.get("parameters", 1), 1)), math.log10(max(c.get("samples", 1), 1)), c.get("gradient_sparsity", 0.0) * 5, c.get("gradient_noise", 0.0) * 5], dtype=torch.float64)
    def remember(self, characteristics: dict, config: dict, score: float): self.memory.append((self._vec(characteristics), config, score))
    def with_defaults(self):
        self.remember({"parameters": 1e8, "samples": 1e9, "gradient_noise": 0.3}, {"optimizer": "adamw", "lr": 3e-4, "weight_decay": 0.1, "betas": (0.9, 0.95)}, 1.0)
        self.remember({"parameters": 2.5e7, "samples": 1.3e6, "gradient_noise": 0.1}, {"optimizer": "sgd", "lr": 0.1, "momentum": 0.9, "weight_decay": 1e-4}, 1.0)
        self.remember({"parameters": 1e6, "samples": 1e5, "gradient_sparsity": 0.95}, {"optimizer": "adagrad", "lr": 0.05}, 1.0)
        self.remember({"parameters": 1e4, "samples": 1e3}, {"optimizer": "lbfgs", "lr": 1.0}, 1.0)
        return self
    def suggest(self, characteristics: dict, k: int = 1) -> dict:
        v = self._vec(characteristics)
        ranked = sorted(self.memory, key=lambda m: float((m[0] - v).norm()) - 0.1 * m[2])
        return {**ranked[0][1], "distance": float((ranked[0][0] - v).norm()), "alternatives": [r[1]["optimizer"] for r in ranked[1:k + 1]]}
