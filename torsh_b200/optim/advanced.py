"""Optimizer wrappers and specialised methods (the remaining files of ``crates/torsh-optim/src``):

* continual learning: EWC, MAS and Synaptic Intelligence penalties applied inside the step (``continual_learning.rs``);
* differentially private SGD with per-sample clipping, Gaussian noise and an RDP accountant (``differential_privacy.rs``);
* online / variance-reduced methods: OGD with regret tracking, proximal gradient, SVRG, SAGA (``online_learning.rs``);
* composition of optimizers: sequential phases, switching on a criterion, averaged or voted updates (``composition.rs``);
* analysis: convergence tracking, gradient statistics, recommendations, hyper-parameter sensitivity (``debugging.rs``);
* storage: 8-bit block-quantised and bf16 optimizer state (``low_precision.rs``), factored second moments and a bounded
  L-BFGS history (``memory_efficient.rs``), state in memory-mapped files (``memory_mapped.rs``);
* update skipping: lazy updates by importance (``lazy_updates.rs``), top-k sparse updates with residuals
  (``sparse_updates.rs``);
* state-dict tools: compression, memory estimate, conversion between optimizers (``state_dict_ops.rs``);
* search: hyper-parameter tuner with successive halving (``hyperparameter_tuning.rs``), a learned optimizer
  (``neural_optimizer.rs``), task-matched optimizer choice (``meta_learning.rs``);
* robustness guards with rollback (``robustness.rs``), energy / carbon aware stepping (``green_ai.rs``),
  spike-timing and event-driven updates (``neuromorphic.rs``), quantum-inspired global search (``quantum_inspired.rs``),
  and step-for-step comparison with another framework's optimizer (``cross_framework_validation.rs``).
"""
from __future__ import annotations

import copy
import io
import math
import time
import zlib
from pathlib import Path
from typing import Callable

import numpy as np
import torch

from .extra import _Mixin


def _params(opt):
    return [p for g in opt.param_groups for p in g["params"]]


# ================================================================================================ continual learning
class _PenaltyOptimizer(_Mixin):
    """Wraps an optimizer and adds ``lambda * importance * (theta - anchor)`` to the gradients before each step."""

    def __init__(self, base: torch.optim.Optimizer, lam: float):
        self.base, self.lam, self.param_groups = base, lam, base.param_groups
        self.importance = [torch.zeros_like(p) for p in _params(base)]
        self.anchor = [p.detach().clone() for p in _params(base)]

    def zero_grad(self, set_to_none: bool = True): self.base.zero_grad(set_to_none)
    def state_dict(self): return {"base": self.base.state_dict(), "importance": self.importance, "anchor": self.anchor}

    def penalty(self) -> torch.Tensor:
        return 0.5 * self.lam * sum((w * (p - a) ** 2).sum() for p, w, a in zip(_params(self.base), self.importance, self.anchor))

    def _before_step(self): pass

    @torch.no_grad()
    def step(self, closure=None):
        self._before_step()
        for p, w, a in zip(_params(self.base), self.importance, self.anchor):
            if p.grad is not None:
                p.grad.add_(self.lam * w * (p - a))
        return self.base.step(closure)


class EWCOptimizer(_PenaltyOptimizer):
    """Elastic weight consolidation: importance = diagonal Fisher (mean squared gradient of the log-likelihood)."""

    def consolidate(self, model, batches, loss_fn, online_decay: float | None = None):
        fisher = [torch.zeros_like(p) for p in _params(self.base)]
        n = 0
        for x, y in batches:
            model.zero_grad()
            loss_fn(model(x), y).backward()
            for f, p in zip(fisher, _params(self.base)):
                if p.grad is not None:
                    f += p.grad.detach() ** 2
            n += 1
        model.zero_grad()
        for i, f in enumerate(fisher):
            f /= max(n, 1)
            self.importance[i] = f if online_decay is None else online_decay * self.importance[i] + f
        self.anchor = [p.detach().clone() for p in _params(self.base)]


class MASOptimizer(_PenaltyOptimizer):
    """Memory-aware synapses: importance = mean absolute gradient of the squared output norm (needs no labels)."""

    def consolidate(self, model, inputs):
        imp = [torch.zeros_like(p) for p in _params(self.base)]
        for x in inputs:
            model.zero_grad()
            model(x).pow(2).sum(-1).mean().backward()
            for w, p in zip(imp, _params(self.base)):
                if p.grad is not None:
                    w += p.grad.detach().abs()
        model.zero_grad()
        self.importance = [a + w / max(len(inputs), 1) for a, w in zip(self.importance, imp)]
        self.anchor = [p.detach().clone() for p in _params(self.base)]


class SIOptimizer(_PenaltyOptimizer):
    """Synaptic intelligence: a running path integral ``-sum g * delta_theta`` per parameter during training, turned into
    importance ``omega / (total change^2 + xi)`` at each task boundary."""

    def __init__(self, base, lam: float, xi: float = 1e-3):
        super().__init__(base, lam)
        self.xi = xi
        self.path = [torch.zeros_like(p) for p in _params(base)]
        self.start = [p.detach().clone() for p in _params(base)]
        self._prev = None

    def _before_step(self):
        self._prev = [(p.detach().clone(), None if p.grad is None else p.grad.detach().clone()) for p in _params(self.base)]

    @torch.no_grad()
    def step(self, closure=None):
        out = super().step(closure)
        for w, p, (old, g) in zip(self.path, _params(self.base), self._prev):
            if g is not None:
                w -= g * (p.detach() - old)
        return out

    def consolidate(self):
        for i, p in enumerate(_params(self.base)):
            self.importance[i] = self.importance[i] + (self.path[i] / ((p.detach() - self.start[i]) ** 2 + self.xi)).clamp(min=0)
            self.path[i].zero_()
        self.anchor = [p.detach().clone() for p in _params(self.base)]
        self.start = [p.detach().clone() for p in _params(self.base)]


# ================================================================================================ differential privacy
class RDPAccountant:
    """Renyi-DP of the sampled Gaussian mechanism at integer orders, composed over steps and converted to (eps, delta)."""

    ORDERS = tuple(range(2, 64))

    def __init__(self):
        self.rdp = np.zeros(len(self.ORDERS))
        self.steps = 0

    @staticmethod
    def _log_comb(n, k): return math.lgamma(n + 1) - math.lgamma(k + 1) - math.lgamma(n - k + 1)

    def _rdp_order(self, q: float, sigma: float, alpha: int) -> float:
        if q == 0:
            return 0.0
        if sigma == 0:
            return math.inf                                                   # no noise, no privacy
        if q == 1.0:
            return alpha / (2 * sigma ** 2)
        terms = [self._log_comb(alpha, k) + k * math.log(q) + (alpha - k) * math.log(1 - q) + (k * k - k) / (2 * sigma ** 2) for k in range(alpha + 1)]
        m = max(terms)
        return (m + math.log(sum(math.exp(t - m) for t in terms))) / (alpha - 1)

    def step(self, sample_rate: float, noise_multiplier: float, n: int = 1):
        self.rdp += n * np.array([self._rdp_order(sample_rate, noise_multiplier, a) for a in self.ORDERS])
        self.steps += n

    def get_epsilon(self, delta: float) -> float:
        eps = self.rdp + math.log(1 / delta) / (np.array(self.ORDERS) - 1)
        return float(eps.min())


class DPOptimizer(_Mixin):
    """DP-SGD around any optimizer: ``step(per_sample_grads)`` clips each sample's gradient to ``max_grad_norm`` in global
    L2 norm, sums, adds ``N(0, (noise_multiplier * max_grad_norm)^2)``, divides by the batch size and steps.
    ``per_sample_grads``: one tensor per parameter with a leading batch dimension (see :func:`per_sample_gradients`)."""

    def __init__(self, base, noise_multiplier: float, max_grad_norm: float, sample_rate: float, seed: int | None = None):
        self.base, self.param_groups = base, base.param_groups
        self.sigma, self.clip, self.q = noise_multiplier, max_grad_norm, sample_rate
        self.accountant, self.gen = RDPAccountant(), None
        if seed is not None:
            self.gen = torch.Generator().manual_seed(seed)
        self.clipped_fraction = 0.0

    def zero_grad(self, set_to_none=True): self.base.zero_grad(set_to_none)

    @torch.no_grad()
    def step(self, per_sample_grads):
        b = per_sample_grads[0].shape[0]
        norms = torch.sqrt(sum(g.reshape(b, -1).pow(2).sum(1) for g in per_sample_grads))
        scale = (self.clip / (norms + 1e-12)).clamp(max=1.0)
        self.clipped_fraction = float((scale < 1).float().mean())
        for p, g in zip(_params(self.base), per_sample_grads):
            s = (g * scale.reshape(-1, *[1] * (g.dim() - 1))).sum(0)
            noise = torch.randn(s.shape, generator=self.gen).to(s) * self.sigma * self.clip
            p.grad = (s + noise) / b
        self.base.step()
        self.accountant.step(self.q, self.sigma)

    def privacy_spent(self, delta: float = 1e-5) -> dict:
        return {"epsilon": self.accountant.get_epsilon(delta), "delta": delta, "steps": self.accountant.steps}


def per_sample_gradients(model, loss_fn, x, y):
    """Per-sample gradients through ``torch.func`` (one backward pass, vectorised over the batch)."""
    from torch.func import functional_call, grad, vmap
    names = [n for n, _ in model.named_parameters()]
    params = {n: p.detach() for n, p in model.named_parameters()}
    def one(ps, xi, yi):
        return loss_fn(functional_call(model, ps, (xi[None],)), yi[None])
    g = vmap(grad(one), in_dims=(None, 0, 0))(params, x, y)
    return [g[n] for n in names]


# ================================================================================================ online / variance reduced
class OnlineGradientDescent(_Mixin, torch.optim.Optimizer):
    """``lr_t = lr / sqrt(t)`` with optional projection onto an L2 ball; tracks cumulative loss for regret estimates."""

    def __init__(self, params, lr=0.1, radius: float | None = None):
        super().__init__(params, dict(lr=lr))
        self.radius, self.t, self.cumulative_loss = radius, 0, 0.0

    @torch.no_grad()
    def step(self, loss: float | None = None):
        self.t += 1
        if loss is not None:
            self.cumulative_loss += float(loss)
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    p.add_(p.grad, alpha=-g["lr"] / math.sqrt(self.t))
        if self.radius is not None:
            n = math.sqrt(sum(float(p.pow(2).sum()) for p in _params(self)))
            if n > self.radius:
                for p in _params(self):
                    p.mul_(self.radius / n)

    def regret(self, best_fixed_loss: float) -> float: return self.cumulative_loss - best_fixed_loss


def prox_l1(x, t): return torch.sign(x) * (x.abs() - t).clamp(min=0)
def prox_l2(x, t): return x / (1 + t)
def prox_box(lo, hi): return lambda x, t: x.clamp(lo, hi)


def prox_group_lasso(x, t):
    n = x.norm(dim=-1, keepdim=True).clamp(min=1e-12)
    return x * (1 - t / n).clamp(min=0)


class ProximalGradient(_Mixin, torch.optim.Optimizer):
    """Forward-backward splitting ``x <- prox_{lr * reg}(x - lr * grad)``; ``accelerated`` adds FISTA momentum."""

    def __init__(self, params, lr=0.1, prox: Callable = prox_l1, reg: float = 0.01, accelerated: bool = False):
        super().__init__(params, dict(lr=lr))
        self.prox, self.reg, self.accelerated, self.tk = prox, reg, accelerated, 1.0

    @torch.no_grad()
    def step(self):
        t_next = (1 + math.sqrt(1 + 4 * self.tk ** 2)) / 2
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                new = self.prox(p - g["lr"] * p.grad, g["lr"] * self.reg)
                if self.accelerated:
                    st = self.state[p]
                    prev = st.get("prev", new)
                    st["prev"] = new.clone()
                    p.copy_(new + (self.tk - 1) / t_next * (new - prev))
                else:
                    p.copy_(new)
        self.tk = t_next


class SVRG(_Mixin):
    """Stochastic variance-reduced gradient: ``g_i(w) - g_i(w_snap) + full_grad(w_snap)``; the caller provides
    ``grad_fn(params, indices) -> list of gradients`` and calls :meth:`snapshot` once per epoch."""

    def __init__(self, params, grad_fn, n: int, lr=0.1):
        self.params, self.grad_fn, self.n, self.lr = list(params), grad_fn, n, lr
        self.param_groups = [{"params": self.params, "lr": lr}]
        self.snapshot()

    @torch.no_grad()
    def snapshot(self):
        self.w_snap = [p.detach().clone() for p in self.params]
        self.mu = [g.detach().clone() for g in self.grad_fn(self.w_snap, torch.arange(self.n))]

    @torch.no_grad()
    def step(self, indices):
        g_now, g_old = self.grad_fn(self.params, indices), self.grad_fn(self.w_snap, indices)
        for p, a, b, m in zip(self.params, g_now, g_old, self.mu):
            p.add_(a - b + m, alpha=-self.param_groups[0]["lr"])


class SAGA(_Mixin):
    """Keeps the last gradient of every sample; update direction ``g_i - table_i + mean(table)``."""

    def __init__(self, params, grad_fn, n: int, lr=0.1):
        self.params, self.grad_fn, self.n = list(params), grad_fn, n
        self.param_groups = [{"params": self.params, "lr": lr}]
        self.table = [torch.zeros(n, *p.shape) for p in self.params]
        self.mean = [torch.zeros_like(p) for p in self.params]

    @torch.no_grad()
    def step(self, i: int):
        g = self.grad_fn(self.params, torch.tensor([i]))
        for p, gi, tab, mean in zip(self.params, g, self.table, self.mean):
            p.add_(gi - tab[i] + mean, alpha=-self.param_groups[0]["lr"])
            mean += (gi - tab[i]) / self.n
            tab[i] = gi


# ================================================================================================ composition
class ComposedOptimizer(_Mixin):
    """Several optimizers over the same parameters.

    ``sequential``: optimizer ``i`` runs for ``phases[i]`` steps, then the next (the last one keeps going).
    ``switch``: starts with the first and moves to the next whenever ``criterion(history) -> bool`` fires.
    ``average``: every optimizer proposes an update from the same gradients; the weighted mean is applied.
    ``vote``: the sign of each coordinate's update is the majority sign, its size the median magnitude."""

    def __init__(self, optimizers, strategy="sequential", phases=None, criterion=None, weights=None):
        self.opts, self.strategy, self.phases, self.criterion = list(optimizers), strategy, phases, criterion
        self.weights = weights or [1.0 / len(self.opts)] * len(self.opts)
        self.active, self.steps, self.history, self.switches = 0, 0, [], []
        self.param_groups = self.opts[0].param_groups

    def zero_grad(self, set_to_none=True):
        for o in self.opts:
            o.zero_grad(set_to_none)

    @torch.no_grad()
    def step(self, loss: float | None = None):
        self.steps += 1
        if loss is not None:
            self.history.append(float(loss))
        if self.strategy in ("sequential", "switch"):
            if self.strategy == "sequential":
                edges = np.cumsum(self.phases)
                self.active = int(min(np.searchsorted(edges, self.steps - 1, side="right"), len(self.opts) - 1))
            elif self.criterion and self.active < len(self.opts) - 1 and self.criterion(self.history):
                self.active += 1
                self.switches.append(self.steps)
                self.history.clear()
            self.opts[self.active].step()
            return
        ps = _params(self.opts[0])
        start = [p.detach().clone() for p in ps]
        deltas = []
        for o in self.opts:
            o.step()
            deltas.append([p.detach() - s for p, s in zip(ps, start)])
            for p, s in zip(ps, start):
                p.copy_(s)
        for i, p in enumerate(ps):
            d = torch.stack([dl[i] for dl in deltas])
            if self.strategy == "average":
                w = torch.tensor(self.weights, dtype=d.dtype).reshape(-1, *[1] * (d.dim() - 1))
                p.add_((d * w).sum(0))
            else:
                sign = torch.sign(torch.sign(d).sum(0))
                p.add_(sign * d.abs().median(0).values)


def plateau_criterion(patience: int = 20, min_delta: float = 1e-4):
    return lambda h: len(h) > patience and min(h[-patience:]) >= min(h[:-patience]) - min_delta


# ================================================================================================ analysis
class OptimizerAnalyzer:
    """Records loss, gradient norm, update norm and parameter norm per step and derives a report."""

    def __init__(self, optimizer):
        self.opt, self.records, self._before = optimizer, [], None

    def before_step(self):
        self._before = [p.detach().clone() for p in _params(self.opt)]

    def after_step(self, loss: float):
        ps = _params(self.opt)
        gn = math.sqrt(sum(float(p.grad.pow(2).sum()) for p in ps if p.grad is not None))
        un = math.sqrt(sum(float((p.detach() - b).pow(2).sum()) for p, b in zip(ps, self._before)))
        pn = math.sqrt(sum(float(p.detach().pow(2).sum()) for p in ps))
        self.records.append({"loss": float(loss), "grad_norm": gn, "update_norm": un, "param_norm": pn})

    def report(self) -> dict:
        r = self.records
        loss = np.array([x["loss"] for x in r])
        gn = np.array([x["grad_norm"] for x in r])
        ratio = np.array([x["update_norm"] / max(x["param_norm"], 1e-12) for x in r])
        half = len(loss) // 2
        rate = float(np.polyfit(np.arange(len(loss)), np.log(np.maximum(loss, 1e-300)), 1)[0]) if len(loss) > 2 else 0.0
        osc = float(np.mean(np.diff(np.sign(np.diff(loss))) != 0)) if len(loss) > 3 else 0.0
        recs = []
        if not np.isfinite(loss).all() or (len(loss) > 1 and loss[-1] > 10 * loss[0]):
            recs.append({"category": "learning_rate", "severity": "critical", "message": "loss diverges: lower the learning rate or clip gradients"})
        elif osc > 0.6 and rate > -1e-3:
            recs.append({"category": "learning_rate", "severity": "warning", "message": "loss oscillates without progress: lower the learning rate"})
        elif ratio.mean() < 1e-5:
            recs.append({"category": "learning_rate", "severity": "warning", "message": "updates are tiny next to the weights: raise the learning rate"})
        if len(gn) and gn[-1] < 1e-7:
            recs.append({"category": "gradients", "severity": "warning", "message": "vanishing gradients"})
        if len(gn) and gn.max() > 1e3 * max(np.median(gn), 1e-12):
            recs.append({"category": "gradients", "severity": "warning", "message": "gradient spikes: add clipping"})
        return {"steps": len(r), "convergence_rate": rate, "oscillation": osc, "mean_update_ratio": float(ratio.mean()) if len(ratio) else 0.0,
                "improved": bool(len(loss) > 1 and loss[half:].mean() < loss[:max(half, 1)].mean()), "recommendations": recs}


def hyperparameter_sensitivity(make_run: Callable[[dict], float], base: dict, factors=(0.5, 2.0)) -> dict:
    """Final loss of ``make_run(config)`` when one numeric hyper-parameter at a time is scaled; sensitivity is the
    largest relative change of the final loss."""
    ref = make_run(dict(base))
    out = {}
    for k, v in base.items():
        if isinstance(v, (int, float)) and not isinstance(v, bool):
            losses = [make_run({**base, k: v * f}) for f in factors]
            out[k] = {"losses": losses, "sensitivity": max(abs(l - ref) for l in losses) / max(abs(ref), 1e-12)}
    return {"reference": ref, "parameters": out, "ranking": sorted(out, key=lambda k: -out[k]["sensitivity"])}


# ================================================================================================ state storage
def quantize_blockwise(x: torch.Tensor, block: int = 256, signed: bool = True):
    """8-bit codes with one absmax scale per block; dynamic range is spent where the block's values are."""
    flat = x.reshape(-1)
    pad = (-flat.numel()) % block
    f = torch.cat([flat, flat.new_zeros(pad)]).reshape(-1, block)
    scale = f.abs().amax(1, keepdim=True).clamp(min=1e-30)
    q = (f / scale * (127 if signed else 255)).round().to(torch.int8 if signed else torch.uint8)
    return q, scale.squeeze(1), x.shape, pad


def dequantize_blockwise(q, scale, shape, pad, signed: bool = True):
    f = q.float() / (127 if signed else 255) * scale[:, None]
    flat = f.reshape(-1)
    return (flat[:flat.numel() - pad] if pad else flat).reshape(shape)


class LowPrecisionAdam(_Mixin, torch.optim.Optimizer):
    """Adam whose moments are stored in ``bf16`` or block-quantised ``int8`` (the second moment is stored as its square
    root to keep small values representable); arithmetic is fp32 inside the step."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, state_dtype: str = "int8", block: int = 256):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.state_dtype, self.block = state_dtype, block

    def _load(self, st, key, like, signed):
        if key not in st:
            return torch.zeros_like(like, dtype=torch.float32)
        return st[key].float() if self.state_dtype == "bf16" else dequantize_blockwise(*st[key], signed=signed)

    def _store(self, st, key, v, signed):
        st[key] = v.to(torch.bfloat16) if self.state_dtype == "bf16" else quantize_blockwise(v, self.block, signed)

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                m = self._load(st, "m", p, True).mul_(b1).add_(p.grad.float(), alpha=1 - b1)
                v = self._load(st, "sqrt_v", p, False).pow_(2).mul_(b2).addcmul_(p.grad.float(), p.grad.float(), value=1 - b2)
                self._store(st, "m", m, True)
                self._store(st, "sqrt_v", v.sqrt(), False)
                mh, vh = m / (1 - b1 ** st["step"]), v / (1 - b2 ** st["step"])
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_((mh / (vh.sqrt() + g["eps"])).to(p.dtype), alpha=-g["lr"])

    def state_bytes(self) -> int:
        n = 0
        for st in self.state.values():
            for k in ("m", "sqrt_v"):
                v = st.get(k)
                n += v.numel() * 2 if isinstance(v, torch.Tensor) else (v[0].numel() + v[1].numel() * 4 if v else 0)
        return n


class MemoryEfficientAdam(_Mixin, torch.optim.Optimizer):
    """Factored second moment for matrices (row and column means, as in Adafactor), full second moment for vectors, and
    an optional first moment; state for an ``[n, m]`` matrix is ``n + m`` numbers instead of ``n * m``."""

    def __init__(self, params, lr=1e-2, beta1: float | None = 0.9, beta2=0.999, eps=1e-30, clip_threshold=1.0):
        super().__init__(params, dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, clip=clip_threshold))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st, grad = self.state[p], p.grad.float()
                st["step"] = st.get("step", 0) + 1
                sq = grad * grad + g["eps"]
                if grad.dim() >= 2:
                    r = st.setdefault("row", torch.zeros(grad.shape[:-1])).mul_(g["beta2"]).add_(sq.mean(-1), alpha=1 - g["beta2"])
                    c = st.setdefault("col", torch.zeros(grad.shape[:-2] + grad.shape[-1:])).mul_(g["beta2"]).add_(sq.mean(-2), alpha=1 - g["beta2"])
                    v = r.unsqueeze(-1) * c.unsqueeze(-2) / r.mean(-1, keepdim=True).unsqueeze(-1).clamp(min=1e-30)
                else:
                    v = st.setdefault("v", torch.zeros_like(grad)).mul_(g["beta2"]).add_(sq, alpha=1 - g["beta2"])
                u = grad / (v / (1 - g["beta2"] ** st["step"])).sqrt().clamp(min=1e-30)
                u = u / max(1.0, float(u.pow(2).mean().sqrt()) / g["clip"])
                if g["beta1"] is not None:
                    u = st.setdefault("m", torch.zeros_like(grad)).mul_(g["beta1"]).add_(u, alpha=1 - g["beta1"])
                p.add_(u.to(p.dtype), alpha=-g["lr"])

    def state_numel(self) -> int:
        return sum(v.numel() for st in self.state.values() for v in st.values() if isinstance(v, torch.Tensor))


class CircularBuffer:
    def __init__(self, capacity: int):
        self.capacity, self.items, self.head = capacity, [], 0

    def push(self, x):
        if len(self.items) < self.capacity:
            self.items.append(x)
        else:
            self.items[self.head] = x
            self.head = (self.head + 1) % self.capacity

    def __iter__(self): return iter(self.items[self.head:] + self.items[:self.head])
    def __len__(self): return len(self.items)


class MemoryEfficientLBFGS(_Mixin):
    """Two-loop L-BFGS over a flat view of the parameters with a ring of ``history`` curvature pairs and a backtracking
    Armijo line search; ``step(closure)`` where the closure returns the loss and fills ``.grad``."""

    def __init__(self, params, lr=1.0, history: int = 10, c1: float = 1e-4, max_ls: int = 20):
        self.params, self.pairs, self.c1, self.max_ls = list(params), CircularBuffer(history), c1, max_ls
        self.param_groups = [{"params": self.params, "lr": lr}]
        self._prev = None

    def _flat(self, attr=None):
        return torch.cat([(p if attr is None else getattr(p, attr)).detach().reshape(-1) for p in self.params])

    def _set(self, flat):
        i = 0
        with torch.no_grad():
            for p in self.params:
                p.copy_(flat[i:i + p.numel()].reshape(p.shape))
                i += p.numel()

    def step(self, closure):
        loss = float(closure().detach())
        x, g = self._flat(), self._flat("grad")
        if self._prev is not None:
            s, y = x - self._prev[0], g - self._prev[1]
            if float(s @ y) > 1e-10:
                self.pairs.push((s, y))
        q, alphas = g.clone(), []
        for s, y in reversed(list(self.pairs)):
            a = float(s @ q) / float(y @ s)
            alphas.append(a)
            q -= a * y
        if len(self.pairs):
            s, y = list(self.pairs)[-1]
            q *= float(s @ y) / float(y @ y)
        for (s, y), a in zip(self.pairs, reversed(alphas)):
            q += s * (a - float(y @ q) / float(y @ s))
        d, t = -q, self.param_groups[0]["lr"]
        slope = float(g @ d)
        for k in range(self.max_ls):
            self._set(x + t * d)
            new = float(closure().detach())
            if new <= loss + self.c1 * t * slope:
                if k == 0:                                                    # the first trial already passes: try longer steps
                    for _ in range(self.max_ls):
                        self._set(x + 2 * t * d)
                        longer = float(closure().detach())
                        if longer >= new or longer > loss + self.c1 * 2 * t * slope:
                            self._set(x + t * d)
                            closure()
                            break
                        t, new = 2 * t, longer
                break
            t *= 0.5
        self._prev = (x, g)
        return loss


class MemoryMappedState:
    """Per-parameter optimizer state tensors that live in one memory-mapped file (``numpy.memmap``); tensors returned by
    :meth:`get` alias the file, so in-place updates persist after :meth:`flush`."""

    def __init__(self, path, layout: dict[str, tuple], dtype=np.float32):
        self.path, self.layout, self.offsets, off = Path(path), layout, {}, 0
        for k, shape in layout.items():
            self.offsets[k] = (off, int(np.prod(shape)))
            off += int(np.prod(shape))
        mode = "r+" if self.path.exists() and self.path.stat().st_size == off * np.dtype(dtype).itemsize else "w+"
        self.map = np.memmap(self.path, dtype=dtype, mode=mode, shape=(max(off, 1),))

    def get(self, key: str) -> torch.Tensor:
        off, n = self.offsets[key]
        return torch.from_numpy(self.map[off:off + n]).reshape(self.layout[key])

    def flush(self): self.map.flush()
    def bytes(self): return self.map.nbytes


class MemoryMappedAdam(_Mixin, torch.optim.Optimizer):
    """Adam with both moments in a :class:`MemoryMappedState` file (state survives the process and never sits in the
    allocator's memory)."""

    def __init__(self, params, path, lr=1e-3, betas=(0.9, 0.999), eps=1e-8):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps))
        ps = _params(self)
        layout = {f"{k}{i}": tuple(p.shape) for i, p in enumerate(ps) for k in ("m", "v")} | {"step": (1,)}
        self.store = MemoryMappedState(path, layout)

    @torch.no_grad()
    def step(self):
        step = self.store.get("step")
        step += 1
        t = int(step.item())
        for i, p in enumerate(_params(self)):
            if p.grad is None:
                continue
            g = self.param_groups[0]
            b1, b2 = g["betas"]
            m, v = self.store.get(f"m{i}"), self.store.get(f"v{i}")
            m.mul_(b1).add_(p.grad, alpha=1 - b1)
            v.mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
            p.addcdiv_(m / (1 - b1 ** t), (v / (1 - b2 ** t)).sqrt() + g["eps"], value=-g["lr"])
        self.store.flush()


# ================================================================================================ update skipping
class LazyUpdateOptimizer(_Mixin):
    """Accumulates gradients per parameter tensor and only applies them when the accumulated norm, relative to the
    tensor's own norm, passes ``threshold`` or ``max_delay`` steps have gone by; skipped tensors cost no optimizer work."""

    def __init__(self, base, threshold: float = 1e-3, max_delay: int = 8):
        self.base, self.param_groups, self.threshold, self.max_delay = base, base.param_groups, threshold, max_delay
        self.pending = {p: [torch.zeros_like(p), 0] for p in _params(base)}
        self.applied = self.skipped = 0

    def zero_grad(self, set_to_none=True): self.base.zero_grad(set_to_none)

    @torch.no_grad()
    def step(self):
        for p in _params(self.base):
            if p.grad is None:
                continue
            acc = self.pending[p]
            acc[0] += p.grad
            acc[1] += 1
            importance = float(acc[0].norm()) / max(float(p.norm()), 1e-12)
            if importance >= self.threshold or acc[1] >= self.max_delay:
                p.grad = acc[0] / acc[1]
                self.pending[p] = [torch.zeros_like(p), 0]
                self.applied += 1
            else:
                p.grad = None
                self.skipped += 1
        self.base.step()

    def statistics(self): return {"applied": self.applied, "skipped": self.skipped, "skip_rate": self.skipped / max(self.applied + self.skipped, 1)}


class SparseUpdateOptimizer(_Mixin):
    """Keeps the ``density`` largest-magnitude gradient entries per tensor, stores the rest as a residual that is added to
    the next gradient (error feedback), and tracks which coordinates are touched."""

    def __init__(self, base, density: float = 0.1):
        self.base, self.param_groups, self.density = base, base.param_groups, density
        self.residual = {p: torch.zeros_like(p) for p in _params(base)}
        self.touch = {p: torch.zeros(p.shape, dtype=torch.long) for p in _params(base)}
        self.sent = self.total = 0

    def zero_grad(self, set_to_none=True): self.base.zero_grad(set_to_none)

    @torch.no_grad()
    def step(self):
        for p in _params(self.base):
            if p.grad is None:
                continue
            full = p.grad + self.residual[p]
            k = max(1, int(self.density * full.numel()))
            thresh = full.abs().reshape(-1).topk(k).values[-1]
            mask = full.abs() >= thresh
            self.residual[p] = full * ~mask
            p.grad = full * mask
            self.touch[p] += mask
            self.sent += int(mask.sum())
            self.total += full.numel()
        self.base.step()

    def statistics(self):
        cov = sum(int((t > 0).sum()) for t in self.touch.values()) / max(sum(t.numel() for t in self.touch.values()), 1)
        return {"density": self.sent / max(self.total, 1), "coverage": cov}


# ================================================================================================ state dict tools
class StateDictManager:
    @staticmethod
    def compress(state_dict: dict, level: int = 6) -> bytes:
        buf = io.BytesIO()
        torch.save(state_dict, buf)
        return zlib.compress(buf.getvalue(), level)

    @staticmethod
    def decompress(blob: bytes) -> dict:
        return torch.load(io.BytesIO(zlib.decompress(blob)), weights_only=False)

    @staticmethod
    def memory_estimate(state_dict: dict) -> dict:
        by_key: dict[str, int] = {}
        for st in state_dict["state"].values():
            for k, v in st.items():
                if isinstance(v, torch.Tensor):
                    by_key[k] = by_key.get(k, 0) + v.numel() * v.element_size()
        return {"total_bytes": sum(by_key.values()), "by_key": by_key}

    @staticmethod
    def convert(state_dict: dict, mapping: dict[str, str | None], defaults: dict | None = None) -> dict:
        """Renames per-parameter state entries (``None`` drops one); e.g. SGD ``momentum_buffer`` -> Adam ``exp_avg``."""
        out = copy.deepcopy(state_dict)
        for st in out["state"].values():
            for old, new in mapping.items():
                if old in st:
                    v = st.pop(old)
                    if new is not None:
                        st[new] = v
            for k, fn in (defaults or {}).items():
                if k not in st:
                    st[k] = fn(st)
        return out

    @staticmethod
    def merge(dicts: list[dict], weights: list[float] | None = None) -> dict:
        """Weighted mean of the floating-point state tensors of replicas (used after local-SGD style training)."""
        w = weights or [1.0 / len(dicts)] * len(dicts)
        out = copy.deepcopy(dicts[0])
        for pid, st in out["state"].items():
            for k, v in st.items():
                if isinstance(v, torch.Tensor) and v.is_floating_point() and v.dim() > 0:
                    st[k] = sum(wi * d["state"][pid][k] for wi, d in zip(w, dicts))
        return out


# ================================================================================================ search
class HyperparameterTuner:
    """Search space entries: ``("log", lo, hi)``, ``("uniform", lo, hi)``, ``("int", lo, hi)``, ``("choice", [...])``.
    ``random`` and ``grid`` evaluate every trial at the full budget; ``halving`` starts ``n`` trials at ``min_budget``
    and keeps the best ``1/eta`` at ``eta`` times the budget until one is left (successive halving)."""

    def __init__(self, space: dict, strategy: str = "random", seed: int = 0):
        self.space, self.strategy, self.rng, self.trials = space, strategy, np.random.default_rng(seed), []

    def sample(self) -> dict:
        out = {}
        for k, spec in self.space.items():
            kind = spec[0]
            if kind == "log":
                out[k] = float(np.exp(self.rng.uniform(np.log(spec[1]), np.log(spec[2]))))
            elif kind == "uniform":
                out[k] = float(self.rng.uniform(spec[1], spec[2]))
            elif kind == "int":
                out[k] = int(self.rng.integers(spec[1], spec[2] + 1))
            else:
                out[k] = spec[1][int(self.rng.integers(len(spec[1])))]
        return out

    def grid(self, points: int = 3) -> list[dict]:
        axes = []
        for k, spec in self.space.items():
            if spec[0] == "log":
                axes.append([(k, float(v)) for v in np.exp(np.linspace(np.log(spec[1]), np.log(spec[2]), points))])
            elif spec[0] == "uniform":
                axes.append([(k, float(v)) for v in np.linspace(spec[1], spec[2], points)])
            elif spec[0] == "int":
                axes.append([(k, int(v)) for v in sorted(set(np.linspace(spec[1], spec[2], points).round().astype(int)))])
            else:
                axes.append([(k, v) for v in spec[1]])
        import itertools
        return [dict(c) for c in itertools.product(*axes)]

    def tune(self, objective: Callable[[dict, int], float], n_trials: int = 16, budget: int = 100, min_budget: int = 10, eta: int = 3,
             early_stopping_patience: int | None = None) -> dict:
        configs = self.grid() if self.strategy == "grid" else [self.sample() for _ in range(n_trials)]
        spent = 0
        if self.strategy == "halving":
            b = min_budget
            alive = configs
            while True:
                scored = sorted(((objective(c, b), i, c) for i, c in enumerate(alive)), key=lambda t: t[0])
                spent += b * len(alive)
                self.trials += [{"config": c, "budget": b, "loss": l} for l, _, c in scored]
                if len(alive) == 1 or b >= budget:
                    break
                alive = [c for _, _, c in scored[:max(1, len(alive) // eta)]]
                b = min(budget, b * eta)
            best = scored[0]
            return {"best_config": best[2], "best_loss": best[0], "budget_spent": spent, "trials": len(self.trials)}
        best, since = (math.inf, None), 0
        for c in configs:
            l = objective(c, budget)
            spent += budget
            self.trials.append({"config": c, "budget": budget, "loss": l})
            if l < best[0]:
                best, since = (l, c), 0
            else:
                since += 1
                if early_stopping_patience and since >= early_stopping_patience:
                    break
        return {"best_config": best[1], "best_loss": best[0], "budget_spent": spent, "trials": len(self.trials)}


class NeuralOptimizer(torch.nn.Module):
    """A learned coordinate-wise update rule: a small MLP maps ``(gradient, momentum)`` features (log-magnitude and sign)
    to an update; meta-trained by unrolling it on random quadratics (``meta_train``)."""

    def __init__(self, hidden: int = 16, beta: float = 0.9, out_scale: float = 0.1):
        super().__init__()
        self.net = torch.nn.Sequential(torch.nn.Linear(4, hidden), torch.nn.Tanh(), torch.nn.Linear(hidden, 1))
        self.beta, self.out_scale = beta, out_scale
        with torch.no_grad():
            self.net[-1].weight.mul_(0.1)

    @staticmethod
    def _feat(x):
        return torch.stack([torch.log(x.abs() + 1e-8) / 10, torch.sign(x)], -1)

    def update(self, grad, mom):
        mom = self.beta * mom + (1 - self.beta) * grad
        f = torch.cat([self._feat(grad), self._feat(mom)], -1)
        return self.out_scale * self.net(f).squeeze(-1) * (mom.abs() + 1e-8), mom

    def meta_train(self, dim: int = 8, unroll: int = 20, iters: int = 150, lr: float = 1e-2, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        opt = torch.optim.Adam(self.parameters(), lr)
        hist = []
        for _ in range(iters):
            a = torch.rand(dim, generator=g) * 2 + 0.1
            x, mom, total = torch.randn(dim, generator=g), torch.zeros(dim), 0.0
            for _ in range(unroll):
                grad = a * x
                step, mom = self.update(grad, mom)
                x = x + step
                total = total + 0.5 * (a * x * x).sum()
            opt.zero_grad()
            total.backward()
            torch.nn.utils.clip_grad_norm_(self.parameters(), 1.0)
            opt.step()
            hist.append(float(total.detach()))
        return hist

    @torch.no_grad()
    def apply(self, params, state: dict):
        for p in params:
            if p.grad is None:
                continue
            step, state[p] = self.update(p.grad, state.get(p, torch.zeros_like(p)))
            p.add_(step)


class MetaOptimizer:
    """Chooses an optimizer configuration for a new task from the most similar recorded task (cosine similarity of task
    feature vectors such as size, conditioning, noise, sparsity) and records outcomes to improve later choices."""

    def __init__(self):
        self.memory: list[dict] = []

    @staticmethod
    def characterize(grad_samples: torch.Tensor) -> dict:
        """``grad_samples``: ``[k, n]`` gradients at ``k`` mini-batches of one point."""
        mean, std = grad_samples.mean(0), grad_samples.std(0)
        return {"log_dim": math.log10(grad_samples.shape[1]), "noise": float(std.norm() / mean.norm().clamp(min=1e-12)),
                "sparsity": float((grad_samples.abs() < 1e-8).float().mean()),
                "scale_spread": float(torch.log10(mean.abs().clamp(min=1e-12)).std())}

    def record(self, features: dict, config: dict, final_loss: float): self.memory.append({"features": features, "config": config, "loss": final_loss})

    def recommend(self, features: dict, default: dict | None = None) -> dict:
        if not self.memory:
            return default or {"optimizer": "adam", "lr": 1e-3}
        keys = sorted(features)
        v = np.array([features[k] for k in keys])
        def sim(m):
            u = np.array([m["features"][k] for k in keys])
            return float(u @ v / max(np.linalg.norm(u) * np.linalg.norm(v), 1e-12)) - 1e-3 * m["loss"]
        return dict(max(self.memory, key=sim)["config"])


# ================================================================================================ robustness / energy
class RobustnessManager(_Mixin):
    """Guards a step: non-finite gradients are skipped, gradient norm is clipped, a loss spike larger than ``spike_factor``
    times the running median rolls parameters and optimizer state back to the last good snapshot and halves the learning rate."""

    def __init__(self, base, max_grad_norm: float | None = 1.0, spike_factor: float = 10.0, snapshot_every: int = 10):
        self.base, self.param_groups = base, base.param_groups
        self.max_norm, self.spike, self.every = max_grad_norm, spike_factor, snapshot_every
        self.losses, self.stats, self._snap, self.t = [], {"skipped": 0, "clipped": 0, "rollbacks": 0}, None, 0
        self._snapshot()

    def _snapshot(self):
        self._snap = ([p.detach().clone() for p in _params(self.base)], copy.deepcopy(self.base.state_dict()))

    def zero_grad(self, set_to_none=True): self.base.zero_grad(set_to_none)

    @torch.no_grad()
    def step(self, loss: float) -> str:
        ps = [p for p in _params(self.base) if p.grad is not None]
        if not math.isfinite(loss) or any(not torch.isfinite(p.grad).all() for p in ps):
            self.stats["skipped"] += 1
            return "skipped"
        if len(self.losses) >= 5 and loss > self.spike * float(np.median(self.losses[-20:])):
            for p, s in zip(_params(self.base), self._snap[0]):
                p.copy_(s)
            self.base.load_state_dict(copy.deepcopy(self._snap[1]))
            for g in self.base.param_groups:
                g["lr"] *= 0.5
            self.param_groups = self.base.param_groups
            self.stats["rollbacks"] += 1
            return "rolled_back"
        if self.max_norm is not None and float(torch.nn.utils.clip_grad_norm_(ps, self.max_norm)) > self.max_norm:
            self.stats["clipped"] += 1
        self.base.step()
        self.losses.append(loss)
        self.t += 1
        if self.t % self.every == 0:
            self._snapshot()
        return "ok"


class EnergyAwareOptimizer(_Mixin):
    """Meters energy per step from a power reader (``read_power() -> watts``; NVML on a GPU box, a constant otherwise),
    converts to CO2 with a grid intensity in g/kWh, and under a power cap or carbon budget skips a fraction of steps
    (gradients keep accumulating, so skipped work is merged into the next step)."""

    def __init__(self, base, read_power: Callable[[], float], carbon_intensity: float = 400.0, power_cap: float | None = None,
                 carbon_budget_g: float | None = None, clock: Callable[[], float] = time.perf_counter):
        self.base, self.param_groups, self.read_power, self.intensity = base, base.param_groups, read_power, carbon_intensity
        self.cap, self.budget, self.clock = power_cap, carbon_budget_g, clock
        self.energy_j, self.steps, self.deferred, self._last = 0.0, 0, 0, clock()

    @property
    def carbon_g(self): return self.energy_j / 3.6e6 * self.intensity
    def zero_grad(self, set_to_none=True): self.base.zero_grad(set_to_none)

    def step(self) -> bool:
        now, watts = self.clock(), self.read_power()
        self.energy_j += watts * (now - self._last)
        self._last = now
        if self.budget is not None and self.carbon_g >= self.budget:
            raise RuntimeError(f"carbon budget of {self.budget} g spent ({self.carbon_g:.3f} g)")
        if self.cap is not None and watts > self.cap and self.deferred < 3:
            self.deferred += 1
            return False
        self.deferred = 0
        self.base.step()
        self.steps += 1
        return True

    def metrics(self): return {"energy_kwh": self.energy_j / 3.6e6, "carbon_g": self.carbon_g, "steps": self.steps, "j_per_step": self.energy_j / max(self.steps, 1)}


# ================================================================================================ neuromorphic
class STDPOptimizer:
    """Pair-based spike-timing-dependent plasticity for a weight matrix ``[post, pre]`` with exponential traces:
    a post spike potentiates by the pre trace, a pre spike depresses by the post trace."""

    def __init__(self, weight: torch.Tensor, a_plus=0.01, a_minus=0.012, tau_plus=20.0, tau_minus=20.0, w_min=0.0, w_max=1.0):
        self.w, self.ap, self.am, self.tp, self.tm, self.lo, self.hi = weight, a_plus, a_minus, tau_plus, tau_minus, w_min, w_max
        self.pre_trace, self.post_trace = torch.zeros(weight.shape[1]), torch.zeros(weight.shape[0])

    @torch.no_grad()
    def step(self, pre_spikes: torch.Tensor, post_spikes: torch.Tensor, dt: float = 1.0):
        self.pre_trace.mul_(math.exp(-dt / self.tp))
        self.post_trace.mul_(math.exp(-dt / self.tm))
        self.w += self.ap * torch.outer(post_spikes.float(), self.pre_trace) - self.am * torch.outer(self.post_trace, pre_spikes.float())
        self.pre_trace += pre_spikes.float()
        self.post_trace += post_spikes.float()
        self.w.clamp_(self.lo, self.hi)


class EventDrivenOptimizer(_Mixin):
    """Applies SGD only to coordinates whose accumulated gradient crosses ``threshold`` (an integrate-and-fire rule per
    weight); the accumulated value is spent by the update."""

    def __init__(self, params, lr=0.1, threshold=0.05, leak=0.0):
        self.params, self.threshold, self.leak = list(params), threshold, leak
        self.param_groups = [{"params": self.params, "lr": lr}]
        self.potential = [torch.zeros_like(p) for p in self.params]
        self.events = self.coords = 0

    @torch.no_grad()
    def step(self):
        for p, v in zip(self.params, self.potential):
            if p.grad is None:
                continue
            v.mul_(1 - self.leak).add_(p.grad)
            fire = v.abs() >= self.threshold
            p.add_(torch.where(fire, v, torch.zeros_like(v)), alpha=-self.param_groups[0]["lr"])
            v.masked_fill_(fire, 0.0)
            self.events += int(fire.sum())
            self.coords += v.numel()

    def event_rate(self): return self.events / max(self.coords, 1)


# ================================================================================================ quantum-inspired search
class QuantumAnnealing:
    """Simulated quantum annealing: ``replicas`` coupled copies (Trotter slices) under Metropolis moves; the coupling
    that pulls neighbouring replicas together grows as the transverse field ``gamma`` decays."""

    def __init__(self, dim: int, bounds=(-5.0, 5.0), replicas: int = 8, steps: int = 400, t: float = 0.1, gamma0: float = 3.0, seed: int = 0):
        self.dim, self.lo, self.hi, self.p, self.steps, self.t, self.g0 = dim, bounds[0], bounds[1], replicas, steps, t, gamma0
        self.rng = np.random.default_rng(seed)

    def minimize(self, f: Callable[[np.ndarray], float]) -> dict:
        x = self.rng.uniform(self.lo, self.hi, (self.p, self.dim))
        e = np.array([f(v) for v in x])
        best = (e.min(), x[e.argmin()].copy())
        for s in range(self.steps):
            frac = s / self.steps
            gamma = self.g0 * (1 - frac) + 1e-3
            coupling = -0.5 * self.p * self.t * math.log(math.tanh(gamma / (self.p * self.t)))
            width = (self.hi - self.lo) * 0.2 * (1 - frac) + 1e-3
            for k in range(self.p):
                cand = np.clip(x[k] + self.rng.normal(0, width, self.dim), self.lo, self.hi)
                ec = f(cand)
                nb = x[(k - 1) % self.p], x[(k + 1) % self.p]
                d_couple = coupling * (sum(((cand - n) ** 2).sum() for n in nb) - sum(((x[k] - n) ** 2).sum() for n in nb)) / self.dim
                if (ec - e[k]) / self.p + d_couple * 1e-2 < 0 or self.rng.random() < math.exp(-((ec - e[k]) / self.p + d_couple * 1e-2) / self.t):
                    x[k], e[k] = cand, ec
                    if ec < best[0]:
                        best = (ec, cand.copy())
        return {"x": best[1], "fun": float(best[0]), "evaluations": self.p * (self.steps + 1)}


class QuantumPSO:
    """Quantum-behaved particle swarm: particles are drawn around an attractor between personal and global bests with a
    spread set by the distance to the mean best position (no velocities)."""

    def __init__(self, dim: int, bounds=(-5.0, 5.0), particles: int = 20, iters: int = 150, seed: int = 0):
        self.dim, self.lo, self.hi, self.n, self.iters, self.rng = dim, bounds[0], bounds[1], particles, iters, np.random.default_rng(seed)

    def minimize(self, f) -> dict:
        x = self.rng.uniform(self.lo, self.hi, (self.n, self.dim))
        pb, pe = x.copy(), np.array([f(v) for v in x])
        for it in range(self.iters):
            beta = 1.0 - 0.5 * it / self.iters
            g, mbest = pb[pe.argmin()], pb.mean(0)
            phi, u = self.rng.random((self.n, self.dim)), self.rng.random((self.n, self.dim))
            attractor = phi * pb + (1 - phi) * g
            sign = np.where(self.rng.random((self.n, self.dim)) < 0.5, -1.0, 1.0)
            x = np.clip(attractor + sign * beta * np.abs(mbest - x) * np.log(1 / np.maximum(u, 1e-12)), self.lo, self.hi)
            e = np.array([f(v) for v in x])
            better = e < pe
            pb[better], pe[better] = x[better], e[better]
        return {"x": pb[pe.argmin()], "fun": float(pe.min()), "evaluations": self.n * (self.iters + 1)}


class QuantumGeneticAlgorithm:
    """Each gene is a qubit angle; measuring gives a bit string, and angles rotate toward the best string seen."""

    def __init__(self, n_bits: int, population: int = 12, iters: int = 80, delta: float = 0.05 * math.pi, seed: int = 0):
        self.n, self.pop, self.iters, self.delta, self.rng = n_bits, population, iters, delta, np.random.default_rng(seed)

    def maximize(self, fitness: Callable[[np.ndarray], float]) -> dict:
        theta = np.full((self.pop, self.n), math.pi / 4)
        best = (-math.inf, None)
        for _ in range(self.iters):
            bits = (self.rng.random((self.pop, self.n)) < np.sin(theta) ** 2).astype(int)
            fit = np.array([fitness(b) for b in bits])
            if fit.max() > best[0]:
                best = (float(fit.max()), bits[fit.argmax()].copy())
            toward = np.where(best[1] == 1, 1.0, -1.0)
            theta = np.clip(theta + self.delta * toward * (bits != best[1]), 0.02, math.pi / 2 - 0.02)
        return {"bits": best[1], "fitness": best[0]}


# ================================================================================================ cross-framework validation
class CrossFrameworkValidator:
    """Runs two optimizers from the same start on the same gradient stream and reports the largest parameter difference
    per step; used to pin this package's optimizers against ``torch.optim``."""

    def __init__(self, rtol: float = 1e-5, atol: float = 1e-7):
        self.rtol, self.atol = rtol, atol

    def validate(self, make_ours, make_theirs, shapes=((4, 3), (3,)), steps: int = 10, seed: int = 0) -> dict:
        g = torch.Generator().manual_seed(seed)
        start = [torch.randn(s, generator=g) for s in shapes]
        a = [torch.nn.Parameter(t.clone()) for t in start]
        b = [torch.nn.Parameter(t.clone()) for t in start]
        oa, ob = make_ours(a), make_theirs(b)
        worst = []
        for _ in range(steps):
            grads = [torch.randn(s, generator=g) for s in shapes]
            for pa, pb, gr in zip(a, b, grads):
                pa.grad, pb.grad = gr.clone(), gr.clone()
            oa.step()
            ob.step()
            worst.append(max(float((pa.detach() - pb.detach()).abs().max()) for pa, pb in zip(a, b)))
        ok = all(torch.allclose(pa, pb, rtol=self.rtol, atol=self.atol) for pa, pb in zip(a, b))
        return {"passed": ok, "max_abs_diff_per_step": worst, "max_abs_diff": max(worst)}
