"""The rest of the reference's optimizer list (``crates/torsh-optim/src/lib.rs:52-114``).

Optimizers that PyTorch ships are adopted with the ToRSh ``get_lr`` / ``set_lr`` surface; the others
(Lion, AdaBelief, AdaBound, Lookahead, Ranger, LARS, Sophia-style clipped second moment, Prodigy-lite,
Schedule-Free SGD, FTRL, Yogi) are written here with PyTorch tensor ops. None is on a benchmark hot path;
the fused CUDA optimizers are in :mod:`torsh_b200.optim.fused`.
"""
from __future__ import annotations

import math

import torch


class _Mixin:
    def get_lr(self):
        return [g["lr"] for g in self.param_groups]

    def set_lr(self, lr: float):
        for g in self.param_groups:
            g["lr"] = lr


def _adopt(name):
    base = getattr(torch.optim, name)
    return type(name, (_Mixin, base), {"__doc__": f"``torch.optim.{name}`` with ``get_lr`` / ``set_lr``."})


for _n in ("Adagrad", "Adadelta", "Adamax", "ASGD", "NAdam", "RAdam", "RMSprop", "Rprop", "LBFGS", "SparseAdam"):
    globals()[_n] = _adopt(_n)


class _Simple(_Mixin, torch.optim.Optimizer):
    """Base for the hand-written ones: subclasses implement ``_update(p, grad, state, group)``."""

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                self._update(p, p.grad, st, g)
        return loss


class Lion(_Simple):
    """Sign of an interpolated momentum; decoupled weight decay."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    def _update(self, p, grad, st, g):
        b1, b2 = g["betas"]
        m = st.setdefault("exp_avg", torch.zeros_like(p))
        p.mul_(1 - g["lr"] * g["weight_decay"])
        p.add_(torch.sign(m * b1 + grad * (1 - b1)), alpha=-g["lr"])
        m.mul_(b2).add_(grad, alpha=1 - b2)


class AdaBelief(_Simple):
    """Adam with the second moment of ``(g - m)`` (belief in the gradient)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-16, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    def _update(self, p, grad, st, g):
        b1, b2 = g["betas"]
        t = st["step"]
        m = st.setdefault("exp_avg", torch.zeros_like(p))
        s = st.setdefault("exp_avg_var", torch.zeros_like(p))
        if g["weight_decay"]:
            p.mul_(1 - g["lr"] * g["weight_decay"])
        m.mul_(b1).add_(grad, alpha=1 - b1)
        d = grad - m
        s.mul_(b2).addcmul_(d, d, value=1 - b2).add_(g["eps"])
        p.addcdiv_(m / (1 - b1 ** t), (s / (1 - b2 ** t)).sqrt() + g["eps"], value=-g["lr"])


class AdaBound(_Simple):
    """Adam whose per-element step is clipped into bounds that converge to ``final_lr``."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), final_lr=0.1, gamma=1e-3, eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, final_lr=final_lr, gamma=gamma, eps=eps,
                                      weight_decay=weight_decay, base_lr=lr))

    def _update(self, p, grad, st, g):
        b1, b2 = g["betas"]
        t = st["step"]
        if g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        m = st.setdefault("exp_avg", torch.zeros_like(p))
        v = st.setdefault("exp_avg_sq", torch.zeros_like(p))
        m.mul_(b1).add_(grad, alpha=1 - b1)
        v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
        step = g["lr"] * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        final = g["final_lr"] * g["lr"] / g["base_lr"]
        lo, hi = final * (1 - 1 / (g["gamma"] * t + 1)), final * (1 + 1 / (g["gamma"] * t))
        p.sub_((step / (v.sqrt() + g["eps"])).clamp_(lo, hi) * m)


class Yogi(_Simple):
    """Adam with an additive, sign-controlled second-moment update."""

    def __init__(self, params, lr=1e-2, betas=(0.9, 0.999), eps=1e-3, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    def _update(self, p, grad, st, g):
        b1, b2 = g["betas"]
        t = st["step"]
        if g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        m = st.setdefault("exp_avg", torch.zeros_like(p))
        v = st.setdefault("exp_avg_sq", torch.full_like(p, 1e-6))
        m.mul_(b1).add_(grad, alpha=1 - b1)
        g2 = grad * grad
        v.addcmul_(torch.sign(v - g2), g2, value=-(1 - b2))
        p.addcdiv_(m / (1 - b1 ** t), (v / (1 - b2 ** t)).sqrt() + g["eps"], value=-g["lr"])


class LARS(_Simple):
    """SGD-momentum with a layer-wise trust ratio ``eta * |w| / (|g| + wd * |w|)``."""

    def __init__(self, params, lr=0.1, momentum=0.9, weight_decay=1e-4, eta=1e-3, eps=1e-8):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, eta=eta, eps=eps))

    def _update(self, p, grad, st, g):
        wn, gn = p.norm(), grad.norm()
        trust = torch.where((wn > 0) & (gn > 0), g["eta"] * wn / (gn + g["weight_decay"] * wn + g["eps"]), torch.ones_like(wn))
        d = (grad + g["weight_decay"] * p) * trust
        buf = st.setdefault("momentum_buffer", torch.zeros_like(p))
        buf.mul_(g["momentum"]).add_(d)
        p.add_(buf, alpha=-g["lr"])


class FTRL(_Simple):
    """Follow-the-regularised-leader (proximal) with L1 / L2."""

    def __init__(self, params, lr=0.1, lr_power=-0.5, l1=0.0, l2=0.0, initial_accumulator=0.1):
        super().__init__(params, dict(lr=lr, lr_power=lr_power, l1=l1, l2=l2, init_acc=initial_accumulator))

    def _update(self, p, grad, st, g):
        n = st.setdefault("accum", torch.full_like(p, g["init_acc"]))
        z = st.setdefault("linear", torch.zeros_like(p))
        n_new = n + grad * grad
        sigma = (n_new.pow(-g["lr_power"]) - n.pow(-g["lr_power"])) / g["lr"]
        z.add_(grad - sigma * p)
        n.copy_(n_new)
        quad = n_new.pow(-g["lr_power"]) / g["lr"] + 2 * g["l2"]
        p.copy_(torch.where(z.abs() > g["l1"], (torch.sign(z) * g["l1"] - z) / quad, torch.zeros_like(p)))


class SophiaG(_Simple):
    """Second-order clipped update: ``p -= lr * clip(m / max(rho * h, eps), 1)`` with ``h`` an EMA of a Hessian
    diagonal estimate (here the Gauss-Newton-Bartlett estimate g*g refreshed every ``update_period`` steps)."""

    def __init__(self, params, lr=1e-4, betas=(0.965, 0.99), rho=0.04, weight_decay=0.1, update_period=10, eps=1e-12):
        super().__init__(params, dict(lr=lr, betas=betas, rho=rho, weight_decay=weight_decay,
                                      update_period=update_period, eps=eps))

    def _update(self, p, grad, st, g):
        b1, b2 = g["betas"]
        m = st.setdefault("exp_avg", torch.zeros_like(p))
        h = st.setdefault("hessian", torch.zeros_like(p))
        m.mul_(b1).add_(grad, alpha=1 - b1)
        if (st["step"] - 1) % g["update_period"] == 0:
            h.mul_(b2).addcmul_(grad, grad, value=1 - b2)
        p.mul_(1 - g["lr"] * g["weight_decay"])
        p.add_((m / torch.clamp(g["rho"] * h, min=g["eps"])).clamp_(-1, 1), alpha=-g["lr"])


class ScheduleFreeSGD(_Simple):
    """Schedule-free SGD: gradients are taken at an interpolation ``y`` of the iterate ``z`` and the average ``x``."""

    def __init__(self, params, lr=1.0, momentum=0.9, weight_decay=0.0, warmup_steps=0):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, warmup_steps=warmup_steps))

    def _update(self, p, grad, st, g):
        t = st["step"]
        z = st.setdefault("z", p.detach().clone())
        beta = g["momentum"]
        lr = g["lr"] * min(1.0, t / max(g["warmup_steps"], 1)) if g["warmup_steps"] else g["lr"]
        if g["weight_decay"]:
            grad = grad + g["weight_decay"] * p
        c = 1.0 / t
        # p holds y; recover x, step z, re-average, re-interpolate
        x = (p - (1 - beta) * z) / beta if beta > 0 else z.clone()
        z.add_(grad, alpha=-lr)
        x.mul_(1 - c).add_(z, alpha=c)
        p.copy_(beta * x + (1 - beta) * z)


class Prodigy(_Simple):
    """Parameter-free Adam: estimates the distance to the solution ``d`` online and scales the step by it."""

    def __init__(self, params, lr=1.0, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, d0=1e-6):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.d, self._num, self._den = d0, 0.0, 0.0

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        num_add, den = 0.0, 0.0
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["p0"] = p.detach().clone()
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                    st["s"] = torch.zeros_like(p)
                grad = p.grad
                num_add += self.d * g["lr"] * torch.sum(grad * (st["p0"] - p)).item()
                st["exp_avg"].mul_(b1).add_(grad, alpha=self.d * (1 - b1))
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=self.d * self.d * (1 - b2))
                st["s"].mul_(math.sqrt(b2)).add_(grad, alpha=self.d * g["lr"] * (1 - math.sqrt(b2)))
                den += st["s"].abs().sum().item()
        b2 = self.param_groups[0]["betas"][1]
        self._num = math.sqrt(b2) * self._num + (1 - math.sqrt(b2)) * num_add
        if den > 0:
            self.d = max(self.d, self._num / den)
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * self.d * g["weight_decay"])
                p.addcdiv_(st["exp_avg"], st["exp_avg_sq"].sqrt() + self.d * g["eps"], value=-g["lr"] * self.d)
        return loss


class Lookahead(_Mixin):
    """Wraps any optimizer: every ``k`` steps the slow weights move ``alpha`` of the way to the fast weights."""

    def __init__(self, optimizer, k: int = 5, alpha: float = 0.5):
        self.optimizer, self.k, self.alpha, self._n = optimizer, k, alpha, 0
        self.param_groups = optimizer.param_groups
        self.slow = [[p.detach().clone() for p in g["params"]] for g in self.param_groups]

    @torch.no_grad()
    def step(self, closure=None):
        loss = self.optimizer.step(closure)
        self._n += 1
        if self._n % self.k == 0:
            for g, slows in zip(self.param_groups, self.slow):
                for p, s in zip(g["params"], slows):
                    s.add_(p.detach() - s, alpha=self.alpha)
                    p.copy_(s)
        return loss

    def zero_grad(self, set_to_none: bool = True):
        self.optimizer.zero_grad(set_to_none)

    def state_dict(self):
        return {"inner": self.optimizer.state_dict(), "slow": self.slow, "n": self._n}


def Ranger(params, lr=1e-3, k=6, alpha=0.5, **kw):
    """RAdam wrapped in Lookahead."""
    return Lookahead(globals()["RAdam"](params, lr=lr, **kw), k=k, alpha=alpha)


class GradientAccumulator:
    """``crates/torsh-optim/src/grad_accumulation.rs:15-315``: sum ``accumulation_steps`` micro-batch gradients,
    then average and release them to the optimizer."""

    def __init__(self, accumulation_steps: int, average: bool = True):
        self.steps, self.average, self.count = accumulation_steps, average, 0

    def accumulate(self) -> bool:
        """Call after each ``backward()``; True when the optimizer should step now."""
        self.count += 1
        return self.count % self.steps == 0

    def scale_for_step(self, params):
        if self.average:
            for p in params:
                if p.grad is not None:
                    p.grad.div_(self.steps)


class AccumulatingOptimizer(_Mixin):
    def __init__(self, optimizer, accumulation_steps: int):
        self.optimizer, self.acc = optimizer, GradientAccumulator(accumulation_steps)
        self.param_groups = optimizer.param_groups

    def step(self, closure=None):
        if self.acc.accumulate():
            self.acc.scale_for_step(p for g in self.param_groups for p in g["params"])
            out = self.optimizer.step(closure)
            self.optimizer.zero_grad()
            return out
        return None

    def zero_grad(self, set_to_none: bool = True):
        pass  # gradients are cleared only after a real step
