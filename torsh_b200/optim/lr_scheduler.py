"""Learning-rate schedulers (``crates/torsh-optim/src/lr_scheduler.rs:136-598``,
``lr_scheduler_additional.rs:9-544``, ``lr_scheduler_enhanced.rs:19-559``): StepLR, MultiStepLR, ExponentialLR,
CosineAnnealingLR, CosineAnnealingWarmRestarts (+warm-up), ReduceLROnPlateau, OneCycleLR, CyclicLR, PolynomialLR,
LinearLR, ConstantLR, PolynomialDecayWithWarmup, AdaptiveLRScheduler.

They drive anything with ``param_groups`` (the fused optimizers, the flat optimizers, PyTorch optimizers).
"""
from __future__ import annotations

import math


class LRScheduler:
    def __init__(self, optimizer, last_epoch: int = -1):
        self.optimizer = optimizer
        self.base_lrs = [g["lr"] for g in optimizer.param_groups]
        self.last_epoch = last_epoch
        self.step()

    def get_lr(self) -> list[float]:
        raise NotImplementedError

    def get_last_lr(self) -> list[float]:
        return [g["lr"] for g in self.optimizer.param_groups]

    def step(self, epoch: int | None = None):
        self.last_epoch = self.last_epoch + 1 if epoch is None else epoch
        for g, lr in zip(self.optimizer.param_groups, self.get_lr()):
            g["lr"] = lr

    def state_dict(self) -> dict:
        return {k: v for k, v in self.__dict__.items() if k != "optimizer" and not callable(v)}

    def load_state_dict(self, sd: dict):
        self.__dict__.update(sd)


class StepLR(LRScheduler):
    def __init__(self, optimizer, step_size: int, gamma: float = 0.1, last_epoch: int = -1):
        self.step_size, self.gamma = step_size, gamma
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        return [b * self.gamma ** (self.last_epoch // self.step_size) for b in self.base_lrs]


class MultiStepLR(LRScheduler):
    def __init__(self, optimizer, milestones, gamma: float = 0.1, last_epoch: int = -1):
        self.milestones, self.gamma = sorted(milestones), gamma
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        k = sum(1 for m in self.milestones if m <= self.last_epoch)
        return [b * self.gamma ** k for b in self.base_lrs]


class ExponentialLR(LRScheduler):
    def __init__(self, optimizer, gamma: float, last_epoch: int = -1):
        self.gamma = gamma
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        return [b * self.gamma ** self.last_epoch for b in self.base_lrs]


class CosineAnnealingLR(LRScheduler):
    def __init__(self, optimizer, T_max: int, eta_min: float = 0.0, last_epoch: int = -1):
        self.T_max, self.eta_min = T_max, eta_min
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        c = (1 + math.cos(math.pi * self.last_epoch / self.T_max)) / 2
        return [self.eta_min + (b - self.eta_min) * c for b in self.base_lrs]


class CosineAnnealingWarmRestarts(LRScheduler):
    def __init__(self, optimizer, T_0: int, T_mult: int = 1, eta_min: float = 0.0, warmup_steps: int = 0,
                 last_epoch: int = -1):
        self.T_0, self.T_mult, self.eta_min, self.warmup_steps = T_0, T_mult, eta_min, warmup_steps
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        t = self.last_epoch
        if t < self.warmup_steps:
            return [b * (t + 1) / self.warmup_steps for b in self.base_lrs]
        t -= self.warmup_steps
        T_i = self.T_0
        while t >= T_i:
            t -= T_i
            T_i *= self.T_mult
        c = (1 + math.cos(math.pi * t / T_i)) / 2
        return [self.eta_min + (b - self.eta_min) * c for b in self.base_lrs]


CosineAnnealingWarmRestartsWithWarmup = CosineAnnealingWarmRestarts


class LinearLR(LRScheduler):
    def __init__(self, optimizer, start_factor: float = 1.0 / 3, end_factor: float = 1.0, total_iters: int = 5,
                 last_epoch: int = -1):
        self.start_factor, self.end_factor, self.total_iters = start_factor, end_factor, total_iters
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        f = min(self.last_epoch, self.total_iters) / self.total_iters
        k = self.start_factor + (self.end_factor - self.start_factor) * f
        return [b * k for b in self.base_lrs]


class ConstantLR(LRScheduler):
    def __init__(self, optimizer, factor: float = 1.0 / 3, total_iters: int = 5, last_epoch: int = -1):
        self.factor, self.total_iters = factor, total_iters
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        return [b * (self.factor if self.last_epoch < self.total_iters else 1.0) for b in self.base_lrs]


class PolynomialLR(LRScheduler):
    def __init__(self, optimizer, total_iters: int = 5, power: float = 1.0, last_epoch: int = -1):
        self.total_iters, self.power = total_iters, power
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        f = (1 - min(self.last_epoch, self.total_iters) / self.total_iters) ** self.power
        return [b * f for b in self.base_lrs]


class PolynomialDecayWithWarmup(LRScheduler):
    def __init__(self, optimizer, warmup_steps: int, total_steps: int, end_lr: float = 0.0, power: float = 1.0,
                 last_epoch: int = -1):
        self.warmup_steps, self.total_steps, self.end_lr, self.power = warmup_steps, total_steps, end_lr, power
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        t = self.last_epoch
        if t < self.warmup_steps:
            return [b * (t + 1) / max(self.warmup_steps, 1) for b in self.base_lrs]
        p = min(1.0, (t - self.warmup_steps) / max(self.total_steps - self.warmup_steps, 1))
        return [(b - self.end_lr) * (1 - p) ** self.power + self.end_lr for b in self.base_lrs]


class OneCycleLR(LRScheduler):
    def __init__(self, optimizer, max_lr: float, total_steps: int, pct_start: float = 0.3, div_factor: float = 25.0,
                 final_div_factor: float = 1e4, anneal_strategy: str = "cos", last_epoch: int = -1):
        self.max_lr, self.total_steps, self.pct_start = max_lr, total_steps, pct_start
        self.initial_lr, self.min_lr = max_lr / div_factor, max_lr / div_factor / final_div_factor
        self.anneal = anneal_strategy
        super().__init__(optimizer, last_epoch)

    def _interp(self, a, b, p):
        return b + (a - b) * (1 + math.cos(math.pi * p)) / 2 if self.anneal == "cos" else a + (b - a) * p

    def get_lr(self):
        t = min(self.last_epoch, self.total_steps - 1)
        up = max(1.0, self.pct_start * self.total_steps - 1)
        if t <= up:
            lr = self._interp(self.initial_lr, self.max_lr, t / up)
        else:
            lr = self._interp(self.max_lr, self.min_lr, (t - up) / max(self.total_steps - 1 - up, 1))
        return [lr for _ in self.base_lrs]


class CyclicLR(LRScheduler):
    def __init__(self, optimizer, base_lr: float, max_lr: float, step_size_up: int = 2000, step_size_down: int | None = None,
                 mode: str = "triangular", gamma: float = 1.0, last_epoch: int = -1):
        self.lo, self.hi, self.up = base_lr, max_lr, step_size_up
        self.down = step_size_down or step_size_up
        self.mode, self.gamma = mode, gamma
        super().__init__(optimizer, last_epoch)

    def get_lr(self):
        total = self.up + self.down
        cycle = self.last_epoch // total
        x = self.last_epoch % total
        frac = x / self.up if x <= self.up else 1 - (x - self.up) / self.down
        scale = {"triangular": 1.0, "triangular2": 1 / 2 ** cycle, "exp_range": self.gamma ** self.last_epoch}[self.mode]
        return [self.lo + (self.hi - self.lo) * frac * scale for _ in self.base_lrs]


class ReduceLROnPlateau:
    def __init__(self, optimizer, mode: str = "min", factor: float = 0.1, patience: int = 10, threshold: float = 1e-4,
                 cooldown: int = 0, min_lr: float = 0.0):
        self.optimizer, self.mode, self.factor, self.patience = optimizer, mode, factor, patience
        self.threshold, self.cooldown, self.min_lr = threshold, cooldown, min_lr
        self.best = math.inf if mode == "min" else -math.inf
        self.bad, self.cool = 0, 0

    def step(self, metric: float):
        better = metric < self.best * (1 - self.threshold) if self.mode == "min" else metric > self.best * (1 + self.threshold)
        if better:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
        if self.cool > 0:
            self.cool -= 1
            self.bad = 0
        if self.bad > self.patience:
            for g in self.optimizer.param_groups:
                g["lr"] = max(g["lr"] * self.factor, self.min_lr)
            self.cool, self.bad = self.cooldown, 0

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]


class AdaptiveLRScheduler:
    """Raises the rate while the loss keeps falling, cuts it when the loss rises
    (``crates/torsh-optim/src/lr_scheduler_enhanced.rs``)."""

    def __init__(self, optimizer, increase: float = 1.05, decrease: float = 0.7, window: int = 5, min_lr: float = 1e-7,
                 max_lr: float = 1.0):
        self.optimizer, self.increase, self.decrease, self.window = optimizer, increase, decrease, window
        self.min_lr, self.max_lr, self.history = min_lr, max_lr, []

    def step(self, loss: float):
        self.history.append(loss)
        if len(self.history) <= self.window:
            return
        recent = sum(self.history[-self.window:]) / self.window
        prev = sum(self.history[-self.window - 1:-1]) / self.window
        k = self.increase if recent < prev else self.decrease
        for g in self.optimizer.param_groups:
            g["lr"] = min(max(g["lr"] * k, self.min_lr), self.max_lr)
