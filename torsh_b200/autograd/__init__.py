"""Autograd utilities over ``torch.autograd``.

Reference surface: grad-mode guards ``no_grad / enable_grad / inference_mode / detect_anomaly / set_grad_enabled``
(``crates/torsh-autograd/src/grad_mode.rs:51-310``, ``guards.rs:34-156``), ``Function`` with ``FunctionContext``
(``function.rs:19-341``), gradient hooks with priorities (``gradient_hooks.rs:41-385``), clipping strategies
(``gradient_clipping.rs:39-286``), ``clip_grad_norm / clip_grad_value`` (``lib.rs:633-715``), finite-difference
gradcheck (``gradient_checking.rs:17-461``), checkpoint scheduling (``checkpoint_scheduler.rs:15-490``), anomaly
detection (``anomaly_detection.rs``). The reference tape differentiates only add/sub/mul/matmul/pow/mean/sum; here
PyTorch's engine differentiates everything and the kernels plug in as ``torch.autograd.Function``s.
"""
from __future__ import annotations

from enum import Enum

import torch
from torch.autograd import Function, backward, grad
from torch.autograd import detect_anomaly  # noqa: F401
from torch.utils.checkpoint import checkpoint as _checkpoint

no_grad, enable_grad, inference_mode = torch.no_grad, torch.enable_grad, torch.inference_mode
set_grad_enabled, is_grad_enabled = torch.set_grad_enabled, torch.is_grad_enabled
FunctionContext = torch.autograd.function.FunctionCtx

_grad_stack: list[bool] = []


def push_grad_enabled(flag: bool):
    _grad_stack.append(torch.is_grad_enabled())
    torch.set_grad_enabled(flag)


def pop_grad_enabled():
    if _grad_stack:
        torch.set_grad_enabled(_grad_stack.pop())


class ClippingStrategy(Enum):
    NORM = "norm"; L1 = "l1"; VALUE = "value"; ADAPTIVE = "adaptive"


def _grads(params):
    return [p.grad for p in params if p.grad is not None]


def clip_grad_norm(params, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
    """Scales gradients so their global norm is at most ``max_norm``; returns the norm before clipping.
    CUDA fp32/bf16 gradients use the multi-tensor kernels (one sum-of-squares pass, one scale pass)."""
    params = [p for p in params if p.grad is not None]
    if not params:
        return torch.zeros(())
    g0 = params[0].grad
    if norm_type == 2.0 and g0.is_cuda and all(p.grad.dtype == g0.dtype and p.grad.is_contiguous() for p in params) \
            and g0.dtype in (torch.float32, torch.bfloat16):
        from ..ops import multi_tensor as mt
        tt = mt.TensorTable([(p.grad,) for p in params], g0.device)
        sq = torch.zeros(1, dtype=torch.float32, device=g0.device)
        mt.sq_norm(tt, 0, g0.dtype, sq)
        mt.scale_(tt, 0, g0.dtype, clip_sqnorm=sq, max_norm=max_norm)
        return sq.sqrt().squeeze(0)
    return torch.nn.utils.clip_grad_norm_(params, max_norm, norm_type)


def clip_grad_value(params, clip_value: float) -> None:
    torch.nn.utils.clip_grad_value_([p for p in params if p.grad is not None], clip_value)


def clip_gradients(params, strategy: ClippingStrategy, threshold: float, percentile: float = 0.95):
    params = list(params)
    if strategy is ClippingStrategy.NORM:
        return clip_grad_norm(params, threshold)
    if strategy is ClippingStrategy.L1:
        return clip_grad_norm(params, threshold, 1.0)
    if strategy is ClippingStrategy.VALUE:
        return clip_grad_value(params, threshold)
    flat = torch.cat([g.reshape(-1).abs().float() for g in _grads(params)])
    k = max(1, int(percentile * flat.numel()))
    cut = flat.kthvalue(k).values.item()
    return clip_grad_value(params, min(cut, threshold) if threshold > 0 else cut)


def grad_norm(params, norm_type: float = 2.0) -> torch.Tensor:
    gs = _grads(params)
    if not gs:
        return torch.zeros(())
    return torch.norm(torch.stack([g.float().norm(norm_type) for g in gs]), norm_type)


class HookType(Enum):
    PRE_ACCUMULATE = "pre"; POST_ACCUMULATE = "post"


class GradientHookManager:
    """Per-parameter and global gradient hooks with priorities and call statistics."""

    def __init__(self):
        self._global: list[tuple[int, object]] = []
        self.calls = 0

    def register_global(self, fn, priority: int = 0):
        self._global.append((priority, fn))
        self._global.sort(key=lambda t: -t[0])

    def attach(self, param: torch.Tensor, fn=None, hook_type: HookType = HookType.PRE_ACCUMULATE):
        def run(g):
            self.calls += 1
            for _, h in self._global:
                out = h(g)
                g = g if out is None else out
            if fn is not None:
                out = fn(g)
                g = g if out is None else out
            return g
        if hook_type is HookType.POST_ACCUMULATE:
            return param.register_post_accumulate_grad_hook(lambda p: run(p.grad) and None)
        return param.register_hook(run)


def gradcheck(fn, inputs, eps: float = 1e-6, atol: float = 1e-5, rtol: float = 1e-3) -> bool:
    """Finite differences against the analytic gradient (double precision inputs)."""
    return torch.autograd.gradcheck(fn, inputs, eps=eps, atol=atol, rtol=rtol)


def numerical_gradient(fn, x: torch.Tensor, eps: float = 1e-4) -> torch.Tensor:
    x = x.detach().clone().double()
    g = torch.zeros_like(x)
    flat, gf = x.view(-1), g.view(-1)
    for i in range(flat.numel()):
        old = flat[i].item()
        flat[i] = old + eps
        hi = fn(x).item()
        flat[i] = old - eps
        lo = fn(x).item()
        flat[i] = old
        gf[i] = (hi - lo) / (2 * eps)
    return g


class CheckpointStrategy(Enum):
    NONE = "none"; UNIFORM = "uniform"; SQRT = "sqrt"; MEMORY_BUDGET = "memory_budget"


class CheckpointScheduler:
    """Chooses which of ``n`` sequential segments to recompute in backward."""

    def __init__(self, strategy: CheckpointStrategy = CheckpointStrategy.SQRT, every: int = 2, memory_budget_bytes: int = 0):
        self.strategy, self.every, self.budget = strategy, every, memory_budget_bytes

    def plan(self, n: int, activation_bytes: list[int] | None = None) -> list[bool]:
        if self.strategy is CheckpointStrategy.NONE:
            return [False] * n
        if self.strategy is CheckpointStrategy.UNIFORM:
            return [i % self.every == 0 for i in range(n)]
        if self.strategy is CheckpointStrategy.SQRT:
            k = max(1, int(round(n ** 0.5)))
            return [i % k != 0 for i in range(n)]
        sizes = activation_bytes or [1] * n
        order = sorted(range(n), key=lambda i: -sizes[i])
        keep, used = [False] * n, sum(sizes)
        for i in order:
            if used <= self.budget:
                break
            keep[i] = True
            used -= sizes[i]
        return keep


def checkpoint(fn, *args, **kwargs):
    """Recompute ``fn`` in backward instead of storing its activations."""
    kwargs.setdefault("use_reentrant", False)
    return _checkpoint(fn, *args, **kwargs)


def has_nan_or_inf(t: torch.Tensor) -> bool:
    """``crates/torsh-tensor/src/nan_inf_detection.rs:21-290``."""
    return not bool(torch.isfinite(t).all())


class AnomalyDetector:
    """Scans gradients after backward; records the first parameter with a non-finite value."""

    def __init__(self):
        self.events: list[dict] = []

    def check(self, named_params) -> bool:
        ok = True
        for name, p in named_params:
            g = p.grad if p.grad is not None else getattr(p, "main_grad", None)
            if g is not None and has_nan_or_inf(g):
                self.events.append({"parameter": name, "kind": "non_finite_gradient"})
                ok = False
        return ok
