"""Loss scaling and mixed-precision optimizer wrappers (``crates/torsh-optim/src/mixed_precision.rs:18-419``,
``crates/torsh-nn/src/mixed_precision.rs:23-517``, ``crates/torsh-backend/src/cuda/mixed_precision.rs:13-494``).

``GradScaler``: dynamic loss scale (init 65536, growth x2 every 2000 clean steps, backoff x0.5 on overflow).  On a GPU
``unscale_`` is ONE multi-tensor kernel over all gradients that multiplies by 1/scale and raises a device flag when a
value is not finite; the host reads that flag once per step.  ``MixedPrecisionOptimizer`` keeps fp32 master weights for
low-precision parameters, steps the masters and copies them back.  bf16 training needs no scaling
(``BF16Config``)."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class MixedPrecisionConfig:
    enabled: bool = True
    dtype: torch.dtype = torch.bfloat16
    init_scale: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000
    min_scale: float = 1.0
    max_scale: float = 2.0 ** 24
    dynamic: bool = True


BF16Config = lambda **kw: MixedPrecisionConfig(dtype=torch.bfloat16, dynamic=False, init_scale=1.0, **kw)  # noqa: E731


class GradScaler:
    def __init__(self, config: MixedPrecisionConfig | None = None, **kw):
        self.cfg = config or MixedPrecisionConfig(**kw)
        self.scale_value = self.cfg.init_scale
        self._good_steps = 0
        self._found_inf: torch.Tensor | None = None
        self._tables: dict = {}
        self.stats = {"steps": 0, "skipped": 0, "growths": 0, "backoffs": 0}

    def get_scale(self) -> float:
        return self.scale_value

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self.scale_value if self.cfg.enabled else loss

    def unscale_(self, optimizer) -> bool:
        """Divide every gradient by the scale; returns True when all are finite."""
        params = [p for g in optimizer.param_groups for p in g["params"] if p.grad is not None]
        if not params:
            return True
        inv = 1.0 / self.scale_value
        cuda = [p for p in params if p.grad.is_cuda and p.grad.dtype in (torch.float32, torch.bfloat16) and p.grad.is_contiguous()]
        rest = [p for p in params if p not in cuda]
        finite = True
        if cuda:
            from ..ops import multi_tensor as mt
            dev = cuda[0].device
            if self._found_inf is None or self._found_inf.device != dev:
                self._found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
            self._found_inf.zero_()
            by_dtype: dict = {}
            for p in cuda:
                by_dtype.setdefault(p.grad.dtype, []).append(p)
            for dt, ps in by_dtype.items():
                tt = mt.TensorTable.cached(self._tables, str(dt), [(p.grad,) for p in ps], dev)
                mt.scale_(tt, 0, dt, inv, found_inf=self._found_inf)
            finite = int(self._found_inf.item()) == 0
        for p in rest:
            p.grad.mul_(inv)
            finite = finite and bool(torch.isfinite(p.grad).all())
        return finite

    def step(self, optimizer, unscaled: bool | None = None) -> bool:
        """Unscale (unless already done), step when finite, update the scale. Returns whether the step was taken."""
        finite = self.unscale_(optimizer) if unscaled is None else unscaled
        self.stats["steps"] += 1
        if finite:
            optimizer.step()
        else:
            self.stats["skipped"] += 1
        self.update(finite)
        return finite

    def update(self, finite: bool) -> None:
        if not self.cfg.dynamic:
            return
        if finite:
            self._good_steps += 1
            if self._good_steps >= self.cfg.growth_interval:
                self.scale_value = min(self.scale_value * self.cfg.growth_factor, self.cfg.max_scale)
                self._good_steps = 0
                self.stats["growths"] += 1
        else:
            self.scale_value = max(self.scale_value * self.cfg.backoff_factor, self.cfg.min_scale)
            self._good_steps = 0
            self.stats["backoffs"] += 1

    def state_dict(self) -> dict:
        return {"scale": self.scale_value, "good_steps": self._good_steps, **self.stats}

    def load_state_dict(self, sd: dict) -> None:
        self.scale_value, self._good_steps = sd["scale"], sd["good_steps"]


DynamicLossScaler = GradScaler


class MixedPrecisionOptimizer:
    """Wraps an optimizer class: low-precision parameters get fp32 master copies which the inner optimizer steps."""

    def __init__(self, params, optimizer_cls, config: MixedPrecisionConfig | None = None, **opt_kw):
        self.cfg = config or MixedPrecisionConfig()
        self.model_params = [p for p in params if p.requires_grad]
        self.masters = [torch.nn.Parameter(p.detach().float().clone()) if p.dtype != torch.float32 else p for p in self.model_params]
        self.inner = optimizer_cls(self.masters, **opt_kw)
        self.scaler = GradScaler(self.cfg)
        self.param_groups = self.inner.param_groups

    def scale_loss(self, loss):
        return self.scaler.scale(loss)

    def zero_grad(self, set_to_none: bool = True):
        for p in self.model_params:
            p.grad = None if set_to_none else (p.grad.zero_() if p.grad is not None else None)
        self.inner.zero_grad(set_to_none)

    @torch.no_grad()
    def step(self) -> bool:
        for p, m in zip(self.model_params, self.masters):
            if m is not p and p.grad is not None:
                m.grad = p.grad.float()
        ok = self.scaler.step(self.inner)
        if ok:
            for p, m in zip(self.model_params, self.masters):
                if m is not p:
                    p.copy_(m)
        return ok


class AutocastModel(torch.nn.Module):
    """Runs the wrapped module under autocast with the configured dtype (fp32 when disabled or on CPU bf16-incapable)."""

    def __init__(self, module: torch.nn.Module, config: MixedPrecisionConfig | None = None):
        super().__init__()
        self.module, self.cfg = module, config or MixedPrecisionConfig()

    def forward(self, *a, **kw):
        dev = next(self.module.parameters()).device.type
        with torch.autocast(dev, dtype=self.cfg.dtype, enabled=self.cfg.enabled):
            return self.module(*a, **kw)


class MixedPrecisionTrainer:
    """``train_step(loss_fn)`` = autocast forward, scaled backward, unscale + clip, guarded step."""

    def __init__(self, model, optimizer, config: MixedPrecisionConfig | None = None, max_grad_norm: float | None = None):
        self.model, self.opt = AutocastModel(model, config), optimizer
        self.scaler, self.max_grad_norm = GradScaler(config), max_grad_norm

    def train_step(self, loss_fn) -> tuple[float, bool]:
        self.opt.zero_grad(set_to_none=True)
        loss = loss_fn(self.model)
        self.scaler.scale(loss).backward()
        finite = self.scaler.unscale_(self.opt)
        if finite and self.max_grad_norm:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_grad_norm)
        self.scaler.step(self.opt, unscaled=finite)
        return float(loss.detach()), finite


BF16Trainer = lambda model, optimizer, **kw: MixedPrecisionTrainer(model, optimizer, BF16Config(), **kw)  # noqa: E731


class AmpContext:
    """Per-operation precision policy (``crates/torsh-backend/src/cuda/mixed_precision.rs:13-494``: ``AmpContext``):
    contractions run in the low-precision dtype, reductions / normalisations / losses in fp32, everything else keeps its
    input dtype; ``cast`` applies the policy to an operation's inputs and ``saturate`` clamps to the target's finite range
    before a down-cast (fp16 overflows at 65504)."""

    LOW = {"matmul", "linear", "conv2d", "conv1d", "bmm", "attention", "embedding"}
    FP32 = {"softmax", "log_softmax", "layer_norm", "rms_norm", "batch_norm", "cross_entropy", "mse_loss", "sum", "mean",
            "exp", "log", "pow", "norm"}

    def __init__(self, config: MixedPrecisionConfig | None = None, overrides: dict | None = None):
        self.cfg = config or MixedPrecisionConfig()
        self.overrides = dict(overrides or {})
        self.stats = {"casts": 0, "saturated": 0}

    def dtype_for(self, op: str, input_dtype: torch.dtype = torch.float32) -> torch.dtype:
        if op in self.overrides:
            return self.overrides[op]
        if not self.cfg.enabled or not input_dtype.is_floating_point:
            return input_dtype
        if op in self.LOW:
            return self.cfg.dtype
        if op in self.FP32:
            return torch.float32
        return input_dtype

    def saturate(self, t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        if not dtype.is_floating_point or torch.finfo(dtype).max >= torch.finfo(t.dtype).max:
            return t
        lim = torch.finfo(dtype).max
        over = t.abs() > lim
        if bool(over.any()):
            self.stats["saturated"] += int(over.sum())
            t = t.clamp(-lim, lim)
        return t

    def cast(self, op: str, *tensors):
        out = []
        for t in tensors:
            if isinstance(t, torch.Tensor) and t.is_floating_point():
                dt = self.dtype_for(op, t.dtype)
                if dt != t.dtype:
                    self.stats["casts"] += 1
                    t = self.saturate(t, dt).to(dt)
            out.append(t)
        return out[0] if len(out) == 1 else tuple(out)


GradientScaler = GradScaler
