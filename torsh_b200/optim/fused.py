"""AdamW / Adam / SGD / LAMB with the reference's exact arithmetic.

CUDA parameters are updated by one multi-tensor kernel launch per step
(``csrc/kernels/optim.cu``); CPU parameters run the same formulas in PyTorch, which doubles as the
numerical oracle. bf16 parameters automatically get fp32 master weights (the kernel writes both the
fp32 master and the bf16 copy), as in the reference's ``MixedPrecisionOptimizer``
(``crates/torsh-optim/src/mixed_precision.rs:18-419``).

Arithmetic (do not "fix" these, they are the reference's):
* AdamW (``crates/torsh-optim/src/adam.rs:809-950``): ``p -= lr·wd·p``; moments; ``m̂ = m/(1-β1ᵗ)``,
  ``v̂ = v/(1-β2ᵗ)``; ``p -= lr·m̂/(√v̂ + eps)``. Defaults lr 1e-3, betas (0.9, 0.999), eps 1e-8, wd 0.01.
* Adam (``adam.rs:292-673``): same with ``g += wd·p`` instead of the decoupled decay (wd default 0).
* SGD (``crates/torsh-optim/src/sgd.rs:443-610``): ``d = g + wd·p``; ``buf = μ·buf + (1-damp)·d`` with the
  buffer starting at zero; nesterov ``d += μ·buf`` else ``d = buf``; ``p -= lr·d``.
* LAMB (``crates/torsh-optim/src/lamb.rs:24-140``): ``g' = g + wd·p`` before the moments;
  ``u = m̂/(√v̂ + eps)``; trust ``= ‖p‖/‖u‖`` if both > eps else 1, clamped to ``≤ trust_ratio_threshold``
  (default 1.0); one global step count; eps 1e-6, wd 0.01.
"""
from __future__ import annotations

import torch

from ..ops import multi_tensor as mt


class _Base(torch.optim.Optimizer):
    """Adds the ToRSh ``Optimizer`` trait surface (``crates/torsh-optim/src/lib.rs:194-236``) to
    ``torch.optim.Optimizer``: ``get_lr``, ``set_lr``, ``add_param_group``, ``torsh_state_dict``."""

    def get_lr(self) -> list[float]:
        return [g["lr"] for g in self.param_groups]

    def set_lr(self, lr: float) -> None:
        for g in self.param_groups:
            g["lr"] = lr

    def torsh_state_dict(self) -> dict:
        """``OptimizerState`` schema (``crates/torsh-optim/src/lib.rs:242-262``)."""
        groups, state, pid = [], {}, 0
        for g in self.param_groups:
            opts = {k: v for k, v in g.items() if k not in ("params", "lr") and isinstance(v, (int, float, bool))}
            groups.append({"lr": g["lr"], "options": opts, "param_count": len(g["params"])})
            for p in g["params"]:
                st = self.state.get(p, {})
                state[f"param_{pid}"] = {k: v.detach().clone() for k, v in st.items() if isinstance(v, torch.Tensor)}
                pid += 1
        return {"optimizer_type": type(self).__name__, "version": "0.1.0", "param_groups": groups, "state": state,
                "global_state": {"step_count": float(getattr(self, "_step_count_torsh", 0))}}

    # ---- shared helpers ---------------------------------------------------
    def _cuda_groups(self, group, slots_fn):
        """Split params with grads into (cuda list, cpu list)."""
        cuda, cpu = [], []
        for p in group["params"]:
            if p.grad is None:
                continue
            (cuda if p.is_cuda else cpu).append(p)
        return cuda, cpu

    def _master(self, p, st):
        """fp32 master copy for low-precision CUDA params."""
        if p.dtype == torch.float32:
            return p.data, None
        if "master" not in st:
            st["master"] = p.data.float()
        return st["master"], p.data


class AdamW(_Base):
    decoupled = True

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 amsgrad: bool = False, found_inf: torch.Tensor | None = None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad))
        self._tables: dict = {}
        self.found_inf = found_inf

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for gi, g in enumerate(self.param_groups):
            b1, b2 = g["betas"]
            cuda, cpu = self._cuda_groups(g, None)
            for p in cuda + cpu:
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                    if g["amsgrad"]:
                        st["max_exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
            # ---- CUDA: one launch per (group, grad dtype)
            by_dtype: dict = {}
            for p in cuda:
                by_dtype.setdefault(p.grad.dtype, []).append(p)
            for gdt, ps in by_dtype.items():
                rows = []
                for p in ps:
                    st = self.state[p]
                    master, lowp = self._master(p, st)
                    grad = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                    rows.append((lowp, master, grad, st["exp_avg"], st["exp_avg_sq"], st.get("max_exp_avg_sq")))
                tt = mt.TensorTable.cached(self._tables, (gi, gdt), rows, ps[0].device)
                mt.adam_step(tt, lr=g["lr"], beta1=b1, beta2=b2, eps=g["eps"], weight_decay=g["weight_decay"],
                             step=self.state[ps[0]]["step"], decoupled=self.decoupled, amsgrad=g["amsgrad"],
                             grad_dtype=gdt, found_inf=self.found_inf)
            # ---- CPU: identical arithmetic
            for p in cpu:
                st = self.state[p]
                t = st["step"]
                grad = p.grad.float()
                w = p.data.float()
                if self.decoupled:
                    w = w - g["lr"] * g["weight_decay"] * w
                else:
                    grad = grad + g["weight_decay"] * w
                st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                m_hat = st["exp_avg"] / (1 - b1 ** t)
                v_hat = st["exp_avg_sq"] / (1 - b2 ** t)
                if g["amsgrad"]:
                    torch.maximum(st["max_exp_avg_sq"], v_hat, out=st["max_exp_avg_sq"])
                    v_hat = st["max_exp_avg_sq"]
                w = w - g["lr"] * m_hat / (v_hat.sqrt() + g["eps"])
                p.data.copy_(w)
        self._step_count_torsh = getattr(self, "_step_count_torsh", 0) + 1
        return loss


class Adam(AdamW):
    decoupled = False

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 amsgrad: bool = False, found_inf=None):
        super().__init__(params, lr, betas, eps, weight_decay, amsgrad, found_inf)


class SGD(_Base):
    def __init__(self, params, lr: float = 0.01, momentum: float = 0.0, dampening: float = 0.0,
                 weight_decay: float = 0.0, nesterov: bool = False, found_inf=None, zero_grad_in_step: bool = False):
        # zero_grad_in_step: the update kernel clears each gradient in the pass that reads it, so the gradients keep
        # their addresses from step to step (what a captured CUDA graph needs) and no separate zeroing pass runs
        self.zero_grad_in_step = zero_grad_in_step
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov))
        self._tables: dict = {}
        self.found_inf = found_inf

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for gi, g in enumerate(self.param_groups):
            mu = g["momentum"]
            cuda, cpu = self._cuda_groups(g, None)
            for p in cuda + cpu:
                st = self.state[p]
                if mu != 0 and "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
            by_dtype: dict = {}
            for p in cuda:
                by_dtype.setdefault(p.grad.dtype, []).append(p)
            for gdt, ps in by_dtype.items():
                rows = []
                for p in ps:
                    st = self.state[p]
                    master, lowp = self._master(p, st)
                    grad = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                    rows.append((lowp, master, grad, st.get("momentum_buffer")))
                tt = mt.TensorTable.cached(self._tables, (gi, gdt), rows, ps[0].device)
                mt.sgd_step(tt, lr=g["lr"], momentum=mu, dampening=g["dampening"], weight_decay=g["weight_decay"],
                            nesterov=g["nesterov"], grad_dtype=gdt, found_inf=self.found_inf,
                            zero_grad=self.zero_grad_in_step)
            for p in cpu:
                st = self.state[p]
                w = p.data.float()
                d = p.grad.float() + g["weight_decay"] * w
                if mu != 0:
                    buf = st["momentum_buffer"]
                    buf.mul_(mu).add_(d, alpha=1 - g["dampening"])
                    d = d + mu * buf if g["nesterov"] else buf
                p.data.copy_(w - g["lr"] * d)
        return loss


class LAMB(_Base):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-6, weight_decay: float = 0.01,
                 bias_correction: bool = True, trust_ratio_threshold: float = 1.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      bias_correction=bias_correction, trust_ratio_threshold=trust_ratio_threshold))
        self._tables: dict = {}
        self.step_count = 0

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self.step_count += 1
        t = self.step_count
        for gi, g in enumerate(self.param_groups):
            b1, b2 = g["betas"]
            cuda, cpu = self._cuda_groups(g, None)
            for p in cuda + cpu:
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            by_dtype: dict = {}
            for p in cuda:
                by_dtype.setdefault(p.grad.dtype, []).append(p)
            for gdt, ps in by_dtype.items():
                rows = []
                for p in ps:
                    st = self.state[p]
                    master, lowp = self._master(p, st)
                    if "update" not in st:
                        st["update"] = torch.empty_like(master)
                    grad = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                    rows.append((lowp, master, grad, st["exp_avg"], st["exp_avg_sq"], st["update"]))
                tt = mt.TensorTable.cached(self._tables, (gi, gdt), rows, ps[0].device)
                norms = self._tables.setdefault(("norms", gi, gdt), torch.zeros(2 * len(ps), device=ps[0].device))
                if norms.numel() != 2 * len(ps):
                    norms = self._tables[("norms", gi, gdt)] = torch.zeros(2 * len(ps), device=ps[0].device)
                mt.lamb_step(tt, norms, lr=g["lr"], beta1=b1, beta2=b2, eps=g["eps"], weight_decay=g["weight_decay"],
                             step=t, bias_correction=g["bias_correction"], trust_clip=g["trust_ratio_threshold"],
                             grad_dtype=gdt)
            for p in cpu:
                st = self.state[p]
                w = p.data.float()
                grad = p.grad.float() + g["weight_decay"] * w
                st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                bc1 = 1 - b1 ** t if g["bias_correction"] else 1.0
                bc2 = 1 - b2 ** t if g["bias_correction"] else 1.0
                u = (st["exp_avg"] / bc1) / ((st["exp_avg_sq"] / bc2).sqrt() + g["eps"])
                pn, un = w.norm().item(), u.norm().item()
                trust = pn / un if pn > g["eps"] and un > g["eps"] else 1.0
                trust = min(trust, g["trust_ratio_threshold"])
                p.data.copy_(w - g["lr"] * trust * u)
        return loss
