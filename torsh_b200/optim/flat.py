"""Flat mixed-precision parameter storage and its fused optimizer.

All parameters of a model (or of one FSDP unit) live in three aligned flat buffers: a bf16 buffer the
forward/backward read, an fp32 master copy, and an fp32 gradient buffer into which the GEMM
epilogues, norm and embedding backward kernels accumulate directly (each parameter carries a
``main_grad`` view). One fused kernel launch then applies AdamW to the whole model, refreshes the
bf16 copy and clears the gradient in the same pass. This is the single-GPU form of the FSDP
unit layout; the sharded form slices the same buffers by rank.

Policy counterpart in the reference: ``MixedPrecisionOptimizer`` (fp32 master weights, copy
master→params: ``crates/torsh-optim/src/mixed_precision.rs:18-419``) and the CPU multi-tensor loops
``fused_adam_step`` (``crates/torsh-optim/src/fused_kernels.rs:32-389``).
"""
from __future__ import annotations

import torch

from ..ops import multi_tensor as mt

ALIGN = 128  # elements; keeps every parameter 256-byte aligned in the bf16 buffer


class FlatParameters:
    def __init__(self, params, lowp_dtype=torch.bfloat16, with_adam_state: bool = True):
        params = [p for p in params]
        seen, uniq = set(), []
        for p in params:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append(p)
        self.params = uniq
        self.device = uniq[0].device
        self.offsets, off = [], 0
        for p in uniq:
            self.offsets.append(off)
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.total = off
        self.lowp = torch.zeros(off, dtype=lowp_dtype, device=self.device)
        self.master = torch.zeros(off, dtype=torch.float32, device=self.device)
        self.grad = torch.zeros(off, dtype=torch.float32, device=self.device)
        with torch.no_grad():
            for p, o in zip(uniq, self.offsets):
                n = p.numel()
                self.master[o:o + n].copy_(p.detach().reshape(-1).float())
                self.lowp[o:o + n].copy_(self.master[o:o + n])
                p.data = self.lowp[o:o + n].view(p.shape)
                p.main_grad = self.grad[o:o + n].view(p.shape)
                p.grad = None
        if with_adam_state:
            self.exp_avg = torch.zeros(off, dtype=torch.float32, device=self.device)
            self.exp_avg_sq = torch.zeros(off, dtype=torch.float32, device=self.device)
        self._tables: dict = {}

    def zero_grad(self):
        self.grad.zero_()

    def numel(self) -> int:
        return sum(p.numel() for p in self.params)


class FlatAdamW:
    """AdamW over :class:`FlatParameters` (one kernel launch per step, gradient cleared in the same pass)."""

    def __init__(self, flat: FlatParameters, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01):
        self.flat, self.lr, self.betas, self.eps, self.weight_decay = flat, lr, betas, eps, weight_decay
        self.step_count = 0
        self.param_groups = [{"lr": lr, "params": flat.params}]
        self.dyn = torch.zeros(3, dtype=torch.float32, device=flat.device)
        self._dyn_host = torch.zeros(8, 3, dtype=torch.float32)
        if flat.device.type == "cuda":
            self._dyn_host = self._dyn_host.pin_memory()

    def get_lr(self):
        return [self.param_groups[0]["lr"]]

    def set_lr(self, lr):
        self.param_groups[0]["lr"] = lr

    def prepare_step(self):
        """Host part of a step: advance the step count and upload lr and the two bias corrections.
        Runs outside any CUDA graph; :meth:`launch` is the capturable device part."""
        self.step_count += 1
        # one pinned row per step in flight: the asynchronous upload of an earlier step may not have run yet
        row = self._dyn_host[self.step_count % self._dyn_host.shape[0]]
        row[0] = self.param_groups[0]["lr"]
        row[1] = 1.0 - self.betas[0] ** self.step_count
        row[2] = 1.0 - self.betas[1] ** self.step_count
        self.dyn.copy_(row, non_blocking=True)

    def step(self, grad_scale: float = 1.0, zero_grad: bool = True):
        self.prepare_step()
        self.launch(grad_scale, zero_grad)

    @torch.no_grad()
    def launch(self, grad_scale: float = 1.0, zero_grad: bool = True):
        f = self.flat
        lr = self.param_groups[0]["lr"]
        if f.device.type == "cuda":
            tt = mt.TensorTable.cached(f._tables, "adamw", [(f.lowp, f.master, f.grad, f.exp_avg, f.exp_avg_sq, None)], f.device)
            mt.adam_step(tt, lr=lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps,
                         weight_decay=self.weight_decay, step=max(self.step_count, 1), decoupled=True,
                         grad_dtype=torch.float32, grad_scale=grad_scale, zero_grad=zero_grad, dyn=self.dyn)
            return
        # without the kernels autograd leaves gradients in p.grad instead of accumulating them into main_grad
        for prm in f.params:
            if prm.grad is not None:
                prm.main_grad.add_(prm.grad.to(prm.main_grad.dtype))
                prm.grad = None
        b1, b2 = self.betas
        g = f.grad * grad_scale
        w = f.master
        w.sub_(lr * self.weight_decay * w)
        f.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        f.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        m_hat = f.exp_avg / (1 - b1 ** self.step_count)
        v_hat = f.exp_avg_sq / (1 - b2 ** self.step_count)
        w.sub_(lr * m_hat / (v_hat.sqrt() + self.eps))
        f.lowp.copy_(w)
        if zero_grad:
            f.grad.zero_()

    def zero_grad(self, set_to_none: bool = False):
        self.flat.zero_grad()

    def state_dict(self) -> dict:
        """fp32 master weights, both moments, the step count and the learning rate (flat tensors on the CPU)."""
        f = self.flat
        return {"step_count": self.step_count, "lr": self.param_groups[0]["lr"], "total": f.total,
                "master": f.master.detach().cpu().clone(), "exp_avg": f.exp_avg.detach().cpu().clone(),
                "exp_avg_sq": f.exp_avg_sq.detach().cpu().clone()}

    @torch.no_grad()
    def load_state_dict(self, sd: dict):
        """Restores the master weights FIRST and refreshes the bf16 parameters from them: a restore that wrote only the
        bf16 views would be undone by the next step, which rewrites them from the master copy."""
        f = self.flat
        if int(sd.get("total", f.total)) != f.total:
            raise ValueError(f"optimizer state has {sd.get('total')} elements, this model has {f.total}")
        f.master.copy_(sd["master"]); f.exp_avg.copy_(sd["exp_avg"]); f.exp_avg_sq.copy_(sd["exp_avg_sq"])
        f.lowp.copy_(f.master)
        self.step_count = int(sd["step_count"])
        self.param_groups[0]["lr"] = sd.get("lr", self.param_groups[0]["lr"])

    def grad_sq_norm(self) -> torch.Tensor:
        f = self.flat
        out = torch.zeros(1, dtype=torch.float32, device=f.device)
        if f.device.type == "cuda":
            tt = mt.TensorTable.cached(f._tables, "adamw", [(f.lowp, f.master, f.grad, f.exp_avg, f.exp_avg_sq, None)], f.device)
            mt.sq_norm(tt, 2, torch.float32, out)
        else:
            out[0] = f.grad.pow(2).sum()
        return out
