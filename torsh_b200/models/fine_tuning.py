"""Parameter-efficient fine-tuning: LoRA / AdaLoRA-style low-rank updates, bottleneck adapters, prefix tuning, layer
freezing with progressive unfreezing, layer-wise learning-rate decay and an EWC penalty.

Reference: ``crates/torsh-models/src/fine_tuning.rs`` (``AdapterType {Standard, LoRA, AdaLoRA, PrefixTuning, PtuningV2,
Compacter}`` ``:94-132``, ``FreezingStrategy`` ``:53-68``, ``LayerLearningRateSchedule`` ``:35-51``, progressive
unfreezing ``:179-215``, ``EWCConfig`` ``:294-303``, ``FineTuningEngine`` ``:391-470``) and the LoRA merge / extract
helpers of ``model_merging.rs:403-555``.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field

import torch

from .. import nn


# ------------------------------------------------------------------------------------------------- LoRA
class LoRALinear(nn.Module):
    """``y = base(x) + (alpha / r) * dropout(x) A^T B^T`` with the base layer frozen. ``B`` starts at zero, so the wrapped
    layer initially computes exactly what the base computes."""

    def __init__(self, base: torch.nn.Linear, rank: int = 8, alpha: float = 16.0, dropout: float = 0.0):
        super().__init__()
        self.base, self.rank, self.alpha = base, rank, alpha
        for p in base.parameters():
            p.requires_grad_(False)
        dev, dt = base.weight.device, base.weight.dtype
        self.lora_A = nn.Parameter(torch.empty(rank, base.in_features, device=dev, dtype=dt))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, rank, device=dev, dtype=dt))
        torch.nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        self.drop = nn.Dropout(dropout) if dropout > 0 else None
        self.merged = False

    @property
    def scaling(self) -> float:
        return self.alpha / self.rank

    def delta_weight(self) -> torch.Tensor:
        return (self.lora_B @ self.lora_A) * self.scaling

    def forward(self, x):
        y = self.base(x)
        if self.merged:
            return y
        h = self.drop(x) if self.drop is not None else x
        return y + torch.nn.functional.linear(torch.nn.functional.linear(h, self.lora_A), self.lora_B) * self.scaling

    @torch.no_grad()
    def merge(self):
        """Fold the update into the base weight (inference without the extra GEMMs)."""
        if not self.merged:
            self.base.weight.add_(self.delta_weight().to(self.base.weight.dtype))
            self.merged = True

    @torch.no_grad()
    def unmerge(self):
        if self.merged:
            self.base.weight.sub_(self.delta_weight().to(self.base.weight.dtype))
            self.merged = False


def _replace_modules(model: torch.nn.Module, pattern: str, make) -> list[str]:
    rx, done = re.compile(pattern), []
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if isinstance(child, torch.nn.Linear) and rx.search(full):
                setattr(module, child_name, make(child))
                done.append(full)
    return done


def apply_lora(model: torch.nn.Module, target: str = r"(q|k|v|out)_proj|attn|fc\d|dense", rank: int = 8, alpha: float = 16.0,
               dropout: float = 0.0, freeze_rest: bool = True) -> list[str]:
    """Wrap every ``nn.Linear`` whose dotted name matches ``target`` in :class:`LoRALinear`; with ``freeze_rest`` all
    other parameters stop training. Returns the wrapped layer names."""
    if freeze_rest:
        for p in model.parameters():
            p.requires_grad_(False)
    return _replace_modules(model, target, lambda lin: LoRALinear(lin, rank, alpha, dropout))


def merge_lora(model: torch.nn.Module) -> int:
    n = 0
    for m in model.modules():
        if isinstance(m, LoRALinear):
            m.merge(); n += 1
    return n


def lora_state_dict(model: torch.nn.Module) -> dict:
    return {k: v for k, v in model.state_dict().items() if "lora_A" in k or "lora_B" in k}


def extract_lora(base_weight: torch.Tensor, tuned_weight: torch.Tensor, rank: int, alpha: float | None = None):
    """Best rank-``rank`` factors of ``tuned - base`` (truncated SVD): returns ``(A [r, in], B [out, r])`` with
    ``(alpha / r) * B A ≈ tuned - base`` (``LoRAMerger::extract_lora``)."""
    alpha = float(rank) if alpha is None else alpha
    U, S, Vh = torch.linalg.svd((tuned_weight - base_weight).float(), full_matrices=False)
    s = S[:rank].sqrt()
    scale = math.sqrt(rank / alpha)
    return (s[:, None] * Vh[:rank]) * scale, (U[:, :rank] * s[None, :]) * scale


class AdaLoRALinear(LoRALinear):
    """LoRA in SVD form ``B diag(lambda) A`` whose singular values can be pruned by importance (AdaLoRA): ``prune_to(k)``
    keeps the ``k`` largest ``|lambda|`` and zeroes the rest."""

    def __init__(self, base, rank=8, alpha=16.0, dropout=0.0):
        super().__init__(base, rank, alpha, dropout)
        torch.nn.init.normal_(self.lora_B, std=0.02)
        self.lora_E = nn.Parameter(torch.zeros(rank, device=base.weight.device, dtype=base.weight.dtype))
        self.register_buffer("rank_mask", torch.ones(rank, device=base.weight.device, dtype=base.weight.dtype))

    def delta_weight(self):
        return (self.lora_B * (self.lora_E * self.rank_mask)) @ self.lora_A * self.scaling

    def forward(self, x):
        y = self.base(x)
        if self.merged:
            return y
        h = self.drop(x) if self.drop is not None else x
        z = torch.nn.functional.linear(h, self.lora_A) * (self.lora_E * self.rank_mask)
        return y + torch.nn.functional.linear(z, self.lora_B) * self.scaling

    @torch.no_grad()
    def prune_to(self, keep: int):
        idx = self.lora_E.abs().topk(min(keep, self.rank)).indices
        self.rank_mask.zero_()
        self.rank_mask[idx] = 1

    def orthogonality_penalty(self) -> torch.Tensor:
        eye = torch.eye(self.rank, device=self.lora_A.device, dtype=self.lora_A.dtype)
        return ((self.lora_A @ self.lora_A.t() - eye) ** 2).sum() + ((self.lora_B.t() @ self.lora_B - eye) ** 2).sum()


# ------------------------------------------------------------------------------------------------- adapters / prefixes
class BottleneckAdapter(nn.Module):
    """Houlsby-style adapter: ``x + up(act(down(x)))`` with ``hidden / reduction_factor`` bottleneck units; ``up`` starts at
    zero (identity at insertion)."""

    def __init__(self, hidden: int, reduction_factor: int = 16, activation: str = "relu"):
        super().__init__()
        r = max(1, hidden // reduction_factor)
        self.down, self.up = nn.Linear(hidden, r), nn.Linear(r, hidden)
        torch.nn.init.zeros_(self.up.weight); torch.nn.init.zeros_(self.up.bias)
        self.act = {"relu": torch.relu, "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu, "tanh": torch.tanh}[activation]

    def forward(self, x):
        return x + self.up(self.act(self.down(x)))


class _WithAdapter(nn.Module):
    def __init__(self, inner, adapter):
        super().__init__()
        self.inner, self.adapter = inner, adapter

    def forward(self, *a, **k):
        out = self.inner(*a, **k)
        if isinstance(out, tuple):
            return (self.adapter(out[0]),) + out[1:]
        return self.adapter(out)


def insert_adapters(model: torch.nn.Module, target: str, hidden: int, reduction_factor: int = 16, activation: str = "relu",
                    freeze_rest: bool = True) -> list[str]:
    """Append a :class:`BottleneckAdapter` after every sub-module whose dotted name matches ``target``."""
    if freeze_rest:
        for p in model.parameters():
            p.requires_grad_(False)
    rx, done = re.compile(target), []
    for name, module in list(model.named_modules()):
        for child_name, child in list(module.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if rx.fullmatch(full) and not isinstance(child, _WithAdapter):
                setattr(module, child_name, _WithAdapter(child, BottleneckAdapter(hidden, reduction_factor, activation)))
                done.append(full)
    return done


class PrefixEncoder(nn.Module):
    """Prefix tuning / P-tuning v2: ``prefix_length`` trainable virtual tokens per layer, produced through a small MLP
    re-parametrisation during training. ``forward()`` returns ``[num_layers, prefix_length, hidden]``; prepend slice ``l``
    to the keys and values (or to the input) of layer ``l``."""

    def __init__(self, num_layers: int, prefix_length: int, hidden: int, reparam_hidden: int | None = None):
        super().__init__()
        self.num_layers, self.prefix_length, self.hidden = num_layers, prefix_length, hidden
        self.embedding = nn.Parameter(torch.empty(prefix_length, hidden).normal_(0, 0.02))
        if reparam_hidden:
            self.mlp = nn.Sequential(nn.Linear(hidden, reparam_hidden), nn.Tanh(), nn.Linear(reparam_hidden, num_layers * hidden))
        else:
            self.mlp = None
            self.per_layer = nn.Parameter(torch.empty(num_layers, prefix_length, hidden).normal_(0, 0.02))

    def forward(self):
        if self.mlp is None:
            return self.per_layer
        return self.mlp(self.embedding).view(self.prefix_length, self.num_layers, self.hidden).transpose(0, 1)


# ------------------------------------------------------------------------------------------------- freezing / schedules
@dataclass
class FineTuningConfig:
    base_lr: float = 1e-4
    layer_lr_decay: float = 1.0          # < 1: deeper (earlier) layers train with smaller rates
    freeze_patterns: list = field(default_factory=list)       # regexes of parameter names to freeze
    unfreeze_patterns: list = field(default_factory=list)     # regexes that stay trainable even if a freeze pattern matches
    progressive_unfreeze_every: int = 0  # steps between unfreezing one more layer group (0 = off)
    ewc_lambda: float = 0.0


def freeze_parameters(model: torch.nn.Module, freeze: list[str], keep: list[str] | None = None) -> int:
    frx, krx = [re.compile(p) for p in freeze], [re.compile(p) for p in (keep or [])]
    n = 0
    for name, p in model.named_parameters():
        if any(r.search(name) for r in frx) and not any(r.search(name) for r in krx):
            p.requires_grad_(False); n += 1
    return n


def _layer_index(name: str) -> int | None:
    m = re.search(r"\.(\d+)\.", "." + name)
    return int(m.group(1)) if m else None


def layerwise_lr_groups(model: torch.nn.Module, base_lr: float, decay: float) -> list[dict]:
    """Optimizer parameter groups with ``lr = base_lr * decay ** (depth_from_top)``: the last numbered layer and everything
    after it get ``base_lr``, embeddings (no layer index before the first layer) the smallest rate."""
    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    idx = [i for i in (_layer_index(n) for n, _ in named) if i is not None]
    top = max(idx) if idx else 0
    groups: dict[float, list] = {}
    seen_layer = False
    for n, p in named:
        i = _layer_index(n)
        if i is not None:
            seen_layer = True
            depth = top - i
        else:
            depth = 0 if seen_layer else top + 1
        groups.setdefault(base_lr * decay ** depth, []).append(p)
    return [{"params": ps, "lr": lr} for lr, ps in sorted(groups.items())]


class ProgressiveUnfreezer:
    """Starts with only the head trainable and unfreezes one numbered layer (top first) every ``every`` steps."""

    def __init__(self, model: torch.nn.Module, every: int):
        self.model, self.every, self.step_count = model, every, 0
        self.layers = sorted({i for i in (_layer_index(n) for n, _ in model.named_parameters()) if i is not None}, reverse=True)
        self.unfrozen = 0
        for n, p in model.named_parameters():
            if _layer_index(n) is not None:
                p.requires_grad_(False)

    def step(self) -> int | None:
        self.step_count += 1
        if self.every and self.step_count % self.every == 0 and self.unfrozen < len(self.layers):
            layer = self.layers[self.unfrozen]
            for n, p in self.model.named_parameters():
                if _layer_index(n) == layer:
                    p.requires_grad_(True)
            self.unfrozen += 1
            return layer
        return None


class EWCPenalty:
    """Elastic weight consolidation: ``lambda / 2 * sum F_i (theta_i - theta*_i)^2`` with a diagonal Fisher estimate
    accumulated from squared gradients on the old task."""

    def __init__(self, model: torch.nn.Module, lam: float = 0.4):
        self.model, self.lam = model, lam
        self.anchor = {n: p.detach().clone() for n, p in model.named_parameters() if p.requires_grad}
        self.fisher = {n: torch.zeros_like(p) for n, p in self.anchor.items()}
        self.samples = 0

    def accumulate(self):
        """Call after ``backward()`` on an old-task batch."""
        for n, p in self.model.named_parameters():
            if n in self.fisher and p.grad is not None:
                self.fisher[n] += p.grad.detach() ** 2
        self.samples += 1

    def penalty(self) -> torch.Tensor:
        k = max(self.samples, 1)
        return 0.5 * self.lam * sum(((self.fisher[n] / k) * (p - self.anchor[n]) ** 2).sum()
                                    for n, p in self.model.named_parameters() if n in self.anchor)


def trainable_summary(model: torch.nn.Module) -> dict:
    tot = sum(p.numel() for p in model.parameters())
    tr = sum(p.numel() for p in model.parameters() if p.requires_grad)
    return {"total": tot, "trainable": tr, "fraction": tr / max(tot, 1)}
