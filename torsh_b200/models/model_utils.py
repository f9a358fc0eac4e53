"""Model-level utilities: weight merging (average, weighted, EMA, task arithmetic, SLERP, max-magnitude, consensus, TIES,
model soups), sharding plans over devices, surgery (replace / graft / insert layers), knowledge distillation losses,
pruning with masks and schedules, and ensembling.

Reference: ``crates/torsh-models/src/{model_merging.rs:19-640, model_sharding.rs:18-450, surgery.rs:19-620,
distillation.rs:16-580, pruning.rs:17-610, ensembling.rs}``.
"""
from __future__ import annotations

import json
import math
import re
from dataclasses import dataclass, field
from enum import Enum

import torch


# ------------------------------------------------------------------------------------------------- merging
class MergeStrategy(Enum):
    AVERAGE = "average"
    WEIGHTED_AVERAGE = "weighted_average"
    EMA = "ema"
    TASK_ARITHMETIC = "task_arithmetic"
    SLERP = "slerp"
    MAX_MAGNITUDE = "max_magnitude"
    CONSENSUS = "consensus"
    TIES = "ties"


def _states(models) -> list[dict]:
    return [m if isinstance(m, dict) else {k: v.detach() for k, v in m.state_dict().items()} for m in models]


def slerp(a: torch.Tensor, b: torch.Tensor, t: float, eps: float = 1e-7) -> torch.Tensor:
    """Spherical interpolation of two tensors seen as vectors; falls back to linear when they are nearly parallel."""
    af, bf = a.float().reshape(-1), b.float().reshape(-1)
    cos = (af @ bf) / (af.norm() * bf.norm()).clamp(min=eps)
    cos = cos.clamp(-1, 1)
    omega = torch.acos(cos)
    if omega.abs() < 1e-4:
        return ((1 - t) * af + t * bf).view_as(a).to(a.dtype)
    so = torch.sin(omega)
    return ((torch.sin((1 - t) * omega) / so) * af + (torch.sin(t * omega) / so) * bf).view_as(a).to(a.dtype)


class ModelMerger:
    def __init__(self, strategy: MergeStrategy = MergeStrategy.AVERAGE, weights: list[float] | None = None, alpha: float = 0.5,
                 t: float = 0.5, threshold: float = 0.1, base=None, scaling: float = 1.0, density: float = 0.2):
        if weights is not None and abs(sum(weights) - 1.0) > 1e-4:
            raise ValueError("merge weights must sum to 1")
        self.strategy, self.weights, self.alpha, self.t, self.threshold = strategy, weights, alpha, t, threshold
        self.base = _states([base])[0] if base is not None else None
        self.scaling, self.density = scaling, density

    def merge_models(self, models) -> dict:
        sds = _states(models)
        if not sds:
            raise ValueError("nothing to merge")
        keys = list(sds[0])
        for sd in sds[1:]:
            if list(sd) != keys or any(sd[k].shape != sds[0][k].shape for k in keys):
                raise ValueError("models to merge must have identical parameter names and shapes")
        out = {}
        for k in keys:
            ts = [sd[k] for sd in sds]
            if not ts[0].is_floating_point():
                out[k] = ts[0].clone()
                continue
            fs = [t.float() for t in ts]
            s = self.strategy
            if s is MergeStrategy.AVERAGE:
                r = sum(fs) / len(fs)
            elif s is MergeStrategy.WEIGHTED_AVERAGE:
                w = self.weights or [1 / len(fs)] * len(fs)
                r = sum(wi * f for wi, f in zip(w, fs))
            elif s is MergeStrategy.EMA:
                r = fs[0]
                for f in fs[1:]:
                    r = self.alpha * f + (1 - self.alpha) * r
            elif s is MergeStrategy.SLERP:
                if len(fs) != 2:
                    raise ValueError("SLERP merges exactly two models")
                r = slerp(fs[0], fs[1], self.t)
            elif s is MergeStrategy.MAX_MAGNITUDE:
                st = torch.stack(fs)
                r = st.gather(0, st.abs().argmax(0, keepdim=True))[0]
            elif s is MergeStrategy.CONSENSUS:
                st = torch.stack(fs)
                mean = st.mean(0)
                agree = (st - mean).abs().amax(0) <= self.threshold * mean.abs().clamp(min=1e-8)
                r = torch.where(agree, mean, fs[0])
            elif s in (MergeStrategy.TASK_ARITHMETIC, MergeStrategy.TIES):
                if self.base is None:
                    raise ValueError("task arithmetic / TIES need the base model")
                b = self.base[k].float()
                taus = [f - b for f in fs]
                if s is MergeStrategy.TIES:
                    trimmed = []
                    for tau in taus:                      # keep the top `density` fraction by magnitude
                        kk = max(1, int(self.density * tau.numel()))
                        thr = tau.abs().reshape(-1).kthvalue(tau.numel() - kk + 1).values
                        trimmed.append(torch.where(tau.abs() >= thr, tau, torch.zeros_like(tau)))
                    st = torch.stack(trimmed)
                    sign = torch.sign(st.sum(0))          # elected sign per element
                    agree = (torch.sign(st) == sign) & (st != 0)
                    r = b + self.scaling * (st * agree).sum(0) / agree.sum(0).clamp(min=1)
                else:
                    r = b + self.scaling * sum(taus)
            else:
                raise ValueError(s)
            out[k] = r.to(ts[0].dtype)
        return out


class ModelSoup:
    """Uniform soup = plain average; greedy soup adds models (best first) only while the validation metric does not drop."""

    def __init__(self, greedy_threshold: float = 0.0):
        self.models: list = []
        self.greedy_threshold = greedy_threshold

    def add_model(self, m):
        self.models.append(m)

    def uniform_soup(self) -> dict:
        return ModelMerger(MergeStrategy.AVERAGE).merge_models(self.models)

    def greedy_soup(self, validate_fn) -> dict:
        sds = _states(self.models)
        order = sorted(range(len(sds)), key=lambda i: -validate_fn(sds[i]))
        soup, best = [sds[order[0]]], validate_fn(sds[order[0]])
        for i in order[1:]:
            cand = ModelMerger(MergeStrategy.AVERAGE).merge_models(soup + [sds[i]])
            score = validate_fn(cand)
            if score >= best - self.greedy_threshold:
                soup.append(sds[i]); best = max(best, score)
        return ModelMerger(MergeStrategy.AVERAGE).merge_models(soup)


# ------------------------------------------------------------------------------------------------- sharding plans
class ShardingStrategy(Enum):
    NONE = "none"
    PIPELINE = "pipeline"
    TENSOR_PARALLEL = "tensor_parallel"
    EXPERT_PARALLEL = "expert_parallel"
    ZERO_STAGE1 = "zero1"
    ZERO_STAGE2 = "zero2"
    ZERO_STAGE3 = "zero3"


@dataclass
class ShardingStats:
    params_per_device: list
    bytes_per_device: list

    def max_params_per_device(self): return max(self.params_per_device)
    def min_params_per_device(self): return min(self.params_per_device)
    def balance_ratio(self): return self.min_params_per_device() / max(self.max_params_per_device(), 1)
    def max_memory_mb(self): return max(self.bytes_per_device) / 2 ** 20


class ModelSharder:
    """Splits a model's ``state_dict`` into per-device dictionaries: whole layers by balanced parameter count (pipeline),
    matrices along their larger dimension (tensor parallel), experts round-robin, or flat 1 / N slices (ZeRO-3)."""

    def __init__(self, strategy: ShardingStrategy, num_devices: int):
        self.strategy, self.num_devices = strategy, num_devices

    def shard_model(self, model) -> list[dict]:
        sd = _states([model])[0]
        N, s = self.num_devices, self.strategy
        if s in (ShardingStrategy.NONE, ShardingStrategy.ZERO_STAGE1, ShardingStrategy.ZERO_STAGE2):
            return [dict(sd) for _ in range(N)]           # parameters replicated (only optimizer state / gradients shard)
        out = [dict() for _ in range(N)]
        if s is ShardingStrategy.PIPELINE:
            groups: dict = {}
            for k in sd:
                m = re.search(r"(.*?\.\d+)\.", k)
                groups.setdefault(m.group(1) if m else k.split(".")[0], []).append(k)
            sizes = [sum(sd[k].numel() for k in ks) for ks in groups.values()]
            target, dev, acc = sum(sizes) / N, 0, 0
            for (g, ks), sz in zip(groups.items(), sizes):
                if acc >= target * (dev + 1) - sz / 2 and dev < N - 1:
                    dev += 1
                acc += sz
                for k in ks:
                    out[dev][k] = sd[k]
        elif s is ShardingStrategy.TENSOR_PARALLEL:
            for k, v in sd.items():
                if v.dim() >= 2 and max(v.shape[:2]) % N == 0:
                    dim = 0 if v.shape[0] >= v.shape[1] and v.shape[0] % N == 0 else 1
                    if v.shape[dim] % N:
                        dim = 1 - dim
                    for d, part in enumerate(v.chunk(N, dim)):
                        out[d][k] = part
                else:
                    for d in range(N):
                        out[d][k] = v
        elif s is ShardingStrategy.EXPERT_PARALLEL:
            for k, v in sd.items():
                m = re.search(r"experts?\.(\d+)\.", k)
                if m:
                    out[int(m.group(1)) % N][k] = v
                else:
                    for d in range(N):
                        out[d][k] = v
        elif s is ShardingStrategy.ZERO_STAGE3:
            for k, v in sd.items():
                flat = v.reshape(-1)
                per = -(-flat.numel() // N)
                for d in range(N):
                    out[d][k] = flat[d * per:(d + 1) * per]
        return out

    def get_stats(self, shards: list[dict]) -> ShardingStats:
        return ShardingStats([sum(v.numel() for v in s.values()) for s in shards],
                             [sum(v.numel() * v.element_size() for v in s.values()) for s in shards])


# ------------------------------------------------------------------------------------------------- surgery
class ModelSurgeon:
    """Replace, insert, remove or graft sub-modules by dotted name and keep a log of the parameter-count changes."""

    def __init__(self, model: torch.nn.Module):
        self.model, self.log = model, []

    def _parent(self, name: str):
        parts = name.split(".")
        m = self.model
        for p in parts[:-1]:
            m = getattr(m, p) if not p.isdigit() else m[int(p)]
        return m, parts[-1]

    def _get(self, parent, leaf):
        return parent[int(leaf)] if leaf.isdigit() else getattr(parent, leaf)

    def _set(self, parent, leaf, value):
        if leaf.isdigit():
            parent[int(leaf)] = value
        else:
            setattr(parent, leaf, value)

    def replace_layer(self, name: str, new: torch.nn.Module, copy_weights: bool = False):
        parent, leaf = self._parent(name)
        old = self._get(parent, leaf)
        if copy_weights:
            with torch.no_grad():
                for (n, p), (_, q) in zip(new.named_parameters(), old.named_parameters()):
                    sl = tuple(slice(0, min(a, b)) for a, b in zip(p.shape, q.shape))
                    p[sl].copy_(q[sl])
        self._set(parent, leaf, new)
        self.log.append({"op": "replace", "layer": name, "params_before": sum(p.numel() for p in old.parameters()),
                         "params_after": sum(p.numel() for p in new.parameters())})
        return old

    def insert_after(self, name: str, extra: torch.nn.Module):
        parent, leaf = self._parent(name)
        self._set(parent, leaf, torch.nn.Sequential(self._get(parent, leaf), extra))
        self.log.append({"op": "insert_after", "layer": name, "params_added": sum(p.numel() for p in extra.parameters())})

    def remove_layer(self, name: str):
        return self.replace_layer(name, torch.nn.Identity())

    def graft(self, name: str, donor: torch.nn.Module, donor_name: str):
        """Take sub-module ``donor_name`` of ``donor`` (weights included) and put it at ``name`` of this model."""
        d = donor
        for p in donor_name.split("."):
            d = d[int(p)] if p.isdigit() else getattr(d, p)
        return self.replace_layer(name, d)

    def stats(self) -> dict:
        return {"operations": len(self.log), "log": self.log, "parameters_now": sum(p.numel() for p in self.model.parameters())}

    def save_plan(self, path):
        open(path, "w").write(json.dumps(self.log, indent=2))


# ------------------------------------------------------------------------------------------------- distillation
class DistillationStrategy(Enum):
    RESPONSE = "response"
    FEATURE = "feature"
    ATTENTION = "attention"
    RELATION = "relation"
    MULTI_LEVEL = "multi_level"


@dataclass
class DistillationConfig:
    strategy: DistillationStrategy = DistillationStrategy.RESPONSE
    temperature: float = 4.0
    alpha: float = 0.7            # weight of the distillation term; 1 - alpha on the hard-label loss
    feature_weight: float = 1.0
    attention_weight: float = 1.0


class DistillationTrainer:
    def __init__(self, config: DistillationConfig | None = None):
        self.cfg = config or DistillationConfig()
        self.adapters: dict[str, torch.nn.Module] = {}

    def add_adaptation_layer(self, name: str, layer: torch.nn.Module):
        self.adapters[name] = layer

    def response_loss(self, student_logits, teacher_logits) -> torch.Tensor:
        T = self.cfg.temperature
        return torch.nn.functional.kl_div(torch.log_softmax(student_logits.float() / T, -1), torch.softmax(teacher_logits.float() / T, -1),
                                          reduction="batchmean") * T * T

    def feature_loss(self, student_feats: dict, teacher_feats: dict) -> torch.Tensor:
        loss = 0.0
        for k, s in student_feats.items():
            t = teacher_feats[k]
            if k in self.adapters:
                s = self.adapters[k](s)
            loss = loss + torch.nn.functional.mse_loss(s.float(), t.float())
        return loss

    def attention_loss(self, student_maps: list, teacher_maps: list) -> torch.Tensor:
        norm = lambda a: torch.nn.functional.normalize(a.float().pow(2).mean(1).flatten(1), dim=-1)
        return sum((norm(s) - norm(t)).pow(2).sum(-1).mean() for s, t in zip(student_maps, teacher_maps))

    def relation_loss(self, student_emb, teacher_emb) -> torch.Tensor:
        def dist(e):
            d = torch.cdist(e.float(), e.float())
            return d / d[d > 0].mean().clamp(min=1e-8)
        return torch.nn.functional.smooth_l1_loss(dist(student_emb), dist(teacher_emb))

    def compute_distillation_loss(self, student_logits, teacher_logits, labels=None, student_feats=None, teacher_feats=None,
                                  student_attn=None, teacher_attn=None) -> dict:
        c = self.cfg
        out = {"distillation": self.response_loss(student_logits, teacher_logits)}
        total = c.alpha * out["distillation"]
        if labels is not None:
            out["hard"] = torch.nn.functional.cross_entropy(student_logits.float(), labels)
            total = total + (1 - c.alpha) * out["hard"]
        if student_feats is not None and c.strategy in (DistillationStrategy.FEATURE, DistillationStrategy.MULTI_LEVEL):
            out["feature"] = self.feature_loss(student_feats, teacher_feats)
            total = total + c.feature_weight * out["feature"]
        if student_attn is not None and c.strategy in (DistillationStrategy.ATTENTION, DistillationStrategy.MULTI_LEVEL):
            out["attention"] = self.attention_loss(student_attn, teacher_attn)
            total = total + c.attention_weight * out["attention"]
        out["total"] = total
        return out


def compression_ratio(teacher_params: int, student_params: int) -> float:
    return teacher_params / max(student_params, 1)


# ------------------------------------------------------------------------------------------------- pruning
class PruningMethod(Enum):
    MAGNITUDE = "magnitude"
    RANDOM = "random"
    SNIP = "snip"          # |g * w|
    FISHER = "fisher"      # g^2 * w^2
    LAMP = "lamp"          # layer-adaptive magnitude: w^2 / sum of larger-or-equal w^2


@dataclass
class PruningConfig:
    sparsity: float = 0.5
    method: PruningMethod = PruningMethod.MAGNITUDE
    structured: bool = False            # prune whole output rows by their L2 norm
    include: str = r"weight$"
    exclude: str = r"(norm|ln|bias|embed)"
    schedule: str = "one_shot"          # or "polynomial"
    initial_sparsity: float = 0.0
    steps: int = 1
    power: float = 3.0


class ModelPruner:
    def __init__(self, config: PruningConfig | None = None):
        self.cfg = config or PruningConfig()
        self.masks: dict[str, torch.Tensor] = {}
        self.step_count = 0

    def current_sparsity(self) -> float:
        c = self.cfg
        if c.schedule == "one_shot" or c.steps <= 1:
            return c.sparsity
        t = min(self.step_count, c.steps) / c.steps
        return c.sparsity + (c.initial_sparsity - c.sparsity) * (1 - t) ** c.power

    def _scores(self, p: torch.Tensor) -> torch.Tensor:
        m, w = self.cfg.method, p.detach().float()
        if m is PruningMethod.RANDOM:
            return torch.rand_like(w)
        if m is PruningMethod.SNIP and p.grad is not None:
            return (p.grad.float() * w).abs()
        if m is PruningMethod.FISHER and p.grad is not None:
            return p.grad.float().pow(2) * w.pow(2)
        if m is PruningMethod.LAMP:
            flat = w.pow(2).reshape(-1)
            srt, idx = flat.sort()
            denom = srt.flip(0).cumsum(0).flip(0)              # sum of all entries >= this one
            out = torch.empty_like(flat)
            out[idx] = srt / denom.clamp(min=1e-30)
            return out.view_as(w)
        return w.abs()

    @torch.no_grad()
    def prune_model(self, model: torch.nn.Module) -> dict:
        inc, exc = re.compile(self.cfg.include), re.compile(self.cfg.exclude)
        sp = self.current_sparsity()
        stats = {}
        for n, p in model.named_parameters():
            if not inc.search(n) or exc.search(n) or p.dim() < 2:
                continue
            sc = self._scores(p)
            if self.cfg.structured:
                rows = sc.flatten(1).norm(dim=1)
                k = int(sp * rows.numel())
                mask = torch.ones_like(rows, dtype=torch.bool)
                if k > 0:
                    mask[rows.topk(k, largest=False).indices] = False
                mask = mask.view(-1, *([1] * (p.dim() - 1))).expand_as(p)
            else:
                k = int(sp * sc.numel())
                mask = torch.ones(sc.numel(), dtype=torch.bool, device=p.device)
                if k > 0:
                    mask[sc.reshape(-1).topk(k, largest=False).indices] = False
                mask = mask.view_as(p)
            self.masks[n] = mask
            p.mul_(mask.to(p.dtype))
            stats[n] = 1.0 - mask.float().mean().item()
        self.step_count += 1
        total = sum(m.numel() for m in self.masks.values())
        return {"layers": stats, "overall_sparsity": 1.0 - sum(m.sum().item() for m in self.masks.values()) / max(total, 1)}

    @torch.no_grad()
    def apply_masks(self, model: torch.nn.Module):
        """Re-apply the stored masks (after an optimizer step, so pruned weights stay zero)."""
        for n, p in model.named_parameters():
            if n in self.masks:
                p.mul_(self.masks[n].to(p.dtype))

    def save_masks(self, path):
        torch.save({k: v.cpu() for k, v in self.masks.items()}, path)

    def load_masks(self, path):
        self.masks = torch.load(path, weights_only=True)


def calculate_sparsity(t: torch.Tensor) -> float:
    return 1.0 - (t != 0).float().mean().item()


# ------------------------------------------------------------------------------------------------- ensembling
class Ensemble(torch.nn.Module):
    """Average (or weighted / majority-vote) combination of several models' outputs."""

    def __init__(self, models, weights: list[float] | None = None, mode: str = "mean"):
        super().__init__()
        self.models = torch.nn.ModuleList(models)
        self.weights, self.mode = weights, mode

    def forward(self, *a, **k):
        outs = [m(*a, **k) for m in self.models]
        if self.mode == "vote":
            votes = torch.stack([o.argmax(-1) for o in outs])
            return torch.mode(votes, 0).values
        probs = torch.stack([torch.softmax(o.float(), -1) if self.mode == "prob" else o.float() for o in outs])
        w = torch.tensor(self.weights or [1 / len(outs)] * len(outs), device=probs.device).view(-1, *([1] * (probs.dim() - 1)))
        return (probs * w).sum(0)
