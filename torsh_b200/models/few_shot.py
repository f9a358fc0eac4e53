"""Few-shot learning: episodic N-way K-shot sampling, prototypical networks (Euclidean / cosine / Manhattan distances),
MAML (second- or first-order inner loop through ``torch.func.functional_call``) and Reptile, with an evaluator that reports
mean accuracy and a 95 % confidence interval over episodes. Reference: crates/torsh-models/src/few_shot.rs.
"""
from __future__ import annotations

import copy
import math
import random
from dataclasses import dataclass

import torch
from torch import nn


@dataclass
class FewShotConfig:
    n_way: int = 5
    k_shot: int = 1
    n_query: int = 5
    distance: str = "euclidean"        # "cosine", "manhattan"
    inner_lr: float = 0.1
    inner_steps: int = 1
    first_order: bool = False


@dataclass
class Episode:
    support_x: torch.Tensor
    support_y: torch.Tensor
    query_x: torch.Tensor
    query_y: torch.Tensor


class FewShotDataset:
    """Samples episodes from ``(x [M, ...], y [M])``: N classes, K support and Q query examples each, labels 0..N-1."""

    def __init__(self, x: torch.Tensor, y: torch.Tensor, cfg: FewShotConfig, seed: int = 0):
        self.x, self.cfg, self.rng = x, cfg, random.Random(seed)
        self.by_class = {int(c): (y == c).nonzero().flatten().tolist() for c in y.unique()}
        need = cfg.k_shot + cfg.n_query
        self.classes = [c for c, idx in self.by_class.items() if len(idx) >= need]
        if len(self.classes) < cfg.n_way:
            raise ValueError(f"need {cfg.n_way} classes with at least {need} examples, found {len(self.classes)}")

    def sample_episode(self) -> Episode:
        c = self.cfg
        sx, sy, qx, qy = [], [], [], []
        for label, cls in enumerate(self.rng.sample(self.classes, c.n_way)):
            idx = self.rng.sample(self.by_class[cls], c.k_shot + c.n_query)
            sx.append(self.x[idx[:c.k_shot]]); sy += [label] * c.k_shot
            qx.append(self.x[idx[c.k_shot:]]); qy += [label] * c.n_query
        return Episode(torch.cat(sx), torch.tensor(sy), torch.cat(qx), torch.tensor(qy))


def pairwise_distance(a: torch.Tensor, b: torch.Tensor, metric: str = "euclidean") -> torch.Tensor:
    if metric == "euclidean":
        return torch.cdist(a, b).pow(2)
    if metric == "manhattan":
        return torch.cdist(a, b, p=1)
    if metric == "cosine":
        return 1 - nn.functional.normalize(a, dim=-1) @ nn.functional.normalize(b, dim=-1).t()
    raise ValueError(f"unknown distance {metric!r}")


class PrototypicalNetwork(nn.Module):
    def __init__(self, encoder: nn.Module, cfg: FewShotConfig | None = None):
        super().__init__()
        self.encoder, self.cfg = encoder, cfg or FewShotConfig()

    def prototypes(self, support_x, support_y):
        z = self.encoder(support_x)
        return torch.stack([z[support_y == c].mean(0) for c in range(int(support_y.max()) + 1)])

    def forward(self, ep: Episode):
        """Logits of the query examples: negative distances to the class prototypes."""
        return -pairwise_distance(self.encoder(ep.query_x), self.prototypes(ep.support_x, ep.support_y), self.cfg.distance)

    def loss(self, ep: Episode):
        logits = self(ep)
        return nn.functional.cross_entropy(logits, ep.query_y), (logits.argmax(-1) == ep.query_y).float().mean()


class MAML:
    """Model-agnostic meta-learning: ``adapt`` takes inner gradient steps on the support set and returns the adapted
    parameters; ``meta_loss`` evaluates them on the query set, differentiable w.r.t. the initial parameters."""

    def __init__(self, model: nn.Module, cfg: FewShotConfig | None = None):
        self.model, self.cfg = model, cfg or FewShotConfig()

    def adapt(self, ep: Episode, create_graph: bool | None = None) -> dict:
        cg = (not self.cfg.first_order) if create_graph is None else create_graph
        params = dict(self.model.named_parameters())
        for _ in range(self.cfg.inner_steps):
            loss = nn.functional.cross_entropy(torch.func.functional_call(self.model, params, (ep.support_x,)), ep.support_y)
            grads = torch.autograd.grad(loss, list(params.values()), create_graph=cg)
            params = {n: p - self.cfg.inner_lr * g for (n, p), g in zip(params.items(), grads)}
        return params

    def meta_loss(self, ep: Episode):
        logits = torch.func.functional_call(self.model, self.adapt(ep), (ep.query_x,))
        return nn.functional.cross_entropy(logits, ep.query_y), (logits.argmax(-1) == ep.query_y).float().mean()


class Reptile:
    """First-order meta-learning: train a copy on the task for a few SGD steps, then move the initial weights a
    fraction ``meta_lr`` of the way towards the trained copy."""

    def __init__(self, model: nn.Module, cfg: FewShotConfig | None = None, meta_lr: float = 0.1):
        self.model, self.cfg, self.meta_lr = model, cfg or FewShotConfig(), meta_lr

    def inner_train(self, ep: Episode) -> nn.Module:
        fast = copy.deepcopy(self.model)
        opt = torch.optim.SGD(fast.parameters(), lr=self.cfg.inner_lr)
        for _ in range(self.cfg.inner_steps):
            opt.zero_grad()
            nn.functional.cross_entropy(fast(ep.support_x), ep.support_y).backward()
            opt.step()
        return fast

    @torch.no_grad()
    def _interpolate(self, fast: nn.Module):
        for p, q in zip(self.model.parameters(), fast.parameters()):
            p.add_(self.meta_lr * (q - p))

    def meta_step(self, ep: Episode) -> float:
        fast = self.inner_train(ep)
        with torch.no_grad():
            acc = float((fast(ep.query_x).argmax(-1) == ep.query_y).float().mean())
        self._interpolate(fast)
        return acc


@dataclass
class FewShotMetrics:
    mean_accuracy: float
    ci95: float
    episodes: int


class FewShotEvaluator:
    def __init__(self, dataset: FewShotDataset, episodes: int = 100):
        self.ds, self.episodes = dataset, episodes

    @torch.no_grad()
    def evaluate(self, predict) -> FewShotMetrics:
        """``predict(episode) -> logits [Q, N]`` for the query set."""
        accs = []
        for _ in range(self.episodes):
            ep = self.ds.sample_episode()
            with torch.enable_grad():
                logits = predict(ep)
            accs.append(float((logits.argmax(-1) == ep.query_y).float().mean()))
        m = sum(accs) / len(accs)
        sd = math.sqrt(sum((a - m) ** 2 for a in accs) / max(len(accs) - 1, 1))
        return FewShotMetrics(m, 1.96 * sd / math.sqrt(len(accs)), len(accs))
