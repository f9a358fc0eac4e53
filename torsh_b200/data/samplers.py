"""Index samplers beyond the PyTorch set (``crates/torsh-data/src/sampler/{stratified,importance,curriculum,
active_learning,adaptive,batch,weighted,advanced}.rs``).  Every sampler draws from its own seeded generator, exposes
``set_epoch`` where the order depends on the epoch, and yields plain integer indices (batch samplers yield lists)."""
from __future__ import annotations

import math
from typing import Callable, Iterator, Sequence

import torch
from torch.utils.data import Sampler


class _Seeded(Sampler):
    def __init__(self, seed: int = 0):
        self.seed, self.epoch = seed, 0

    def set_epoch(self, epoch: int): self.epoch = epoch
    def _gen(self): return torch.Generator().manual_seed(self.seed + 1_000_003 * self.epoch)


class StratifiedSampler(_Seeded):
    """Every window of ``num_classes`` consecutive draws contains the classes in proportion: indices of each class are
    shuffled, then interleaved by largest remaining share, so every batch mirrors the label distribution."""

    def __init__(self, labels: Sequence[int], seed: int = 0):
        super().__init__(seed)
        self.labels = torch.as_tensor(labels)

    def __len__(self): return len(self.labels)

    def __iter__(self) -> Iterator[int]:
        g = self._gen()
        pools = {int(c): (self.labels == c).nonzero().flatten()[torch.randperm(int((self.labels == c).sum()), generator=g)].tolist() for c in self.labels.unique()}
        total = {c: len(p) for c, p in pools.items()}
        taken = {c: 0 for c in pools}
        for k in range(1, len(self.labels) + 1):
            c = max((c for c in pools if taken[c] < total[c]), key=lambda c: total[c] * k / len(self.labels) - taken[c])
            yield pools[c][taken[c]]
            taken[c] += 1


class StratifiedSplit:
    """Train / validation split that keeps class proportions (each class is cut at the same fraction)."""

    def __init__(self, labels, val_fraction: float = 0.2, seed: int = 0):
        g = torch.Generator().manual_seed(seed)
        labels = torch.as_tensor(labels)
        tr, va = [], []
        for c in labels.unique():
            idx = (labels == c).nonzero().flatten()
            idx = idx[torch.randperm(len(idx), generator=g)]
            k = max(1, int(round(len(idx) * val_fraction))) if len(idx) > 1 else 0
            va += idx[:k].tolist(); tr += idx[k:].tolist()
        self.train, self.val = sorted(tr), sorted(va)


class ImportanceSampler(_Seeded):
    """Draws with probability proportional to ``weight ** alpha`` (smoothed with ``eps``), reports the importance
    weights ``(1 / (N p_i)) ** beta`` that un-bias the loss, and accepts weight updates between epochs."""

    def __init__(self, weights: torch.Tensor, num_samples: int | None = None, alpha: float = 1.0, beta: float = 1.0, eps: float = 1e-6, seed: int = 0):
        super().__init__(seed)
        self.weights, self.alpha, self.beta, self.eps = weights.double().clone(), alpha, beta, eps
        self.num_samples = num_samples or len(weights)

    def probabilities(self):
        p = (self.weights + self.eps) ** self.alpha
        return p / p.sum()

    def correction(self, indices) -> torch.Tensor:
        w = (1.0 / (len(self.weights) * self.probabilities()[indices])) ** self.beta
        return (w / w.max()).float()

    def update_weights(self, indices, values): self.weights[torch.as_tensor(indices)] = torch.as_tensor(values, dtype=torch.float64)
    def __len__(self): return self.num_samples
    def __iter__(self): return iter(torch.multinomial(self.probabilities(), self.num_samples, True, generator=self._gen()).tolist())


class CurriculumSampler(_Seeded):
    """Samples only from the easiest share of the data, a share that grows with the epoch: ``linear``, ``root`` or
    ``exponential`` pacing from ``start_fraction`` to everything at ``full_epoch``; optional anti-curriculum."""

    def __init__(self, difficulty: torch.Tensor, start_fraction: float = 0.2, full_epoch: int = 10, pacing: str = "linear", reverse: bool = False, seed: int = 0):
        super().__init__(seed)
        self.order = torch.argsort(difficulty, descending=reverse, stable=True)
        self.start, self.full_epoch, self.pacing = start_fraction, full_epoch, pacing

    def fraction(self) -> float:
        t = min(1.0, self.epoch / max(self.full_epoch, 1))
        if self.pacing == "root":
            t = math.sqrt(t)
        elif self.pacing == "exponential":
            t = (math.exp(3 * t) - 1) / (math.exp(3) - 1)
        return min(1.0, self.start + (1 - self.start) * t)

    def __len__(self): return max(1, int(round(self.fraction() * len(self.order))))

    def __iter__(self):
        pool = self.order[:len(self)]
        return iter(pool[torch.randperm(len(pool), generator=self._gen())].tolist())


class ActiveLearningSampler:
    """Pool-based query selection from model probabilities ``[N, C]`` over the unlabelled pool: ``uncertainty`` (least
    confidence), ``margin``, ``entropy``, ``random``, or ``diverse`` (k-centre greedy on features among the most uncertain)."""

    def __init__(self, pool_size: int, strategy: str = "entropy", seed: int = 0):
        self.unlabelled, self.labelled, self.strategy = set(range(pool_size)), [], strategy
        self.gen = torch.Generator().manual_seed(seed)

    @staticmethod
    def scores(probs: torch.Tensor, strategy: str) -> torch.Tensor:
        if strategy == "uncertainty":
            return 1 - probs.max(1).values
        if strategy == "margin":
            top = probs.topk(2, 1).values
            return -(top[:, 0] - top[:, 1])
        return -(probs * probs.clamp(min=1e-12).log()).sum(1)

    def query(self, probs: torch.Tensor, k: int, features: torch.Tensor | None = None) -> list[int]:
        pool = sorted(self.unlabelled)
        k = min(k, len(pool))
        if self.strategy == "random":
            pick = [pool[i] for i in torch.randperm(len(pool), generator=self.gen)[:k].tolist()]
        elif self.strategy == "diverse":
            s = self.scores(probs[pool], "entropy")
            cand = [pool[i] for i in s.topk(min(len(pool), 4 * k)).indices.tolist()]
            f = features[cand]
            chosen = [0]
            d = (f - f[0]).norm(dim=1)
            while len(chosen) < k:
                nxt = int(d.argmax())
                chosen.append(nxt)
                d = torch.minimum(d, (f - f[nxt]).norm(dim=1))
            pick = [cand[i] for i in chosen]
        else:
            s = self.scores(probs[pool], self.strategy)
            pick = [pool[i] for i in s.topk(k).indices.tolist()]
        self.unlabelled -= set(pick)
        self.labelled += pick
        return pick


class AdaptiveSampler(_Seeded):
    """Loss-driven sampling: keeps an exponential average of each example's loss and mixes ``explore`` uniform draws with
    draws proportional to that average, so hard examples recur without starving the rest."""

    def __init__(self, n: int, explore: float = 0.2, momentum: float = 0.8, seed: int = 0):
        super().__init__(seed)
        self.loss, self.seen, self.explore, self.momentum = torch.ones(n, dtype=torch.float64), torch.zeros(n, dtype=torch.long), explore, momentum

    def update(self, indices, losses):
        idx, l = torch.as_tensor(indices), torch.as_tensor(losses, dtype=torch.float64)
        first = self.seen[idx] == 0
        self.loss[idx] = torch.where(first, l, self.momentum * self.loss[idx] + (1 - self.momentum) * l)
        self.seen[idx] += 1

    def probabilities(self):
        p = self.loss.clamp(min=0) + 1e-12
        return self.explore / len(p) + (1 - self.explore) * p / p.sum()

    def __len__(self): return len(self.loss)
    def __iter__(self): return iter(torch.multinomial(self.probabilities(), len(self.loss), True, generator=self._gen()).tolist())


class BucketBatchSampler(_Seeded):
    """Batches of similar length: indices are sorted by length inside shuffled chunks of ``bucket_size`` batches, cut into
    batches, and the batch order is shuffled; ``max_tokens`` caps ``batch * longest`` instead of the count."""

    def __init__(self, lengths: Sequence[int], batch_size: int, bucket_size: int = 50, max_tokens: int | None = None, drop_last: bool = False, seed: int = 0):
        super().__init__(seed)
        self.lengths, self.batch_size, self.bucket, self.max_tokens, self.drop_last = list(lengths), batch_size, bucket_size, max_tokens, drop_last

    def _batches(self):
        g = self._gen()
        perm = torch.randperm(len(self.lengths), generator=g).tolist()
        chunk = self.batch_size * self.bucket
        out = []
        for s in range(0, len(perm), chunk):
            part = sorted(perm[s:s + chunk], key=lambda i: self.lengths[i])
            cur, longest = [], 0
            for i in part:
                nl = max(longest, self.lengths[i])
                if cur and (len(cur) >= self.batch_size or (self.max_tokens and nl * (len(cur) + 1) > self.max_tokens)):
                    out.append(cur)
                    cur, nl = [], self.lengths[i]
                cur.append(i)
                longest = nl
            if cur and not (self.drop_last and len(cur) < self.batch_size):
                out.append(cur)
        return [out[i] for i in torch.randperm(len(out), generator=g).tolist()]

    def __len__(self): return len(self._batches())
    def __iter__(self): return iter(self._batches())


class BalancedBatchSampler(_Seeded):
    """``classes_per_batch`` classes with ``samples_per_class`` examples each (metric-learning batches); classes with too
    few examples are re-sampled with replacement."""

    def __init__(self, labels, classes_per_batch: int, samples_per_class: int, num_batches: int | None = None, seed: int = 0):
        super().__init__(seed)
        labels = torch.as_tensor(labels)
        self.by_class = {int(c): (labels == c).nonzero().flatten() for c in labels.unique()}
        self.p, self.k = classes_per_batch, samples_per_class
        self.num_batches = num_batches or len(labels) // (self.p * self.k)

    def __len__(self): return self.num_batches

    def __iter__(self):
        g, classes = self._gen(), list(self.by_class)
        for _ in range(self.num_batches):
            batch = []
            for ci in torch.randperm(len(classes), generator=g)[:self.p].tolist():
                idx = self.by_class[classes[ci]]
                pick = torch.randperm(len(idx), generator=g)[:self.k] if len(idx) >= self.k else torch.randint(0, len(idx), (self.k,), generator=g)
                batch += idx[pick].tolist()
            yield batch


class WeightedClassSampler(_Seeded):
    """Re-balances classes: every example is drawn with probability inverse to its class frequency (``power`` softens it)."""

    def __init__(self, labels, num_samples: int | None = None, power: float = 1.0, seed: int = 0):
        super().__init__(seed)
        labels = torch.as_tensor(labels)
        counts = torch.bincount(labels).double()
        self.weights = (1.0 / counts[labels]) ** power
        self.num_samples = num_samples or len(labels)

    def __len__(self): return self.num_samples
    def __iter__(self): return iter(torch.multinomial(self.weights, self.num_samples, True, generator=self._gen()).tolist())


class SubsetRandomSampler(_Seeded):
    def __init__(self, indices, seed: int = 0):
        super().__init__(seed)
        self.indices = list(indices)

    def __len__(self): return len(self.indices)
    def __iter__(self): return iter([self.indices[i] for i in torch.randperm(len(self.indices), generator=self._gen()).tolist()])


class InfiniteSampler(_Seeded):
    """Endless stream of shuffled epochs (for step-based training loops)."""

    def __init__(self, n: int, shuffle: bool = True, seed: int = 0):
        super().__init__(seed)
        self.n, self.shuffle = n, shuffle

    def __iter__(self):
        while True:
            yield from (torch.randperm(self.n, generator=self._gen()).tolist() if self.shuffle else range(self.n))
            self.epoch += 1
