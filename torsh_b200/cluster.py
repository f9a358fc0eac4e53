"""Clustering (``crates/torsh-cluster``): k-means (k-means++ init), DBSCAN, Gaussian mixture (EM, diagonal covariance),
agglomerative (average linkage), spectral clustering, and evaluation (silhouette, Davies-Bouldin, adjusted Rand).
All run on tensors of any device."""
from __future__ import annotations

import math

import torch


def kmeans(x: torch.Tensor, k: int, iters: int = 100, tol: float = 1e-4, seed: int = 0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = x.shape[0]
    c = x[torch.randint(0, n, (1,), generator=g)].clone()
    for _ in range(1, k):  # k-means++
        d = torch.cdist(x, c).min(1).values ** 2
        c = torch.cat([c, x[torch.multinomial((d / d.sum()).cpu(), 1, generator=g).to(x.device)]])
    for _ in range(iters):
        lab = torch.cdist(x, c).argmin(1)
        new = torch.stack([x[lab == j].mean(0) if (lab == j).any() else c[j] for j in range(k)])
        shift = (new - c).norm()
        c = new
        if shift < tol:
            break
    return lab, c, (torch.cdist(x, c).min(1).values ** 2).sum().item()


def dbscan(x: torch.Tensor, eps: float, min_samples: int = 5) -> torch.Tensor:
    n = x.shape[0]
    nb = torch.cdist(x, x) <= eps
    core = nb.sum(1) >= min_samples
    lab = torch.full((n,), -1, dtype=torch.long)
    cid = 0
    for i in range(n):
        if lab[i] != -1 or not core[i]:
            continue
        stack, lab[i] = [i], cid
        while stack:
            j = stack.pop()
            if not core[j]:
                continue
            for m in nb[j].nonzero().flatten().tolist():
                if lab[m] == -1:
                    lab[m] = cid
                    stack.append(m)
        cid += 1
    return lab


class GaussianMixture:
    def __init__(self, k: int, iters: int = 100, tol: float = 1e-4, seed: int = 0):
        self.k, self.iters, self.tol, self.seed = k, iters, tol, seed

    def fit(self, x: torch.Tensor):
        _, self.mu, _ = kmeans(x, self.k, 10, seed=self.seed)
        self.var = x.var(0).expand(self.k, -1).clone() + 1e-6
        self.pi = torch.full((self.k,), 1.0 / self.k, device=x.device)
        prev = -math.inf
        for _ in range(self.iters):
            lp = self._log_prob(x)
            ll = torch.logsumexp(lp, 1)
            r = (lp - ll[:, None]).exp()
            nk = r.sum(0) + 1e-10
            self.mu = (r.t() @ x) / nk[:, None]
            self.var = (r.t() @ (x * x)) / nk[:, None] - self.mu ** 2 + 1e-6
            self.pi = nk / x.shape[0]
            if abs(ll.mean().item() - prev) < self.tol:
                break
            prev = ll.mean().item()
        return self

    def _log_prob(self, x):
        d = x[:, None, :] - self.mu[None]
        return self.pi.log()[None] - 0.5 * ((d * d) / self.var[None] + self.var.log()[None] + math.log(2 * math.pi)).sum(-1)

    def predict(self, x): return self._log_prob(x).argmax(1)
    def score(self, x): return torch.logsumexp(self._log_prob(x), 1).mean().item()


def agglomerative(x: torch.Tensor, k: int) -> torch.Tensor:
    n = x.shape[0]
    clusters = [[i] for i in range(n)]
    d = torch.cdist(x, x)
    while len(clusters) > k:
        best, pair = math.inf, None
        for a in range(len(clusters)):
            for b in range(a + 1, len(clusters)):
                v = d[clusters[a]][:, clusters[b]].mean().item()
                if v < best:
                    best, pair = v, (a, b)
        a, b = pair
        clusters[a] += clusters.pop(b)
    lab = torch.empty(n, dtype=torch.long)
    for c, idx in enumerate(clusters):
        lab[idx] = c
    return lab


def spectral_clustering(x: torch.Tensor, k: int, gamma: float = 1.0, seed: int = 0) -> torch.Tensor:
    w = torch.exp(-gamma * torch.cdist(x, x) ** 2)
    dinv = w.sum(1).rsqrt()
    lap = torch.eye(x.shape[0], device=x.device) - dinv[:, None] * w * dinv[None]
    _, vec = torch.linalg.eigh(lap)
    emb = torch.nn.functional.normalize(vec[:, :k], dim=1)
    return kmeans(emb, k, seed=seed)[0]


def silhouette_score(x: torch.Tensor, lab: torch.Tensor) -> float:
    d = torch.cdist(x, x)
    ks = lab.unique()
    s = []
    for i in range(x.shape[0]):
        own = lab == lab[i]
        a = d[i][own].sum() / max(own.sum().item() - 1, 1)
        b = min(d[i][lab == k].mean() for k in ks if k != lab[i]) if len(ks) > 1 else torch.tensor(0.0)
        s.append(((b - a) / max(a, b, torch.tensor(1e-12))).item())
    return sum(s) / len(s)


def davies_bouldin(x, lab) -> float:
    ks = lab.unique()
    c = torch.stack([x[lab == k].mean(0) for k in ks])
    s = torch.stack([(x[lab == k] - c[i]).norm(dim=1).mean() for i, k in enumerate(ks)])
    m = torch.cdist(c, c) + torch.eye(len(ks)) * 1e12
    return ((s[:, None] + s[None]) / m).max(1).values.mean().item()


def adjusted_rand_index(a: torch.Tensor, b: torch.Tensor) -> float:
    ka, kb = a.unique(), b.unique()
    cont = torch.tensor([[((a == i) & (b == j)).sum().item() for j in kb] for i in ka], dtype=torch.float64)
    comb = lambda v: (v * (v - 1) / 2).sum()
    s, sa, sb, n = comb(cont), comb(cont.sum(1)), comb(cont.sum(0)), len(a)
    exp = sa * sb / (n * (n - 1) / 2)
    return ((s - exp) / (0.5 * (sa + sb) - exp)).item()
