"""Clustering (``crates/torsh-cluster``): k-means (k-means++ / Forgy / random-partition init), DBSCAN with parameter
suggestion, OPTICS, Gaussian mixture (EM, diagonal covariance), agglomerative with a merge tree (single / complete /
average / ward), spectral clustering, streaming k-means with drift detectors (Page-Hinkley, ADWIN, DDM), feature scaling,
and evaluation (silhouette, Davies-Bouldin, Calinski-Harabasz, Dunn, gap statistic, Rand / adjusted Rand, mutual-information
family, V-measure, Fowlkes-Mallows, Jaccard, purity). All run on tensors of any device."""
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


# ---- hierarchical clustering with a dendrogram (crates/torsh-cluster/src/algorithms/hierarchical.rs) -----------------------
class HierarchicalResult:
    """Merge history in the usual ``[a, b, distance, size]`` rows (ids >= n name earlier merges)."""

    def __init__(self, n: int, steps: list):
        self.n, self.steps = n, steps

    def _labels(self, keep) -> torch.Tensor:
        parent = list(range(self.n + len(self.steps)))
        def find(v):
            while parent[v] != v:
                parent[v] = parent[parent[v]]
                v = parent[v]
            return v
        for i, (a, b, d, _) in enumerate(self.steps):
            if keep(i, d):
                parent[find(a)] = parent[find(b)] = self.n + i
        roots = [find(i) for i in range(self.n)]
        ids = {r: c for c, r in enumerate(dict.fromkeys(roots))}
        return torch.tensor([ids[r] for r in roots])

    def flat_clusters(self, k: int) -> torch.Tensor:
        if not 1 <= k <= self.n:
            raise ValueError("number of clusters must lie in 1..n")
        return self._labels(lambda i, d: i < self.n - k)

    def clusters_by_distance(self, threshold: float) -> torch.Tensor:
        return self._labels(lambda i, d: d <= threshold)


def linkage(x: torch.Tensor, method: str = "average") -> HierarchicalResult:
    """Agglomerative merge tree by the Lance-Williams update: single, complete, average or ward."""
    if method not in ("single", "complete", "average", "ward"):
        raise ValueError(f"unknown linkage {method!r}")
    n = x.shape[0]
    d = torch.cdist(x.double(), x.double())
    if method == "ward":
        d = d ** 2
    d.fill_diagonal_(math.inf)
    size = torch.ones(n, dtype=torch.float64)
    ids, alive, steps = list(range(n)), torch.ones(n, dtype=torch.bool), []
    for s in range(n - 1):
        flat = int(d.argmin())
        a, b = sorted(divmod(flat, n))
        dab = d[a, b].item()
        na, nb = size[a], size[b]
        if method == "single":
            new = torch.minimum(d[a], d[b])
        elif method == "complete":
            new = torch.maximum(d[a], d[b])
        elif method == "average":
            new = (na * d[a] + nb * d[b]) / (na + nb)
        else:
            tot = na + nb + size
            new = ((na + size) * d[a] + (nb + size) * d[b] - size * dab) / tot
        steps.append((ids[a], ids[b], math.sqrt(dab) if method == "ward" else dab, int(na + nb)))
        new[~alive] = math.inf
        d[a], d[:, a] = new, new
        d[a, a] = math.inf
        d[b], d[:, b] = math.inf, math.inf
        alive[b] = False
        size[a] = na + nb
        ids[a] = n + s
    return HierarchicalResult(n, steps)


class AgglomerativeClustering:
    def __init__(self, n_clusters: int, linkage: str = "ward"):
        self.n_clusters, self.method = n_clusters, linkage

    def fit(self, x):
        self.result = linkage(x, self.method)
        self.labels = self.result.flat_clusters(self.n_clusters)
        return self


# ---- OPTICS (crates/torsh-cluster/src/algorithms/optics.rs) -----------------------------------------------------------------
class OPTICS:
    """Ordering points by reachability; clusters are cut at ``eps`` (DBSCAN-like) from the reachability plot."""

    def __init__(self, max_eps: float = math.inf, min_samples: int = 5):
        self.max_eps, self.min_samples = max_eps, min_samples

    def fit(self, x: torch.Tensor):
        n = x.shape[0]
        d = torch.cdist(x.double(), x.double())
        core = d.kthvalue(min(self.min_samples, n), dim=1).values
        core = torch.where(core <= self.max_eps, core, torch.full_like(core, math.inf))
        reach = torch.full((n,), math.inf, dtype=torch.float64)
        done = torch.zeros(n, dtype=torch.bool)
        order, pred = [], torch.full((n,), -1, dtype=torch.long)
        for start in range(n):
            if done[start]:
                continue
            p = start
            while True:
                done[p] = True
                order.append(p)
                if core[p] < math.inf:
                    cand = torch.maximum(d[p], core[p])
                    upd = (~done) & (d[p] <= self.max_eps) & (cand < reach)
                    reach[upd] = cand[upd]
                    pred[upd] = p
                pending = torch.where(done, torch.full_like(reach, math.inf), reach)
                if not torch.isfinite(pending).any():
                    break
                p = int(pending.argmin())
        self.ordering, self.reachability, self.core_distances, self.predecessor = torch.tensor(order), reach, core, pred
        return self

    def extract_dbscan(self, eps: float) -> torch.Tensor:
        lab = torch.full((len(self.ordering),), -1, dtype=torch.long)
        cid = -1
        for p in self.ordering.tolist():
            if self.reachability[p] > eps:
                if self.core_distances[p] <= eps:
                    cid += 1
                    lab[p] = cid
            else:
                lab[p] = cid
        return lab


# ---- streaming k-means and drift detection (algorithms/incremental.rs, utils/drift_detection.rs) ----------------------------
class OnlineKMeans:
    """Sequential k-means: each point moves its nearest centre by ``1/count`` (or a fixed learning rate)."""

    def __init__(self, n_clusters: int, learning_rate: float | None = None, drift_threshold: float = math.inf, seed: int = 0):
        self.k, self.lr, self.drift_threshold, self.seed = n_clusters, learning_rate, drift_threshold, seed
        self.centers, self.counts, self.n_seen, self.drift_events = None, None, 0, 0
        self._ema = None

    def partial_fit(self, x: torch.Tensor):
        x = x.reshape(-1, x.shape[-1])
        for p in x:
            if self.centers is None or len(self.centers) < self.k:
                self.centers = p[None].clone() if self.centers is None else torch.cat([self.centers, p[None]])
                self.counts = torch.ones(len(self.centers))
                self.n_seen += 1
                continue
            dist = (self.centers - p).norm(dim=1)
            j = int(dist.argmin())
            self.counts[j] += 1
            eta = self.lr if self.lr is not None else 1.0 / self.counts[j].item()
            self.centers[j] += eta * (p - self.centers[j])
            self.n_seen += 1
            dmin = dist[j].item()
            if self._ema is not None and dmin > self.drift_threshold * max(self._ema, 1e-12):
                self.drift_events += 1
            self._ema = dmin if self._ema is None else 0.99 * self._ema + 0.01 * dmin
        return self

    def predict(self, x): return torch.cdist(x, self.centers).argmin(1)


class SlidingWindowKMeans:
    """k-means re-fitted on the most recent ``window_size`` points every ``recompute_frequency`` arrivals."""

    def __init__(self, n_clusters: int, window_size: int = 1000, recompute_frequency: int = 100, seed: int = 0):
        self.k, self.window_size, self.freq, self.seed = n_clusters, window_size, recompute_frequency, seed
        self.window, self.centers, self._since, self.n_refits = None, None, 0, 0

    def partial_fit(self, x: torch.Tensor):
        self.window = x if self.window is None else torch.cat([self.window, x])[-self.window_size:]
        self._since += len(x)
        if len(self.window) >= self.k and (self.centers is None or self._since >= self.freq):
            _, self.centers, _ = kmeans(self.window, self.k, seed=self.seed)
            self._since, self.n_refits = 0, self.n_refits + 1
        return self

    def predict(self, x): return torch.cdist(x, self.centers).argmin(1)


STABLE, WARNING, DRIFT = "stable", "warning", "drift"


class PageHinkley:
    """Cumulative deviation from the running mean; drift when it rises ``lambda`` above its minimum."""

    def __init__(self, delta: float = 0.005, lam: float = 50.0, alpha: float = 0.9999):
        self.delta, self.lam, self.alpha = delta, lam, alpha
        self.reset()

    def reset(self): self.n, self.mean, self.cum, self.min_cum = 0, 0.0, 0.0, 0.0

    def update(self, v: float) -> str:
        self.n += 1
        self.mean += (v - self.mean) / self.n
        self.cum = self.alpha * self.cum + (v - self.mean - self.delta)
        self.min_cum = min(self.min_cum, self.cum)
        stat = self.cum - self.min_cum
        if stat > self.lam:
            self.reset()
            return DRIFT
        return WARNING if stat > 0.5 * self.lam else STABLE

    @property
    def statistic(self): return self.cum - self.min_cum


class ADWIN:
    """Adaptive window: drops the oldest part whenever two sub-windows differ by more than the Hoeffding bound."""

    def __init__(self, delta: float = 0.002, max_window_size: int = 1000):
        self.delta, self.max_window, self.window, self.n_detections = delta, max_window_size, [], 0

    def reset(self): self.window, self.n_detections = [], 0

    @property
    def window_size(self): return len(self.window)

    def update(self, v: float) -> str:
        self.window.append(float(v))
        if len(self.window) > self.max_window:
            self.window.pop(0)
        w = torch.tensor(self.window, dtype=torch.float64)
        n = len(w)
        if n < 10:
            return STABLE
        cs = w.cumsum(0)
        n0 = torch.arange(5, n - 4, dtype=torch.float64)
        m0 = cs[4:n - 5] / n0
        m1 = (cs[-1] - cs[4:n - 5]) / (n - n0)
        harm = 1.0 / (1.0 / n0 + 1.0 / (n - n0))
        eps = torch.sqrt(torch.log(torch.tensor(4.0 * n / self.delta)) / (2 * harm))
        hit = ((m0 - m1).abs() > eps).nonzero()
        if len(hit):
            cut = int(n0[hit[-1, 0]])
            self.window = self.window[cut:]
            self.n_detections += 1
            return DRIFT
        return STABLE


class DDM:
    """Drift detection on a 0/1 error stream: warn / alarm when p + s exceeds its minimum by 2 / 3 deviations."""

    def __init__(self, min_instances: int = 30, warning_level: float = 2.0, drift_level: float = 3.0):
        self.min_instances, self.wl, self.dl = min_instances, warning_level, drift_level
        self.reset()

    def reset(self): self.n, self.p, self.p_min, self.s_min = 0, 0.0, math.inf, math.inf

    @property
    def error_rate(self): return self.p

    def update(self, err: float) -> str:
        self.n += 1
        self.p += (err - self.p) / self.n
        s = math.sqrt(self.p * (1 - self.p) / self.n)
        if self.n < self.min_instances:
            return STABLE
        if self.p + s < self.p_min + self.s_min:
            self.p_min, self.s_min = self.p, s
        if self.p + s > self.p_min + self.dl * self.s_min:
            self.reset()
            return DRIFT
        return WARNING if self.p + s > self.p_min + self.wl * self.s_min else STABLE


class CompositeDriftDetector:
    """Majority vote of Page-Hinkley, ADWIN and (when an error is given) DDM."""

    def __init__(self):
        self.ph, self.adwin, self.ddm = PageHinkley(), ADWIN(), DDM()

    def update(self, value: float, error: float | None = None) -> str:
        votes = [self.ph.update(value), self.adwin.update(value)] + ([self.ddm.update(error)] if error is not None else [])
        if votes.count(DRIFT) >= 2 or (len(votes) == 2 and DRIFT in votes):
            return DRIFT
        return WARNING if DRIFT in votes or WARNING in votes else STABLE

    def reset(self):
        for d in (self.ph, self.adwin, self.ddm):
            d.reset()


# ---- initialisation, preprocessing, parameter suggestion (initialization/*.rs, utils/{preprocessing,adaptive}.rs) -----------
def init_forgy(x, k, seed=0):
    return x[torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(seed))[:k]].clone()


def init_random_partition(x, k, seed=0):
    lab = torch.randint(0, k, (x.shape[0],), generator=torch.Generator().manual_seed(seed))
    lab[:k] = torch.arange(k)
    return torch.stack([x[lab == j].mean(0) for j in range(k)])


def init_kmeans_plus_plus(x, k, seed=0):
    g = torch.Generator().manual_seed(seed)
    c = x[torch.randint(0, x.shape[0], (1,), generator=g)].clone()
    for _ in range(1, k):
        d = torch.cdist(x, c).min(1).values ** 2
        c = torch.cat([c, x[torch.multinomial((d / d.sum()).cpu(), 1, generator=g)]])
    return c


def standardize_features(x): return (x - x.mean(0)) / x.std(0, unbiased=False).clamp(min=1e-12)
def normalize_features(x): return (x - x.min(0).values) / (x.max(0).values - x.min(0).values).clamp(min=1e-12)
def unit_normalize(x): return torch.nn.functional.normalize(x, dim=1)


def robust_scale(x):
    q = torch.quantile(x, torch.tensor([0.25, 0.5, 0.75], dtype=x.dtype), dim=0)
    return (x - q[1]) / (q[2] - q[0]).clamp(min=1e-12)


def suggest_epsilon(x: torch.Tensor, min_samples: int = 5) -> float:
    """Knee of the sorted k-distance curve: the point furthest from the chord between its ends."""
    kd = torch.cdist(x, x).kthvalue(min(min_samples + 1, x.shape[0]), dim=1).values.sort().values.double()
    n = len(kd)
    t = torch.linspace(0, 1, n, dtype=torch.float64)
    y = (kd - kd[0]) / (kd[-1] - kd[0]).clamp(min=1e-12)
    return float(kd[int((t - y).argmax())])


def suggest_dbscan_params(x: torch.Tensor):
    ms = max(2 * x.shape[1], 4) if x.shape[1] <= 8 else x.shape[1] + 1
    return suggest_epsilon(x, ms), ms


def pairwise_distance(x, y, metric: str = "euclidean"):
    if metric == "euclidean":
        return torch.cdist(x, y)
    if metric == "manhattan":
        return torch.cdist(x, y, p=1)
    if metric == "cosine":
        return 1 - torch.nn.functional.normalize(x, dim=1) @ torch.nn.functional.normalize(y, dim=1).t()
    raise ValueError(f"unknown metric {metric!r}")


def validate_cluster_input(x: torch.Tensor, n_clusters: int | None = None):
    if x.dim() != 2 or x.shape[0] == 0 or x.shape[1] == 0:
        raise ValueError("data must be a non-empty [samples, features] matrix")
    if not torch.isfinite(x).all():
        raise ValueError("data contains NaN or infinite values")
    if n_clusters is not None and not 1 <= n_clusters <= x.shape[0]:
        raise ValueError("n_clusters must lie in 1..n_samples")


# ---- evaluation (crates/torsh-cluster/src/evaluation/metrics/*.rs) ---------------------------------------------------------
def _contingency(a, b):
    _, ia = a.unique(return_inverse=True)
    _, ib = b.unique(return_inverse=True)
    m = torch.zeros(int(ia.max()) + 1, int(ib.max()) + 1, dtype=torch.float64)
    return m.index_put_((ia, ib), torch.ones(len(a), dtype=torch.float64), accumulate=True)


def _entropy(p):
    p = p[p > 0]
    return float(-(p * p.log()).sum())


def mutual_information(a, b) -> float:
    c = _contingency(a, b)
    p = c / c.sum()
    outer = p.sum(1, keepdim=True) * p.sum(0, keepdim=True)
    nz = p > 0
    return float((p[nz] * (p[nz] / outer[nz]).log()).sum())


def normalized_mutual_info(a, b, average: str = "arithmetic") -> float:
    c = _contingency(a, b)
    ha, hb = _entropy(c.sum(1) / c.sum()), _entropy(c.sum(0) / c.sum())
    den = {"arithmetic": 0.5 * (ha + hb), "geometric": math.sqrt(ha * hb), "min": min(ha, hb), "max": max(ha, hb)}[average]
    return 1.0 if den == 0 else mutual_information(a, b) / den


def adjusted_mutual_info(a, b) -> float:
    """Mutual information corrected by its expectation under the hypergeometric model of random labelings."""
    c = _contingency(a, b)
    n = int(c.sum())
    ra, cb = c.sum(1).long().tolist(), c.sum(0).long().tolist()
    lg = lambda v: math.lgamma(v + 1)
    emi = 0.0
    for ai in ra:
        for bj in cb:
            for nij in range(max(1, ai + bj - n), min(ai, bj) + 1):
                lp = lg(ai) + lg(bj) + lg(n - ai) + lg(n - bj) - lg(n) - lg(nij) - lg(ai - nij) - lg(bj - nij) - lg(n - ai - bj + nij)
                emi += nij / n * math.log(n * nij / (ai * bj)) * math.exp(lp)
    ha, hb = _entropy(c.sum(1) / n), _entropy(c.sum(0) / n)
    den = 0.5 * (ha + hb) - emi
    return 1.0 if abs(den) < 1e-15 else (mutual_information(a, b) - emi) / den


def homogeneity_completeness_v_measure(truth, pred, beta: float = 1.0):
    c = _contingency(truth, pred)
    ht, hp = _entropy(c.sum(1) / c.sum()), _entropy(c.sum(0) / c.sum())
    mi = mutual_information(truth, pred)
    h = 1.0 if ht == 0 else mi / ht
    cm = 1.0 if hp == 0 else mi / hp
    v = 0.0 if h + cm == 0 else (1 + beta) * h * cm / (beta * h + cm)
    return h, cm, v


def _pair_counts(a, b):
    c = _contingency(a, b)
    n = c.sum()
    tp = ((c * (c - 1)) / 2).sum()
    pa, pb = (c.sum(1) * (c.sum(1) - 1) / 2).sum(), (c.sum(0) * (c.sum(0) - 1) / 2).sum()
    return float(tp), float(pa - tp), float(pb - tp), float(n * (n - 1) / 2 - pa - pb + tp)


def fowlkes_mallows(a, b) -> float:
    tp, fn, fp, _ = _pair_counts(a, b)
    return 0.0 if tp == 0 else tp / math.sqrt((tp + fp) * (tp + fn))


def rand_index(a, b) -> float:
    tp, fn, fp, tn = _pair_counts(a, b)
    return (tp + tn) / (tp + fn + fp + tn)


def jaccard_index(a, b) -> float:
    tp, fn, fp, _ = _pair_counts(a, b)
    return tp / (tp + fn + fp) if tp + fn + fp else 1.0


def purity(truth, pred) -> float:
    c = _contingency(truth, pred)
    return float(c.max(0).values.sum() / c.sum())


def calinski_harabasz(x, lab) -> float:
    ks = lab.unique()
    mu = x.mean(0)
    between = sum(float((lab == k).sum()) * float(((x[lab == k].mean(0) - mu) ** 2).sum()) for k in ks)
    within = sum(float(((x[lab == k] - x[lab == k].mean(0)) ** 2).sum()) for k in ks)
    n, k = x.shape[0], len(ks)
    return between / max(within, 1e-300) * (n - k) / (k - 1)


def dunn_index(x, lab) -> float:
    d = torch.cdist(x, x)
    same = lab[:, None] == lab[None]
    return float(d[~same].min() / d[same].max().clamp(min=1e-300))


def inertia(x, lab) -> float:
    return sum(float(((x[lab == k] - x[lab == k].mean(0)) ** 2).sum()) for k in lab.unique())


def gap_statistic(x, k_max: int = 6, n_refs: int = 8, seed: int = 0):
    """Tibshirani's gap: log within-dispersion of uniform reference sets minus that of the data, and the chosen k
    (the smallest k whose gap is within one standard error of the next)."""
    g = torch.Generator().manual_seed(seed)
    lo, hi = x.min(0).values, x.max(0).values
    gaps, sks = [], []
    for k in range(1, k_max + 1):
        wk = math.log(max(kmeans(x, k, seed=seed)[2], 1e-300))
        ref = torch.tensor([math.log(max(kmeans(lo + (hi - lo) * torch.rand(x.shape, generator=g), k, seed=seed)[2], 1e-300)) for _ in range(n_refs)])
        gaps.append(float(ref.mean()) - wk)
        sks.append(float(ref.std(unbiased=False)) * math.sqrt(1 + 1 / n_refs))
    best = next((k for k in range(1, k_max) if gaps[k - 1] >= gaps[k] - sks[k]), k_max)
    return best, gaps, sks
