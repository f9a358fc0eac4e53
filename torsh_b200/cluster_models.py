"""Estimator classes for clustering (``crates/torsh-cluster/src/{algorithms,distance,initialization,evaluation,
memory_efficient}.rs``): ``fit`` / ``predict`` / ``fit_predict`` objects with the reference's names, plus the pieces that
had no function-style counterpart in ``cluster``: HDBSCAN (mutual-reachability spanning tree, condensed tree, excess of
mass selection, membership strengths), Lloyd iterations with restarts, mini-batches and pluggable distances, chunked
assignment that never materialises the full distance matrix, Nystrom-free spectral clustering on k-nearest-neighbour
graphs, and incremental centroid updates.

The distance kernels are matrix products (``|x|^2 + |c|^2 - 2 x c^T``), so on a GPU the assignment step runs on the tensor
cores through the library GEMM and a chunk of ``chunk_size`` rows bounds the memory at ``chunk_size * k`` values."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import cluster as _c

__all__ = [
    "EuclideanDistance", "ManhattanDistance", "CosineDistance", "Forgy", "RandomPartition", "KMeansPlusPlus",
    "KMeansResult", "KMeans", "DBSCAN", "HDBSCANResult", "HDBSCAN", "SpectralClustering", "GapStatistic",
    "IncrementalCentroidUpdater", "ChunkedDataProcessor", "PageHinkleyTest", "EvaluationResult", "evaluate_clustering",
]


# ================================================================================================ distances and seeds
class EuclideanDistance:
    name = "euclidean"
    @staticmethod
    def pairwise(x, c):
        d2 = (x * x).sum(1, keepdim=True) + (c * c).sum(1)[None] - 2 * x @ c.T
        return d2.clamp(min=0).sqrt()
    @staticmethod
    def centroid(points): return points.mean(0)


class ManhattanDistance:
    name = "manhattan"
    @staticmethod
    def pairwise(x, c): return torch.cdist(x, c, p=1)
    @staticmethod
    def centroid(points): return points.median(0).values          # the L1 minimiser


class CosineDistance:
    name = "cosine"
    @staticmethod
    def pairwise(x, c): return 1 - torch.nn.functional.normalize(x, dim=1) @ torch.nn.functional.normalize(c, dim=1).T
    @staticmethod
    def centroid(points): return torch.nn.functional.normalize(torch.nn.functional.normalize(points, dim=1).mean(0), dim=0)


_DIST = {"euclidean": EuclideanDistance, "manhattan": ManhattanDistance, "cosine": CosineDistance}


class Forgy:
    def __call__(self, x, k, seed=0): return _c.init_forgy(x, k, seed)
class RandomPartition:
    def __call__(self, x, k, seed=0): return _c.init_random_partition(x, k, seed)
class KMeansPlusPlus:
    def __call__(self, x, k, seed=0): return _c.init_kmeans_plus_plus(x, k, seed)


_INIT = {"forgy": Forgy, "random_partition": RandomPartition, "k-means++": KMeansPlusPlus, "kmeans++": KMeansPlusPlus}


# ================================================================================================ chunked assignment
class ChunkedDataProcessor:
    """Nearest-centre assignment in row chunks: returns labels and distances; memory is ``chunk_size * k``."""
    def __init__(self, chunk_size: int = 65536, distance=EuclideanDistance): self.chunk, self.dist = chunk_size, distance

    def assign(self, x: torch.Tensor, centres: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        labs, ds = [], []
        for lo in range(0, len(x), self.chunk):
            d, l = self.dist.pairwise(x[lo:lo + self.chunk], centres).min(1)
            labs.append(l); ds.append(d)
        return torch.cat(labs), torch.cat(ds)

    def reduce(self, x: torch.Tensor, labels: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Per-cluster coordinate sums and counts accumulated chunk by chunk."""
        sums = torch.zeros(k, x.shape[1], dtype=x.dtype, device=x.device)
        counts = torch.zeros(k, dtype=x.dtype, device=x.device)
        for lo in range(0, len(x), self.chunk):
            l = labels[lo:lo + self.chunk]
            sums.index_add_(0, l, x[lo:lo + self.chunk])
            counts.index_add_(0, l, torch.ones(len(l), dtype=x.dtype, device=x.device))
        return sums, counts


class IncrementalCentroidUpdater:
    """Running means: ``update(batch, labels)`` moves every centre by ``sum(batch points - centre) / new count``; with
    ``decay < 1`` old counts fade so that the centres follow a drifting stream."""
    def __init__(self, centres: torch.Tensor, decay: float = 1.0):
        self.centres, self.counts, self.decay = centres.clone(), torch.zeros(len(centres), dtype=centres.dtype, device=centres.device), decay

    def update(self, batch: torch.Tensor, labels: torch.Tensor | None = None) -> torch.Tensor:
        if labels is None:
            labels = EuclideanDistance.pairwise(batch, self.centres).argmin(1)
        k = len(self.centres)
        sums = torch.zeros_like(self.centres).index_add_(0, labels, batch)
        cnt = torch.zeros_like(self.counts).index_add_(0, labels, torch.ones(len(batch), dtype=self.counts.dtype, device=batch.device))
        self.counts = self.counts * self.decay
        tot = self.counts + cnt
        hit = cnt > 0
        self.centres[hit] = (self.centres[hit] * self.counts[hit, None] + sums[hit]) / tot[hit, None]
        self.counts = tot
        return labels


# ================================================================================================ k-means
@dataclass
class KMeansResult:
    labels: torch.Tensor
    centers: torch.Tensor
    inertia: float
    n_iter: int
    converged: bool


class KMeans:
    """Lloyd's algorithm with ``n_init`` restarts (best inertia wins), a choice of seeding and distance, optional
    mini-batches (``batch_size``) and chunked assignment.  Empty clusters are re-seeded at the point farthest from its
    centre."""

    def __init__(self, n_clusters: int, init: str = "k-means++", n_init: int = 4, max_iter: int = 100, tol: float = 1e-5, distance: str = "euclidean",
                 batch_size: int | None = None, chunk_size: int = 65536, seed: int = 0):
        self.k, self.init, self.n_init, self.max_iter, self.tol = n_clusters, init, n_init, max_iter, tol
        self.dist, self.batch, self.seed = _DIST[distance], batch_size, seed
        self.proc = ChunkedDataProcessor(chunk_size, self.dist)

    def _lloyd(self, x, c, gen):
        it, converged = 0, False
        for it in range(1, self.max_iter + 1):
            if self.batch:
                idx = torch.randint(0, len(x), (self.batch,), generator=gen)
                up = self._mb
                up.update(x[idx], self.dist.pairwise(x[idx], up.centres).argmin(1))
                shift = float((up.centres - c).norm())
                c = up.centres.clone()
            else:
                lab, d = self.proc.assign(x, c)
                if self.dist is EuclideanDistance:
                    sums, cnt = self.proc.reduce(x, lab, self.k)
                    new = torch.where(cnt[:, None] > 0, sums / cnt[:, None].clamp(min=1), c)
                else:
                    new = torch.stack([self.dist.centroid(x[lab == j]) if bool((lab == j).any()) else c[j] for j in range(self.k)])
                    cnt = torch.bincount(lab, minlength=self.k)
                for j in (cnt == 0).nonzero().flatten().tolist():
                    far = int(d.argmax())
                    new[j], d[far] = x[far], 0
                shift = float((new - c).norm())
                c = new
            if shift <= self.tol * max(float(c.norm()), 1e-12):
                converged = True
                break
        lab, d = self.proc.assign(x, c)
        cost = float((d ** 2).sum()) if self.dist is EuclideanDistance else float(d.sum())
        return KMeansResult(lab, c, cost, it, converged)

    def fit(self, x: torch.Tensor) -> "KMeans":
        x = x if x.is_floating_point() else x.float()
        best = None
        gen = torch.Generator().manual_seed(self.seed)
        for r in range(self.n_init):
            c = _INIT[self.init]()(x, self.k, self.seed + r).to(x.dtype)
            if self.batch:
                self._mb = IncrementalCentroidUpdater(c)
            res = self._lloyd(x, c, gen)
            if best is None or res.inertia < best.inertia:
                best = res
        self.result = best
        self.labels_, self.cluster_centers_, self.inertia_ = best.labels, best.centers, best.inertia
        return self

    def predict(self, x: torch.Tensor) -> torch.Tensor: return self.proc.assign(x.to(self.cluster_centers_.dtype), self.cluster_centers_)[0]
    def transform(self, x: torch.Tensor) -> torch.Tensor: return self.dist.pairwise(x.to(self.cluster_centers_.dtype), self.cluster_centers_)
    def fit_predict(self, x: torch.Tensor) -> torch.Tensor: return self.fit(x).labels_


# ================================================================================================ density
class DBSCAN:
    """Density clustering with label propagation over the core-point graph (connected components by repeated
    min-label relaxation: tensor operations only); border points take the label of a neighbouring core point, the rest
    are noise (-1)."""
    def __init__(self, eps: float, min_samples: int = 5, distance: str = "euclidean"): self.eps, self.min_samples, self.dist = eps, min_samples, _DIST[distance]

    def fit(self, x: torch.Tensor) -> "DBSCAN":
        n = len(x)
        nb = self.dist.pairwise(x, x) <= self.eps
        core = nb.sum(1) >= self.min_samples
        lab = torch.arange(n)
        big = torch.full((n,), n, dtype=torch.long)
        adj = nb & core[None] & core[:, None]
        while True:
            cand = torch.where(adj, lab[None].expand(n, n), big[None].expand(n, n)).min(1).values
            new = torch.where(core, torch.minimum(lab, cand), lab)
            if torch.equal(new, lab):
                break
            lab = new
        out = torch.full((n,), -1, dtype=torch.long)
        roots = torch.unique(lab[core])
        remap = {int(r): i for i, r in enumerate(roots.tolist())}
        if len(roots):
            out[core] = torch.tensor([remap[int(v)] for v in lab[core].tolist()], dtype=torch.long)
        border = ~core & (nb & core[None]).any(1)
        if bool(border.any()):
            first_core = (nb & core[None])[border].double().argmax(1)
            out[border] = out[first_core]
        self.labels_, self.core_sample_indices_ = out, core.nonzero().flatten()
        self.n_clusters_ = len(roots)
        return self

    def fit_predict(self, x): return self.fit(x).labels_


@dataclass
class HDBSCANResult:
    labels: torch.Tensor
    probabilities: torch.Tensor
    cluster_persistence: list
    n_clusters: int
    outlier_scores: torch.Tensor


class HDBSCAN:
    """Hierarchical density clustering (Campello, Moulavi, Sander).  Core distance = distance to the ``min_samples``-th
    neighbour; mutual reachability = max(core_a, core_b, d(a, b)); its minimum spanning tree (Prim on the dense matrix)
    gives the single-linkage hierarchy; components smaller than ``min_cluster_size`` fall out of their parent instead of
    splitting it (condensed tree); the flat clustering maximises the total excess of mass (stability)."""

    def __init__(self, min_cluster_size: int = 5, min_samples: int | None = None, allow_single_cluster: bool = False):
        self.mcs, self.ms, self.single = min_cluster_size, min_samples or min_cluster_size, allow_single_cluster

    @staticmethod
    def _mst(d: torch.Tensor) -> list[tuple[int, int, float]]:
        n = len(d)
        in_tree = torch.zeros(n, dtype=torch.bool)
        best = torch.full((n,), float("inf"), dtype=d.dtype)
        src = torch.zeros(n, dtype=torch.long)
        cur, edges = 0, []
        in_tree[0] = True
        for _ in range(n - 1):
            upd = d[cur] < best
            upd &= ~in_tree
            best = torch.where(upd, d[cur], best)
            src = torch.where(upd, torch.full_like(src, cur), src)
            cand = torch.where(in_tree, torch.full_like(best, float("inf")), best)
            nxt = int(cand.argmin())
            edges.append((int(src[nxt]), nxt, float(best[nxt])))
            in_tree[nxt] = True
            cur = nxt
        return edges

    def fit(self, x: torch.Tensor) -> "HDBSCAN":
        x = x.double()
        n = len(x)
        d = torch.cdist(x, x)
        core = d.kthvalue(min(self.ms + 1, n), dim=1).values           # the point itself is the first neighbour
        mr = torch.maximum(torch.maximum(core[:, None], core[None]), d)
        edges = sorted(self._mst(mr), key=lambda e: e[2])
        # single-linkage dendrogram by union-find; node ids >= n are merges
        parent = list(range(2 * n - 1))
        size = [1] * n + [0] * (n - 1)
        children, height = {}, {}
        def find(a):
            while parent[a] != a:
                parent[a] = parent[parent[a]]
                a = parent[a]
            return a
        nxt = n
        for a, b, w in edges:
            ra, rb = find(a), find(b)
            parent[ra] = parent[rb] = nxt
            children[nxt], height[nxt], size[nxt] = (ra, rb), w, size[ra] + size[rb]
            nxt += 1
        root = nxt - 1

        def leaves(node):
            stack, out = [node], []
            while stack:
                v = stack.pop()
                if v < n:
                    out.append(v)
                else:
                    stack.extend(children[v])
            return out

        # condensed tree: walk down from the root; a split is real when both sides have >= mcs points
        clusters = {0: {"birth": 0.0, "points": {}, "children": [], "parent": None}}
        stack = [(root, 0)]
        next_id = 1
        while stack:
            node, cid = stack.pop()
            if node < n:
                clusters[cid]["points"][node] = clusters[cid]["points"].get(node, float("inf"))
                continue
            lam = 1.0 / height[node] if height[node] > 0 else float("inf")
            l, r = children[node]
            big_l, big_r = size[l] >= self.mcs, size[r] >= self.mcs
            if big_l and big_r:
                for ch in (l, r):
                    clusters[next_id] = {"birth": lam, "points": {}, "children": [], "parent": cid}
                    clusters[cid]["children"].append(next_id)
                    stack.append((ch, next_id))
                    next_id += 1
                clusters[cid]["death"] = lam
            else:
                for ch, big in ((l, big_l), (r, big_r)):
                    if big:
                        stack.append((ch, cid))
                    else:
                        for p in leaves(ch):
                            clusters[cid]["points"][p] = lam       # falls out of the cluster at this density
        for c in clusters.values():
            own = sum(min(l, c.get("death", l)) - c["birth"] for l in c["points"].values() if math.isfinite(l))
            c["stability"] = own
        # children's points leave the parent at the split: add their mass
        order = sorted(clusters, reverse=True)
        def n_points(cid):
            c = clusters[cid]
            return len(c["points"]) + sum(n_points(ch) for ch in c["children"])
        for cid in order:
            c = clusters[cid]
            if c["children"]:
                c["stability"] += sum(n_points(ch) for ch in c["children"]) * (c["death"] - c["birth"])
        selected = {}
        for cid in order:                                            # leaves first
            c = clusters[cid]
            sub = sum(selected_stab for ch in c["children"] for selected_stab in [clusters[ch]["best"]])
            if c["children"] and (sub > c["stability"] or (cid == 0 and not self.single)):
                c["best"], c["pick"] = sub, False
            else:
                c["best"], c["pick"] = c["stability"], True
        def collect(cid):
            c = clusters[cid]
            if c["pick"]:
                return [cid]
            return [s for ch in c["children"] for s in collect(ch)]
        chosen = collect(0)
        if chosen == [0] and not self.single:
            chosen = []

        def members(cid):
            c = clusters[cid]
            out = dict(c["points"])
            for ch in c["children"]:
                sub = members(ch)
                out.update({p: max(l, c["death"]) if math.isfinite(l) else c["death"] for p, l in sub.items()})
            return out
        labels = torch.full((n,), -1, dtype=torch.long)
        prob = torch.zeros(n, dtype=torch.float64)
        persistence = []
        for new_id, cid in enumerate(sorted(chosen)):
            mem = members(cid)
            lam_max = max((l for l in mem.values() if math.isfinite(l)), default=1.0)
            birth = clusters[cid]["birth"]
            for p, l in mem.items():
                labels[p] = new_id
                l = lam_max if not math.isfinite(l) else l
                prob[p] = 1.0 if lam_max <= birth else min(max((l - birth) / (lam_max - birth), 0.0), 1.0)
            persistence.append(clusters[cid]["stability"])
        lam_point = 1.0 / core.clamp(min=1e-300)
        outlier = torch.zeros(n, dtype=torch.float64)
        for cid in sorted(chosen):
            idx = torch.tensor(list(members(cid)), dtype=torch.long)
            top = lam_point[idx].max()
            outlier[idx] = 1 - lam_point[idx] / top
        outlier[labels < 0] = 1.0
        self.result = HDBSCANResult(labels, prob, persistence, len(chosen), outlier)
        self.labels_, self.probabilities_ = labels, prob
        return self

    def fit_predict(self, x): return self.fit(x).labels_


# ================================================================================================ spectral and model selection
class SpectralClustering:
    """Normalised-cut embedding: ``rbf`` affinity or a symmetrised ``knn`` graph, the ``k`` smallest eigenvectors of the
    symmetric normalised Laplacian, row normalisation, then k-means.  ``eigengap`` suggests ``k`` from the spectrum."""
    def __init__(self, n_clusters: int, affinity: str = "rbf", gamma: float = 1.0, n_neighbors: int = 10, seed: int = 0):
        self.k, self.affinity, self.gamma, self.nn, self.seed = n_clusters, affinity, gamma, n_neighbors, seed

    def _affinity(self, x):
        d = torch.cdist(x, x)
        if self.affinity == "rbf":
            return torch.exp(-self.gamma * d ** 2)
        idx = d.topk(self.nn + 1, largest=False).indices[:, 1:]
        w = torch.zeros_like(d).scatter_(1, idx, 1.0)
        return torch.maximum(w, w.T)

    def fit(self, x: torch.Tensor) -> "SpectralClustering":
        x = x.double()
        w = self._affinity(x)
        w.fill_diagonal_(0)
        dinv = w.sum(1).clamp(min=1e-12).rsqrt()
        lap = torch.eye(len(x), dtype=x.dtype) - dinv[:, None] * w * dinv[None]
        val, vec = torch.linalg.eigh(lap)
        self.eigenvalues_ = val
        emb = torch.nn.functional.normalize(vec[:, :self.k], dim=1)
        self.embedding_ = emb
        self.labels_ = KMeans(self.k, n_init=5, seed=self.seed).fit(emb).labels_
        return self

    def eigengap(self, max_k: int = 10) -> int:
        gaps = self.eigenvalues_[1:max_k + 1] - self.eigenvalues_[:max_k]
        return int(gaps.argmax()) + 1

    def fit_predict(self, x): return self.fit(x).labels_


class GapStatistic:
    def __init__(self, k_max: int = 6, n_refs: int = 8, seed: int = 0): self.k_max, self.n_refs, self.seed = k_max, n_refs, seed
    def fit(self, x) -> "GapStatistic":
        self.optimal_k_, self.gaps_, self.std_errors_ = _c.gap_statistic(x, self.k_max, self.n_refs, self.seed)
        return self


PageHinkleyTest = _c.PageHinkley


@dataclass
class EvaluationResult:
    silhouette: float
    davies_bouldin: float
    calinski_harabasz: float
    inertia: float
    n_clusters: int
    noise_fraction: float
    external: dict | None = None


def evaluate_clustering(x: torch.Tensor, labels: torch.Tensor, truth: torch.Tensor | None = None) -> EvaluationResult:
    """Internal indices on the non-noise points and, when ``truth`` is given, the external agreement scores."""
    keep = labels >= 0
    xs, ls = x[keep], labels[keep]
    k = len(torch.unique(ls))
    ok = k >= 2
    ext = None
    if truth is not None:
        ext = {"ari": _c.adjusted_rand_index(truth, labels), "nmi": _c.normalized_mutual_info(truth, labels), "purity": _c.purity(truth[keep], ls)}
    return EvaluationResult(_c.silhouette_score(xs, ls) if ok else float("nan"), _c.davies_bouldin(xs, ls) if ok else float("nan"),
                            _c.calinski_harabasz(xs, ls) if ok else float("nan"), _c.inertia(xs, ls), k, float((~keep).double().mean()), ext)
