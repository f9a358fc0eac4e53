"""Graph learning beyond :mod:`torsh_b200.graph` (``crates/torsh-graph/src``): hierarchical and global pooling
(``pool/``), message passing with edge features and E(n)-equivariant / continuous-filter layers (``conv/``, ``geometric.rs``),
heterogeneous, hyper-, temporal and knowledge graphs, explanation by gradients and mask optimisation
(``explainability.rs``), graph kernels and optimal-transport distances (``kernels.rs``, ``optimal_transport.rs``),
spectral analysis, centralities, partitioning, graph-level heads, a graph autoencoder, and text loaders
(edge list / GML / JSON).  Edge indices are ``[2, E]`` long tensors (source row 0, target row 1)."""
from __future__ import annotations

import json
import math
import re
from collections import Counter, defaultdict, deque

import torch
import torch.nn.functional as F
from torch import nn

from .graph import GCNConv, GraphData, scatter_add


def _dense_adj(edge_index, n, weight=None):
    a = torch.zeros(n, n, dtype=torch.float32 if weight is None else weight.dtype)
    a[edge_index[0], edge_index[1]] = 1.0 if weight is None else weight
    return a


# ================================================================================================ pooling
class DiffPool(nn.Module):
    """Learned soft assignment of nodes to ``clusters``: ``X' = S^T Z``, ``A' = S^T A S`` with the link-prediction and
    entropy auxiliary losses of the paper (dense adjacency)."""

    def __init__(self, cin, hidden, clusters):
        super().__init__()
        self.embed, self.assign = GCNConv(cin, hidden), GCNConv(cin, clusters)

    def forward(self, x, edge_index):
        n = x.shape[0]
        a = _dense_adj(edge_index, n)
        s = self.assign(x, edge_index).softmax(-1)
        z = F.relu(self.embed(x, edge_index))
        self.link_loss = torch.linalg.matrix_norm(a - s @ s.t()) / n
        self.entropy_loss = -(s * torch.log(s + 1e-12)).sum(-1).mean()
        self.assignment = s
        return s.t() @ z, s.t() @ a @ s


class MinCutPool(nn.Module):
    """Assignment trained by the relaxed normalised min-cut objective plus an orthogonality term."""

    def __init__(self, cin, clusters): super().__init__(); self.lin = nn.Linear(cin, clusters)

    def forward(self, x, edge_index):
        n = x.shape[0]
        a = _dense_adj(edge_index, n)
        s = self.lin(x).softmax(-1)
        d = torch.diag(a.sum(1))
        self.cut_loss = -torch.trace(s.t() @ a @ s) / torch.trace(s.t() @ d @ s).clamp(min=1e-12)
        ss = s.t() @ s
        k = s.shape[1]
        self.ortho_loss = torch.linalg.matrix_norm(ss / torch.linalg.matrix_norm(ss) - torch.eye(k) / math.sqrt(k))
        self.assignment = s
        out_a = s.t() @ a @ s
        out_a = out_a - torch.diag(out_a.diagonal())
        deg = out_a.sum(1).clamp(min=1e-12).rsqrt()
        return s.t() @ x, deg[:, None] * out_a * deg[None]


class TopKPool(nn.Module):
    """Keeps the ``ratio`` highest-scoring nodes (score = projection on a learned vector), gates their features by the
    score, and keeps the edges among them."""

    def __init__(self, cin, ratio: float = 0.5): super().__init__(); self.p, self.ratio = nn.Parameter(torch.randn(cin) / math.sqrt(cin)), ratio

    def forward(self, x, edge_index):
        score = (x @ self.p) / self.p.norm()
        k = max(1, int(math.ceil(self.ratio * x.shape[0])))
        keep = score.topk(k).indices.sort().values
        relabel = torch.full((x.shape[0],), -1, dtype=torch.long)
        relabel[keep] = torch.arange(k)
        m = (relabel[edge_index[0]] >= 0) & (relabel[edge_index[1]] >= 0)
        return x[keep] * torch.tanh(score[keep])[:, None], relabel[edge_index[:, m]], keep


class GlobalAttentionPool(nn.Module):
    def __init__(self, cin): super().__init__(); self.gate = nn.Linear(cin, 1)

    def forward(self, x, batch=None):
        batch = torch.zeros(x.shape[0], dtype=torch.long) if batch is None else batch
        g, nb = self.gate(x).squeeze(-1), int(batch.max()) + 1
        mx = torch.full((nb,), -math.inf).scatter_reduce(0, batch, g, "amax")
        e = torch.exp(g - mx[batch])
        w = e / torch.zeros(nb).index_add_(0, batch, e)[batch]
        return torch.zeros(nb, x.shape[1]).index_add_(0, batch, w[:, None] * x)


class Set2Set(nn.Module):
    """Order-invariant read-out: an LSTM queries the node set by attention for ``steps`` rounds; output ``[graphs, 2 * dim]``."""

    def __init__(self, dim, steps: int = 3): super().__init__(); self.lstm, self.steps, self.dim = nn.LSTMCell(2 * dim, dim), steps, dim

    def forward(self, x, batch=None):
        batch = torch.zeros(x.shape[0], dtype=torch.long) if batch is None else batch
        nb = int(batch.max()) + 1
        h, c, q_star = torch.zeros(nb, self.dim), torch.zeros(nb, self.dim), torch.zeros(nb, 2 * self.dim)
        for _ in range(self.steps):
            h, c = self.lstm(q_star, (h, c))
            e = (x * h[batch]).sum(-1)
            mx = torch.full((nb,), -math.inf).scatter_reduce(0, batch, e, "amax")
            a = torch.exp(e - mx[batch])
            a = a / torch.zeros(nb).index_add_(0, batch, a)[batch]
            r = torch.zeros(nb, self.dim).index_add_(0, batch, a[:, None] * x)
            q_star = torch.cat([h, r], -1)
        return q_star


# ================================================================================================ message passing with geometry / edge features
class MPNNConv(nn.Module):
    """Edge-conditioned messages ``m_ij = MLP([h_i, h_j, e_ij])`` summed at the target and combined by a GRU cell."""

    def __init__(self, dim, edge_dim):
        super().__init__()
        self.msg, self.upd = nn.Sequential(nn.Linear(2 * dim + edge_dim, dim), nn.ReLU(), nn.Linear(dim, dim)), nn.GRUCell(dim, dim)

    def forward(self, x, edge_index, edge_attr):
        src, dst = edge_index
        return self.upd(scatter_add(self.msg(torch.cat([x[dst], x[src], edge_attr], -1)), dst, x.shape[0]), x)


class EGNNLayer(nn.Module):
    """E(n)-equivariant layer (Satorras et al.): messages depend on squared distances, coordinates move along relative
    positions, so features are invariant and coordinates equivariant under rotations and translations."""

    def __init__(self, dim, hidden: int = 32):
        super().__init__()
        self.edge = nn.Sequential(nn.Linear(2 * dim + 1, hidden), nn.SiLU(), nn.Linear(hidden, hidden), nn.SiLU())
        self.coord = nn.Sequential(nn.Linear(hidden, hidden), nn.SiLU(), nn.Linear(hidden, 1, bias=False))
        self.node = nn.Sequential(nn.Linear(dim + hidden, hidden), nn.SiLU(), nn.Linear(hidden, dim))

    def forward(self, h, pos, edge_index):
        src, dst = edge_index
        rel = pos[dst] - pos[src]
        m = self.edge(torch.cat([h[dst], h[src], (rel * rel).sum(-1, keepdim=True)], -1))
        deg = torch.bincount(dst, minlength=h.shape[0]).clamp(min=1)[:, None]
        pos = pos + scatter_add(rel * self.coord(m), dst, h.shape[0]) / deg
        return h + self.node(torch.cat([h, scatter_add(m, dst, h.shape[0])], -1)), pos


class RBFLayer(nn.Module):
    def __init__(self, n: int = 16, cutoff: float = 5.0): super().__init__(); self.register_buffer("mu", torch.linspace(0, cutoff, n)); self.gamma = (n / cutoff) ** 2
    def forward(self, d): return torch.exp(-self.gamma * (d[:, None] - self.mu[None]) ** 2)


class SchNetConv(nn.Module):
    """Continuous-filter convolution: neighbour features are weighted by a filter generated from the radial-basis
    expansion of the distance, with a smooth cosine cutoff."""

    def __init__(self, dim, n_rbf: int = 16, cutoff: float = 5.0):
        super().__init__()
        self.rbf, self.cutoff = RBFLayer(n_rbf, cutoff), cutoff
        self.filter, self.lin1, self.lin2 = nn.Sequential(nn.Linear(n_rbf, dim), nn.Softplus(), nn.Linear(dim, dim)), nn.Linear(dim, dim, bias=False), nn.Sequential(nn.Linear(dim, dim), nn.Softplus(), nn.Linear(dim, dim))

    def forward(self, h, pos, edge_index):
        src, dst = edge_index
        d = (pos[dst] - pos[src]).norm(dim=-1)
        w = self.filter(self.rbf(d)) * (0.5 * (torch.cos(math.pi * d / self.cutoff) + 1) * (d < self.cutoff))[:, None]
        return h + self.lin2(scatter_add(self.lin1(h)[src] * w, dst, h.shape[0]))


def radius_graph(pos: torch.Tensor, r: float, loop: bool = False) -> torch.Tensor:
    d = torch.cdist(pos, pos)
    m = d <= r
    if not loop:
        m.fill_diagonal_(False)
    return m.nonzero().t().contiguous()


def knn_graph(pos: torch.Tensor, k: int) -> torch.Tensor:
    d = torch.cdist(pos, pos)
    d.fill_diagonal_(math.inf)
    nb = d.topk(k, largest=False).indices
    return torch.stack([nb.reshape(-1), torch.arange(len(pos)).repeat_interleave(k)])


# ================================================================================================ heterogeneous / hyper / temporal / knowledge graphs
class HeteroGraphData:
    """Node features per type and edge indices per ``(source type, relation, target type)``."""

    def __init__(self): self.x, self.edges = {}, {}
    def add_nodes(self, ntype, x): self.x[ntype] = x
    def add_edges(self, src, rel, dst, edge_index): self.edges[(src, rel, dst)] = edge_index
    def node_types(self): return sorted(self.x)
    def edge_types(self): return sorted(self.edges)
    def metapath_reachable(self, path) -> torch.Tensor:
        """Pairs (start, end) connected by following the relations of ``path`` in order."""
        cur = None
        for et in path:
            a = torch.zeros(self.x[et[0]].shape[0], self.x[et[2]].shape[0])
            a[self.edges[et][0], self.edges[et][1]] = 1
            cur = a if cur is None else (cur @ a > 0).float()
        return cur.nonzero().t()


class HeteroConv(nn.Module):
    """One linear map per relation (R-GCN style, mean-normalised per target), summed over relations plus a self loop."""

    def __init__(self, in_dims: dict, out_dim: int, edge_types):
        super().__init__()
        self.rel = nn.ModuleDict({"__".join(et): nn.Linear(in_dims[et[0]], out_dim, bias=False) for et in edge_types})
        self.self_loop = nn.ModuleDict({t: nn.Linear(d, out_dim) for t, d in in_dims.items()})

    def forward(self, g: HeteroGraphData) -> dict:
        out = {t: self.self_loop[t](x) for t, x in g.x.items()}
        for et, ei in g.edges.items():
            msg = self.rel["__".join(et)](g.x[et[0]])[ei[0]]
            n = g.x[et[2]].shape[0]
            deg = torch.bincount(ei[1], minlength=n).clamp(min=1)[:, None]
            out[et[2]] = out[et[2]] + scatter_add(msg, ei[1], n) / deg
        return {t: F.relu(v) for t, v in out.items()}


class HypergraphConv(nn.Module):
    """``X' = D_v^-1/2 H W D_e^-1 H^T D_v^-1/2 X Theta`` for an incidence list ``(node, hyperedge)``."""

    def __init__(self, cin, cout): super().__init__(); self.lin = nn.Linear(cin, cout)

    def forward(self, x, incidence: torch.Tensor, edge_weight: torch.Tensor | None = None):
        node, he = incidence
        ne = int(he.max()) + 1
        w = torch.ones(ne) if edge_weight is None else edge_weight
        dv = torch.zeros(x.shape[0]).index_add_(0, node, w[he]).clamp(min=1e-12).rsqrt()
        de = torch.bincount(he, minlength=ne).clamp(min=1).float()
        xe = scatter_add((self.lin(x) * dv[:, None])[node], he, ne) * (w / de)[:, None]
        return scatter_add(xe[he], node, x.shape[0]) * dv[:, None]


class TemporalGraphMemory(nn.Module):
    """TGN-style node memory: every interaction ``(src, dst, t, feature)`` writes a message into both endpoints' memory
    through a GRU cell with a cosine time encoding of the time since the node's last update."""

    def __init__(self, num_nodes, mem_dim, feat_dim, time_dim: int = 8):
        super().__init__()
        self.register_buffer("memory", torch.zeros(num_nodes, mem_dim)); self.register_buffer("last", torch.zeros(num_nodes))
        self.w = nn.Parameter(torch.randn(time_dim)); self.cell = nn.GRUCell(2 * mem_dim + feat_dim + time_dim, mem_dim)

    def time_encode(self, dt): return torch.cos(dt[:, None] * self.w[None])

    def update(self, src, dst, t, feat):
        for a, b in ((src, dst), (dst, src)):
            msg = torch.cat([self.memory[a], self.memory[b], feat, self.time_encode(t - self.last[a])], -1)
            new = self.cell(msg, self.memory[a])
            self.memory = self.memory.index_put((a,), new.detach())
        self.last = self.last.index_put((torch.cat([src, dst]),), torch.cat([t, t]))

    def embedding(self, nodes): return self.memory[nodes]


class KnowledgeGraphEmbedding(nn.Module):
    """``transe`` (``-||h + r - t||``), ``distmult`` (``<h, r, t>``) or ``rotate`` (rotation in the complex plane) scores with a
    margin ranking loss against corrupted tails / heads."""

    def __init__(self, n_entities, n_relations, dim: int = 32, model: str = "transe", margin: float = 1.0):
        super().__init__()
        self.ent, self.rel, self.model, self.margin, self.n = nn.Embedding(n_entities, dim), nn.Embedding(n_relations, dim if model != "rotate" else dim // 2), model, margin, n_entities
        nn.init.uniform_(self.ent.weight, -0.5, 0.5)
        nn.init.uniform_(self.rel.weight, -0.5, 0.5)

    def score(self, h, r, t):
        eh, er, et = self.ent(h), self.rel(r), self.ent(t)
        if self.model == "transe":
            return -(eh + er - et).norm(dim=-1)
        if self.model == "distmult":
            return (eh * er * et).sum(-1)
        hr, hi = eh.chunk(2, -1)
        tr, ti = et.chunk(2, -1)
        c, s = torch.cos(er * math.pi), torch.sin(er * math.pi)
        return -torch.sqrt((hr * c - hi * s - tr) ** 2 + (hr * s + hi * c - ti) ** 2 + 1e-12).sum(-1)

    def loss(self, triples: torch.Tensor, generator=None):
        h, r, t = triples.t()
        corrupt = torch.randint(0, self.n, (len(h),), generator=generator)
        head = torch.rand(len(h), generator=generator) < 0.5
        neg = self.score(torch.where(head, corrupt, h), r, torch.where(head, t, corrupt))
        return F.relu(self.margin - self.score(h, r, t) + neg).mean()

    @torch.no_grad()
    def rank_tail(self, h: int, r: int, t: int) -> int:
        s = self.score(torch.full((self.n,), h), torch.full((self.n,), r), torch.arange(self.n))
        return int((s > s[t]).sum()) + 1


# ================================================================================================ explanation
def gradient_attribution(model, x, edge_index, target_node: int, target_class: int) -> dict:
    """Saliency and gradient x input per node feature; node importance is the L1 norm over features."""
    xg = x.clone().requires_grad_(True)
    model(xg, edge_index)[target_node, target_class].backward()
    return {"saliency": xg.grad.abs(), "grad_x_input": (xg.grad * x).abs(), "node_importance": xg.grad.abs().sum(1)}


class GraphExplainer:
    """GNNExplainer-style: learns a soft mask over edges that keeps the model's prediction for one node while being
    sparse; the model must accept ``edge_weight``."""

    def __init__(self, model, epochs: int = 150, lr: float = 0.05, size_coeff: float = 0.01, entropy_coeff: float = 0.05):
        self.model, self.epochs, self.lr, self.size, self.ent = model, epochs, lr, size_coeff, entropy_coeff

    def explain_node(self, x, edge_index, node: int) -> torch.Tensor:
        with torch.no_grad():
            target = self.model(x, edge_index).argmax(-1)[node]
        mask = nn.Parameter(torch.randn(edge_index.shape[1]) * 0.1 + 1.0)
        opt = torch.optim.Adam([mask], self.lr)
        for _ in range(self.epochs):
            m = torch.sigmoid(mask)
            out = self.model(x, edge_index, edge_weight=m)
            loss = F.cross_entropy(out[node:node + 1], target[None]) + self.size * m.sum() + self.ent * (-(m * torch.log(m + 1e-12) + (1 - m) * torch.log(1 - m + 1e-12))).mean()
            opt.zero_grad(); loss.backward(); opt.step()
        return torch.sigmoid(mask).detach()


# ================================================================================================ kernels and transport
def wl_subtree_kernel(graphs, iters: int = 3) -> torch.Tensor:
    """Weisfeiler-Lehman subtree kernel: ``graphs`` is a list of ``(edge_index, labels)``; returns the Gram matrix."""
    labels = [lab.tolist() for _, lab in graphs]
    adj = []
    for (ei, lab) in graphs:
        nb = defaultdict(list)
        for s, d in ei.t().tolist():
            nb[d].append(s)
        adj.append(nb)
    feats = [Counter(l) for l in labels]
    table: dict = {}
    for it in range(iters):
        new = []
        for g, lab in enumerate(labels):
            cur = []
            for v in range(len(lab)):
                sig = (it, lab[v], tuple(sorted(lab[u] for u in adj[g][v])))
                cur.append(table.setdefault(sig, -len(table) - 1))
            new.append(cur)
            feats[g].update(cur)
        labels = new
    keys = sorted({k for f in feats for k in f}, key=str)
    m = torch.tensor([[f.get(k, 0) for k in keys] for f in feats], dtype=torch.float64)
    return m @ m.t()


def shortest_path_kernel(graphs) -> torch.Tensor:
    """Counts pairs with equal (label, label, shortest-path length) triples."""
    feats = []
    for ei, lab in graphs:
        d = floyd_warshall(ei, len(lab))
        c = Counter()
        for i in range(len(lab)):
            for j in range(i + 1, len(lab)):
                if math.isfinite(float(d[i, j])):
                    a, b = sorted((int(lab[i]), int(lab[j])))
                    c[(a, b, int(d[i, j]))] += 1
        feats.append(c)
    keys = sorted({k for f in feats for k in f})
    m = torch.tensor([[f.get(k, 0) for k in keys] for f in feats], dtype=torch.float64)
    return m @ m.t()


def sinkhorn(a: torch.Tensor, b: torch.Tensor, cost: torch.Tensor, reg: float = 0.05, iters: int = 500) -> torch.Tensor:
    """Entropic optimal transport plan between histograms ``a`` and ``b`` (log-domain updates)."""
    la, lb, f, g = torch.log(a), torch.log(b), torch.zeros_like(a), torch.zeros_like(b)
    for _ in range(iters):
        f = reg * (la - torch.logsumexp((g[None] - cost) / reg, 1))
        g = reg * (lb - torch.logsumexp((f[:, None] - cost) / reg, 0))
    return torch.exp((f[:, None] + g[None] - cost) / reg)


def gromov_wasserstein(c1: torch.Tensor, c2: torch.Tensor, p=None, q=None, reg: float = 0.01, outer: int = 30) -> tuple[torch.Tensor, float]:
    """Entropic Gromov-Wasserstein between two intra-graph distance matrices (square loss): alternates the linearised
    cost ``-2 C1 T C2^T + const`` with a Sinkhorn projection.  Returns the coupling and the discrepancy."""
    n, m = len(c1), len(c2)
    p = torch.full((n,), 1.0 / n, dtype=c1.dtype) if p is None else p
    q = torch.full((m,), 1.0 / m, dtype=c1.dtype) if q is None else q
    t = p[:, None] * q[None]
    const = (c1 ** 2 @ p)[:, None] + (c2 ** 2 @ q)[None]
    for _ in range(outer):
        t = sinkhorn(p, q, const - 2 * c1 @ t @ c2.t(), reg * float((const - 2 * c1 @ t @ c2.t()).abs().max().clamp(min=1e-12)), 200)
    gw = float(((const - 2 * c1 @ t @ c2.t()) * t).sum())
    return t, gw


def graph_edit_distance_upper(ei1, n1, ei2, n2) -> float:
    """Upper bound on the unlabeled edit distance: a node assignment from the Hungarian method on degree differences,
    improved by pairwise swaps until no swap lowers the number of mismatched edges."""
    from scipy.optimize import linear_sum_assignment
    d1, d2 = torch.bincount(ei1[0], minlength=n1).double(), torch.bincount(ei2[0], minlength=n2).double()
    n = max(n1, n2)
    d1, d2 = F.pad(d1, (0, n - n1)), F.pad(d2, (0, n - n2))
    r, c = linear_sum_assignment((d1[:, None] - d2[None]).abs().numpy())
    a1, a2 = _dense_adj(ei1, n).double(), _dense_adj(ei2, n).double()
    perm = torch.zeros(n, dtype=torch.long)
    perm[torch.as_tensor(r)] = torch.as_tensor(c)
    cost = lambda p: float((a1 - a2[p][:, p]).abs().sum()) / 2
    best, improved = cost(perm), True
    while improved:
        improved = False
        for i in range(n):
            for j in range(i + 1, n):
                q = perm.clone()
                q[i], q[j] = perm[j], perm[i]
                cq = cost(q)
                if cq < best:
                    perm, best, improved = q, cq, True
    return abs(n1 - n2) + best


# ================================================================================================ analysis
def floyd_warshall(edge_index, n, weight=None) -> torch.Tensor:
    d = torch.full((n, n), math.inf, dtype=torch.float64)
    d[edge_index[0], edge_index[1]] = 1.0 if weight is None else weight.double()
    d.fill_diagonal_(0)
    for k in range(n):
        d = torch.minimum(d, d[:, k:k + 1] + d[k:k + 1, :])
    return d


def laplacian(edge_index, n, kind: str = "sym") -> torch.Tensor:
    a = _dense_adj(edge_index, n).double()
    deg = a.sum(1)
    if kind == "combinatorial":
        return torch.diag(deg) - a
    dinv = deg.clamp(min=1e-12).rsqrt()
    if kind == "sym":
        return torch.eye(n, dtype=torch.float64) - dinv[:, None] * a * dinv[None]
    return torch.eye(n, dtype=torch.float64) - a / deg.clamp(min=1e-12)[:, None]        # random walk


def spectral_analysis(edge_index, n) -> dict:
    vals, vecs = torch.linalg.eigh(laplacian(edge_index, n, "combinatorial"))
    comps = int((vals < 1e-9).sum())
    return {"eigenvalues": vals, "algebraic_connectivity": float(vals[comps]) if comps < n else 0.0, "fiedler_vector": vecs[:, comps] if comps < n else None,
            "components": comps, "spectral_gap": float(vals[comps] - vals[comps - 1]) if comps < n else 0.0, "spectral_radius": float(vals[-1])}


def graph_fourier_transform(x, edge_index, n): _, u = torch.linalg.eigh(laplacian(edge_index, n, "sym")); return u.t() @ x.double(), u


def centrality(edge_index, n) -> dict:
    """Degree, closeness, betweenness (Brandes, unweighted) and eigenvector centralities."""
    nb = defaultdict(list)
    for s, d in edge_index.t().tolist():
        nb[s].append(d)
    deg = torch.bincount(edge_index[0], minlength=n).double() / max(n - 1, 1)
    dist = floyd_warshall(edge_index, n)
    reach = torch.isfinite(dist) & (dist > 0)
    close = torch.where(reach.sum(1) > 0, reach.sum(1).double() ** 2 / ((n - 1) * torch.where(reach, dist, torch.zeros_like(dist)).sum(1)).clamp(min=1e-12), torch.zeros(n, dtype=torch.float64))
    btw = [0.0] * n
    for s in range(n):
        stack, pred, sigma, dd = [], defaultdict(list), [0.0] * n, [-1] * n
        sigma[s], dd[s], q = 1.0, 0, deque([s])
        while q:
            v = q.popleft(); stack.append(v)
            for w in nb[v]:
                if dd[w] < 0:
                    dd[w] = dd[v] + 1; q.append(w)
                if dd[w] == dd[v] + 1:
                    sigma[w] += sigma[v]; pred[w].append(v)
        delta = [0.0] * n
        while stack:
            w = stack.pop()
            for v in pred[w]:
                delta[v] += sigma[v] / sigma[w] * (1 + delta[w])
            if w != s:
                btw[w] += delta[w]
    a = _dense_adj(edge_index, n).double()
    ev = torch.ones(n, dtype=torch.float64)
    for _ in range(200):
        ev = a.t() @ ev + ev * 1e-9
        ev = ev / ev.norm().clamp(min=1e-300)
    return {"degree": deg, "closeness": close, "betweenness": torch.tensor(btw, dtype=torch.float64) / 2, "eigenvector": ev}


def spectral_partition(edge_index, n, parts: int = 2) -> torch.Tensor:
    """Recursive bisection by the sign of the Fiedler vector (median split for balance)."""
    lab = torch.zeros(n, dtype=torch.long)
    groups, nxt = [torch.arange(n)], 1
    while len(groups) < parts:
        g = max(groups, key=len)
        groups.remove(g)
        relabel = torch.full((n,), -1, dtype=torch.long); relabel[g] = torch.arange(len(g))
        m = (relabel[edge_index[0]] >= 0) & (relabel[edge_index[1]] >= 0)
        f = spectral_analysis(relabel[edge_index[:, m]], len(g))["fiedler_vector"]
        f = f if f is not None else torch.arange(len(g), dtype=torch.float64)
        right = f > f.median()
        groups += [g[~right], g[right]]
        lab[g[right]] = nxt
        nxt += 1
    return lab


def edge_cut(edge_index, labels) -> int: return int((labels[edge_index[0]] != labels[edge_index[1]]).sum()) // 2


# ================================================================================================ heads / autoencoder / loaders
class GraphClassifier(nn.Module):
    def __init__(self, cin, hidden, classes, layers: int = 2, readout: str = "mean"):
        super().__init__()
        self.convs = nn.ModuleList(GCNConv(cin if i == 0 else hidden, hidden) for i in range(layers))
        self.head, self.readout = nn.Linear(hidden, classes), readout

    def forward(self, x, edge_index, batch=None):
        batch = torch.zeros(x.shape[0], dtype=torch.long) if batch is None else batch
        for c in self.convs:
            x = F.relu(c(x, edge_index))
        nb = int(batch.max()) + 1
        pooled = torch.zeros(nb, x.shape[1]).index_add_(0, batch, x)
        if self.readout == "mean":
            pooled = pooled / torch.bincount(batch, minlength=nb).clamp(min=1)[:, None]
        return self.head(pooled)


class GraphAutoEncoder(nn.Module):
    """GCN encoder with an inner-product decoder; ``variational`` adds the reparameterised latent and a KL term."""

    def __init__(self, cin, hidden, latent, variational: bool = False):
        super().__init__()
        self.c1, self.mu, self.variational = GCNConv(cin, hidden), GCNConv(hidden, latent), variational
        self.logvar = GCNConv(hidden, latent) if variational else None

    def encode(self, x, edge_index):
        h = F.relu(self.c1(x, edge_index))
        mu = self.mu(h, edge_index)
        if not self.variational:
            return mu
        self._mu, self._lv = mu, self.logvar(h, edge_index).clamp(max=10)
        return mu + torch.randn_like(mu) * torch.exp(0.5 * self._lv) if self.training else mu

    def loss(self, x, pos_edges, neg_edges):
        z = self.encode(x, pos_edges)
        s = lambda e: (z[e[0]] * z[e[1]]).sum(-1)
        rec = F.binary_cross_entropy_with_logits(torch.cat([s(pos_edges), s(neg_edges)]), torch.cat([torch.ones(pos_edges.shape[1]), torch.zeros(neg_edges.shape[1])]))
        return rec + (-0.5 / len(x) * (1 + self._lv - self._mu ** 2 - self._lv.exp()).sum(1).mean() if self.variational else 0.0)


def batch_graphs(graphs: list[GraphData]):
    """Disjoint union: concatenated features, offset edge indices, and the graph id of every node."""
    xs, es, bs, off = [], [], [], 0
    for i, g in enumerate(graphs):
        xs.append(g.x); es.append(g.edge_index + off); bs.append(torch.full((g.x.shape[0],), i, dtype=torch.long))
        off += g.x.shape[0]
    ys = [g.y for g in graphs if g.y is not None]
    return torch.cat(xs), torch.cat(es, 1), torch.cat(bs), (torch.stack(ys) if ys and ys[0].dim() == 0 else (torch.cat(ys) if ys else None))


def load_edge_list(path, directed: bool = False, delimiter=None):
    """``u v [weight]`` per line (``#`` comments); node names are mapped to consecutive ids.  Returns
    ``(edge_index, weights or None, names)``."""
    ids, edges, ws = {}, [], []
    for ln in open(path):
        ln = ln.split("#")[0].strip()
        if not ln:
            continue
        p = ln.split(delimiter)
        u, v = (ids.setdefault(k, len(ids)) for k in p[:2])
        edges.append((u, v)); ws.append(float(p[2]) if len(p) > 2 else None)
    e = torch.tensor(edges, dtype=torch.long).t()
    w = torch.tensor(ws) if all(x is not None for x in ws) and ws else None
    if not directed:
        e, w = torch.cat([e, e.flip(0)], 1), (torch.cat([w, w]) if w is not None else None)
    return e, w, list(ids)


def load_gml(path):
    """Nodes (``id``, ``label``, numeric ``value``) and edges of a GML file."""
    text = open(path).read()
    nodes = [dict(re.findall(r'(\w+)\s+("[^"]*"|[-\w.]+)', blk)) for blk in re.findall(r"node\s*\[(.*?)\]", text, re.S)]
    edges = [dict(re.findall(r"(\w+)\s+([-\w.]+)", blk)) for blk in re.findall(r"edge\s*\[(.*?)\]", text, re.S)]
    idx = {n["id"]: i for i, n in enumerate(nodes)}
    e = torch.tensor([(idx[d["source"]], idx[d["target"]]) for d in edges], dtype=torch.long).t()
    directed = re.search(r"directed\s+1", text) is not None
    return (e if directed else torch.cat([e, e.flip(0)], 1)), [n.get("label", n["id"]).strip('"') for n in nodes], [float(n["value"]) if "value" in n else None for n in nodes]


def load_json_graph(path) -> GraphData:
    """Node-link JSON: ``{"nodes": [{"id", "features", "label"}], "links": [{"source", "target"}]}``."""
    d = json.loads(open(path).read())
    idx = {n["id"]: i for i, n in enumerate(d["nodes"])}
    e = torch.tensor([(idx[l["source"]], idx[l["target"]]) for l in d["links"]], dtype=torch.long).t()
    if not d.get("directed", False):
        e = torch.cat([e, e.flip(0)], 1)
    x = torch.tensor([n.get("features", [1.0]) for n in d["nodes"]], dtype=torch.float32)
    y = torch.tensor([n["label"] for n in d["nodes"]]) if all("label" in n for n in d["nodes"]) else None
    return GraphData(x, e, None, y)
