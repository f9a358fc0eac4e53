"""Graph neural networks (``crates/torsh-graph``): graph container, message passing with a scatter-add aggregation,
GCN / GraphSAGE / GAT / GIN layers, global pooling, and small synthetic datasets.

The reference's generated CUDA string for message passing (``crates/torsh-graph/src/jit.rs:405-450``) adds into the
output without atomics; here aggregation is ``ops.scatter_add`` (atomic fp32 adds, one thread per 16-byte feature chunk
on the GPU; ``index_add_`` on the CPU).  Layers whose message is the
neighbour's feature row times an edge weight (GCN, SAGE, GIN) call the fused gather-scale-scatter kernel and never
materialise the per-edge messages."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


def scatter_add(src: torch.Tensor, index: torch.Tensor, n: int) -> torch.Tensor:
    """``out[index[e]] += src[e]`` with ``out`` of ``n`` rows."""
    if src.dim() == 2:
        from .ops.elementwise import gnn_scatter
        return gnn_scatter(src, index, n)
    return torch.zeros(n, *src.shape[1:], dtype=src.dtype, device=src.device).index_add_(0, index, src)


@dataclass
class GraphData:
    x: torch.Tensor                      # [N, F]
    edge_index: torch.Tensor             # [2, E] (source, target)
    edge_attr: torch.Tensor | None = None
    y: torch.Tensor | None = None
    batch: torch.Tensor | None = None    # node → graph id

    @property
    def num_nodes(self): return self.x.shape[0]
    @property
    def num_edges(self): return self.edge_index.shape[1]

    def add_self_loops(self) -> "GraphData":
        loops = torch.arange(self.num_nodes, device=self.x.device).repeat(2, 1)
        return GraphData(self.x, torch.cat([self.edge_index, loops], 1), None, self.y, self.batch)

    def degree(self) -> torch.Tensor:
        return torch.bincount(self.edge_index[1], minlength=self.num_nodes).to(self.x.dtype)

    def to(self, device):
        mv = lambda t: None if t is None else t.to(device)
        return GraphData(mv(self.x), mv(self.edge_index), mv(self.edge_attr), mv(self.y), mv(self.batch))

    @staticmethod
    def collate(graphs: list["GraphData"]) -> "GraphData":
        off, xs, es, bs, ys = 0, [], [], [], []
        for i, g in enumerate(graphs):
            xs.append(g.x); es.append(g.edge_index + off)
            bs.append(torch.full((g.num_nodes,), i, dtype=torch.long))
            if g.y is not None: ys.append(g.y.reshape(-1))
            off += g.num_nodes
        return GraphData(torch.cat(xs), torch.cat(es, 1), None, torch.cat(ys) if ys else None, torch.cat(bs))


class MessagePassing(nn.Module):
    aggr = "sum"

    def message(self, x_j, x_i, edge_attr): return x_j
    def update(self, agg, x): return agg

    def propagate(self, x, edge_index, edge_attr=None, edge_weight=None):
        src, dst = edge_index
        n = x.shape[0]
        if type(self).message is MessagePassing.message and x.dim() == 2:
            from .ops.elementwise import gnn_scatter
            out = gnn_scatter(x, dst, n, src=src, weight=edge_weight)
        else:
            m = self.message(x[src], x[dst], edge_attr)
            if edge_weight is not None:
                m = m * edge_weight[:, None]
            out = scatter_add(m, dst, n)
        if self.aggr == "mean":
            out = out / torch.bincount(dst, minlength=n).clamp(min=1).to(out.dtype)[:, None]
        return self.update(out, x)


class GCNConv(MessagePassing):
    def __init__(self, in_f, out_f, bias=True):
        super().__init__()
        self.lin = nn.Linear(in_f, out_f, bias=False)
        self.bias = nn.Parameter(torch.zeros(out_f)) if bias else None

    def forward(self, x, edge_index):
        n = x.shape[0]
        loops = torch.arange(n, device=x.device).repeat(2, 1)
        ei = torch.cat([edge_index, loops], 1)
        deg = torch.bincount(ei[1], minlength=n).to(x.dtype)
        w = deg[ei[0]].rsqrt() * deg[ei[1]].rsqrt()
        out = self.propagate(self.lin(x), ei, edge_weight=w)
        return out if self.bias is None else out + self.bias


class SAGEConv(MessagePassing):
    aggr = "mean"

    def __init__(self, in_f, out_f):
        super().__init__()
        self.lin_self, self.lin_nb = nn.Linear(in_f, out_f), nn.Linear(in_f, out_f, bias=False)

    def forward(self, x, edge_index):
        return self.lin_self(x) + self.lin_nb(self.propagate(x, edge_index))


class GINConv(MessagePassing):
    def __init__(self, mlp: nn.Module, eps: float = 0.0, train_eps=False):
        super().__init__()
        self.mlp = mlp
        self.eps = nn.Parameter(torch.tensor(eps)) if train_eps else eps

    def forward(self, x, edge_index):
        return self.mlp((1 + self.eps) * x + self.propagate(x, edge_index))


class GATConv(nn.Module):
    def __init__(self, in_f, out_f, heads=1, negative_slope=0.2, concat=True):
        super().__init__()
        self.h, self.o, self.slope, self.concat = heads, out_f, negative_slope, concat
        self.lin = nn.Linear(in_f, heads * out_f, bias=False)
        self.att_src = nn.Parameter(torch.randn(heads, out_f) * 0.1)
        self.att_dst = nn.Parameter(torch.randn(heads, out_f) * 0.1)
        self.bias = nn.Parameter(torch.zeros(heads * out_f if concat else out_f))

    def forward(self, x, edge_index):
        n = x.shape[0]
        loops = torch.arange(n, device=x.device).repeat(2, 1)
        src, dst = torch.cat([edge_index, loops], 1)
        h = self.lin(x).view(n, self.h, self.o)
        e = F.leaky_relu((h * self.att_src).sum(-1)[src] + (h * self.att_dst).sum(-1)[dst], self.slope)
        emax = torch.full((n, self.h), -1e30, dtype=e.dtype, device=e.device).scatter_reduce(0, dst[:, None].expand_as(e), e, "amax")
        p = (e - emax[dst]).exp()
        alpha = p / scatter_add(p, dst, n)[dst]
        out = scatter_add((h[src] * alpha[..., None]).reshape(-1, self.h * self.o), dst, n).view(n, self.h, self.o)
        return (out.reshape(n, -1) if self.concat else out.mean(1)) + self.bias


def global_add_pool(x, batch, n=None): return scatter_add(x, batch, n or int(batch.max()) + 1)
def global_mean_pool(x, batch, n=None):
    n = n or int(batch.max()) + 1
    return scatter_add(x, batch, n) / torch.bincount(batch, minlength=n).clamp(min=1).to(x.dtype)[:, None]
def global_max_pool(x, batch, n=None):
    n = n or int(batch.max()) + 1
    return torch.full((n, x.shape[1]), -torch.inf, dtype=x.dtype, device=x.device).scatter_reduce(0, batch[:, None].expand_as(x), x, "amax")


class GCN(nn.Module):
    def __init__(self, in_f, hidden, classes, layers=2, dropout=0.5):
        super().__init__()
        dims = [in_f] + [hidden] * (layers - 1) + [classes]
        self.convs = nn.ModuleList(GCNConv(a, b) for a, b in zip(dims[:-1], dims[1:]))
        self.dropout = dropout

    def forward(self, x, edge_index):
        for i, c in enumerate(self.convs):
            x = c(x, edge_index)
            if i + 1 < len(self.convs):
                x = F.dropout(F.relu(x), self.dropout, self.training)
        return x


def stochastic_block_model(sizes=(40, 40), p_in=0.3, p_out=0.02, feat=16, seed=0) -> GraphData:
    g = torch.Generator().manual_seed(seed)
    lab = torch.cat([torch.full((s,), i) for i, s in enumerate(sizes)])
    p = torch.where(lab[:, None] == lab[None], p_in, p_out)
    adj = torch.rand(p.shape, generator=g) < p
    adj = (adj | adj.t()) & ~torch.eye(len(lab), dtype=torch.bool)
    x = torch.randn(len(lab), feat, generator=g) + lab[:, None].float()
    return GraphData(x, adj.nonzero().t().contiguous(), y=lab)


# ---- further layers, sampling, generators, metrics and link prediction (crates/torsh-graph/src/{conv,sampling,generators,
#      metrics,link_prediction,transformer}.rs) --------------------------------------------------------------------------
class ChebConv(nn.Module):
    """Spectral convolution with Chebyshev polynomials of the scaled Laplacian up to order K (Defferrard et al.)."""

    def __init__(self, cin: int, cout: int, K: int = 3):
        super().__init__()
        self.lins = nn.ModuleList(nn.Linear(cin, cout, bias=False) for _ in range(K))
        self.bias = nn.Parameter(torch.zeros(cout))

    def forward(self, x, edge_index):
        n = x.shape[0]
        src, dst = edge_index
        deg = torch.bincount(dst, minlength=n).to(x.dtype).clamp(min=1)
        w = -(deg[src] * deg[dst]).rsqrt()                                   # L~ = L - I = -D^-1/2 A D^-1/2 (lambda_max = 2)
        prop = lambda h: scatter_add(h[src] * w[:, None], dst, n)
        t0, out = x, self.lins[0](x)
        if len(self.lins) > 1:
            t1 = prop(x)
            out = out + self.lins[1](t1)
            for lin in self.lins[2:]:
                t0, t1 = t1, 2 * prop(t1) - t0
                out = out + lin(t1)
        return out + self.bias


class GraphTransformerLayer(nn.Module):
    """Multi-head attention restricted to graph edges (softmax over each node's incoming edges), residual + norm + MLP."""

    def __init__(self, dim: int, heads: int = 4, mlp_ratio: float = 2.0):
        super().__init__()
        self.h, self.dh = heads, dim // heads
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim) for _ in range(4))
        self.n1, self.n2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.mlp = nn.Sequential(nn.Linear(dim, int(dim * mlp_ratio)), nn.GELU(), nn.Linear(int(dim * mlp_ratio), dim))

    def forward(self, x, edge_index):
        n = x.shape[0]
        src, dst = edge_index
        h = self.n1(x)
        q, k, v = (f(h).reshape(n, self.h, self.dh) for f in (self.q, self.k, self.v))
        score = (q[dst] * k[src]).sum(-1) / self.dh ** 0.5                    # [E, heads]
        mx = torch.full((n, self.h), float("-inf"), dtype=score.dtype, device=x.device).scatter_reduce(0, dst[:, None].expand_as(score), score, "amax")
        e = torch.exp(score - mx[dst])
        den = torch.zeros(n, self.h, dtype=e.dtype, device=x.device).index_add_(0, dst, e)
        a = e / den[dst].clamp(min=1e-30)
        agg = torch.zeros(n, self.h, self.dh, dtype=x.dtype, device=x.device).index_add_(0, dst, a[..., None] * v[src])
        x = x + self.o(agg.reshape(n, -1))
        return x + self.mlp(self.n2(x))


class NeighborSampler:
    """Samples, for a batch of seed nodes, up to ``fanout[l]`` incoming neighbours per node and layer (GraphSAGE style).
    Returns the node ids involved (seeds first) and one relabelled edge index per layer, outermost layer first."""

    def __init__(self, edge_index: torch.Tensor, num_nodes: int, fanouts, seed: int = 0):
        src, dst = edge_index
        order = torch.argsort(dst, stable=True)
        self.src = src[order]
        self.ptr = torch.zeros(num_nodes + 1, dtype=torch.long)
        self.ptr[1:] = torch.bincount(dst, minlength=num_nodes).cumsum(0)
        self.fanouts, self.gen = list(fanouts), torch.Generator().manual_seed(seed)

    def sample(self, seeds: torch.Tensor):
        nodes = seeds.tolist()
        index = {v: i for i, v in enumerate(nodes)}
        frontier, layers = list(nodes), []
        for fan in reversed(self.fanouts):
            es, ed, nxt = [], [], []
            for v in frontier:
                nb = self.src[self.ptr[v]:self.ptr[v + 1]]
                if len(nb) > fan:
                    nb = nb[torch.randperm(len(nb), generator=self.gen)[:fan]]
                for u in nb.tolist():
                    if u not in index:
                        index[u] = len(nodes)
                        nodes.append(u)
                        nxt.append(u)
                    es.append(index[u])
                    ed.append(index[v])
            layers.append(torch.tensor([es, ed], dtype=torch.long))
            frontier = frontier + nxt
        return torch.tensor(nodes), layers[::-1]


def erdos_renyi(n: int, p: float, seed: int = 0, directed: bool = False) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    m = torch.rand(n, n, generator=g) < p
    m = m.triu(1) if not directed else m & ~torch.eye(n, dtype=torch.bool)
    e = m.nonzero().t()
    return e if directed else torch.cat([e, e.flip(0)], 1)


def barabasi_albert(n: int, m: int, seed: int = 0) -> torch.Tensor:
    """Preferential attachment: every new node links to ``m`` existing nodes chosen in proportion to their degree."""
    g = torch.Generator().manual_seed(seed)
    edges, targets = [], list(range(m))
    repeated: list[int] = []
    for v in range(m, n):
        for t in set(targets):
            edges.append((v, t))
        repeated += list(set(targets)) + [v] * len(set(targets))
        pick = torch.randint(0, len(repeated), (m * 3,), generator=g).tolist()
        targets = []
        for i in pick:
            if repeated[i] not in targets:
                targets.append(repeated[i])
            if len(targets) == m:
                break
    e = torch.tensor(edges, dtype=torch.long).t()
    return torch.cat([e, e.flip(0)], 1)


def grid_graph(h: int, w: int) -> torch.Tensor:
    idx = torch.arange(h * w).reshape(h, w)
    e = torch.cat([torch.stack([idx[:, :-1].flatten(), idx[:, 1:].flatten()]), torch.stack([idx[:-1].flatten(), idx[1:].flatten()])], 1)
    return torch.cat([e, e.flip(0)], 1)


def modularity(edge_index: torch.Tensor, labels: torch.Tensor) -> float:
    """Newman modularity of a partition of an undirected graph given with both edge directions."""
    src, dst = edge_index
    m2 = float(edge_index.shape[1])
    deg = torch.bincount(src, minlength=labels.numel()).double()
    inside = float((labels[src] == labels[dst]).sum()) / m2
    k = torch.zeros(int(labels.max()) + 1, dtype=torch.float64).index_add_(0, labels, deg)
    return inside - float(((k / m2) ** 2).sum())


def clustering_coefficient(edge_index: torch.Tensor, n: int) -> torch.Tensor:
    a = torch.zeros(n, n)
    a[edge_index[0], edge_index[1]] = 1
    tri = (a @ a * a).sum(1) / 2
    deg = a.sum(1)
    return torch.where(deg > 1, 2 * tri / (deg * (deg - 1)).clamp(min=1), torch.zeros(n))


def connected_components(edge_index: torch.Tensor, n: int) -> torch.Tensor:
    """Component label per node by label propagation (min label over neighbours until nothing changes)."""
    lab = torch.arange(n)
    src, dst = edge_index
    while True:
        new = lab.clone().scatter_reduce(0, dst, lab[src], "amin")
        new = new.scatter_reduce(0, src, new[dst], "amin")
        if torch.equal(new, lab):
            _, inv = torch.unique(lab, return_inverse=True)
            return inv
        lab = new


def pagerank(edge_index: torch.Tensor, n: int, damping: float = 0.85, iters: int = 100, tol: float = 1e-10) -> torch.Tensor:
    src, dst = edge_index
    out_deg = torch.bincount(src, minlength=n).double()
    r = torch.full((n,), 1.0 / n, dtype=torch.float64)
    for _ in range(iters):
        contrib = r / out_deg.clamp(min=1)
        new = torch.zeros(n, dtype=torch.float64).index_add_(0, dst, contrib[src])
        new = damping * (new + r[out_deg == 0].sum() / n) + (1 - damping) / n
        if (new - r).abs().sum() < tol:
            return new
        r = new
    return r


def negative_sampling(edge_index: torch.Tensor, n: int, num: int, seed: int = 0) -> torch.Tensor:
    """``num`` node pairs that are not edges (and not self loops)."""
    g = torch.Generator().manual_seed(seed)
    have = set((edge_index[0] * n + edge_index[1]).tolist())
    out = []
    while len(out) < num:
        c = torch.randint(0, n, (2, 2 * num), generator=g)
        for u, v in c.t().tolist():
            if u != v and u * n + v not in have:
                have.add(u * n + v)
                out.append((u, v))
                if len(out) == num:
                    break
    return torch.tensor(out).t()


def link_prediction_loss(z: torch.Tensor, pos_edges: torch.Tensor, neg_edges: torch.Tensor) -> torch.Tensor:
    """Binary cross entropy of inner-product edge scores for positive and sampled negative pairs."""
    score = lambda e: (z[e[0]] * z[e[1]]).sum(-1)
    return F.binary_cross_entropy_with_logits(torch.cat([score(pos_edges), score(neg_edges)]),
                                              torch.cat([torch.ones(pos_edges.shape[1]), torch.zeros(neg_edges.shape[1])]).to(z))


def load_planetoid_like(content_path, cites_path) -> GraphData:
    """Cora / CiteSeer in their original text form: ``<id> <features...> <label>`` per line and ``<cited> <citing>`` per line."""
    ids, feats, labels = [], [], []
    for ln in open(content_path):
        p = ln.split()
        ids.append(p[0]); feats.append([float(v) for v in p[1:-1]]); labels.append(p[-1])
    idx = {v: i for i, v in enumerate(ids)}
    classes = {c: i for i, c in enumerate(sorted(set(labels)))}
    edges = [(idx[a], idx[b]) for a, b in (ln.split() for ln in open(cites_path)) if a in idx and b in idx]
    e = torch.tensor(edges, dtype=torch.long).t()
    return GraphData(torch.tensor(feats), torch.cat([e, e.flip(0)], 1), None, torch.tensor([classes[c] for c in labels]))
