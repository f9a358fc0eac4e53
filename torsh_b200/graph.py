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
