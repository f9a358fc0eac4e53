"""Graph learning beyond static message passing (``crates/torsh-graph/src``): continuous-time dynamic graphs — functional time
encoding, temporal attention over recent neighbours, an event-stream model with node memory, and graph ODEs
(``continuous_time.rs``); sparse winning tickets for graph networks — joint masks on weights and edges with iterative
pruning and rewinding (``lottery_ticket.rs``); self-supervised pre-training — augmentations, contrastive and masked
objectives, prompt tuning on a frozen encoder (``foundation.rs``)."""
from __future__ import annotations

import copy
import math
from collections import defaultdict, deque
from typing import Callable, Sequence

import torch
from torch import nn

from .graph import GCNConv, global_mean_pool, scatter_add


# ================================================================================================ continuous-time dynamic graphs
class TimeEncoder(nn.Module):
    """``phi(t) = cos(t w + b)`` with frequencies initialised on a geometric grid: inner products of encodings depend on time
    differences, which is what attention over events needs."""

    def __init__(self, dim: int = 16, max_period: float = 1e4):
        super().__init__()
        self.w = nn.Parameter(1.0 / max_period ** torch.linspace(0, 1, dim)); self.b = nn.Parameter(torch.zeros(dim))
    def forward(self, t: torch.Tensor) -> torch.Tensor: return torch.cos(t.unsqueeze(-1) * self.w + self.b)


class TemporalNeighborStore:
    """Most recent ``k`` interactions per node (neighbour, time, edge feature index), updated as events arrive."""

    def __init__(self, k: int = 10): self.k, self.adj = k, defaultdict(lambda: deque(maxlen=k))
    def insert(self, src: int, dst: int, t: float, eid: int): self.adj[src].append((dst, t, eid)); self.adj[dst].append((src, t, eid))
    def recent(self, node: int, before: float) -> list[tuple[int, float, int]]: return [e for e in self.adj[node] if e[1] < before]
    def reset(self): self.adj.clear()


class TemporalAttentionLayer(nn.Module):
    """A node's embedding at time ``t`` attends over its recent neighbours; keys and values carry the neighbour's state, the
    edge feature and the encoding of the elapsed time."""

    def __init__(self, node_dim: int, edge_dim: int, time_dim: int, out_dim: int, heads: int = 2):
        super().__init__()
        self.time = TimeEncoder(time_dim)
        self.q, self.kv = nn.Linear(node_dim + time_dim, out_dim), nn.Linear(node_dim + edge_dim + time_dim, 2 * out_dim)
        self.heads, self.out = heads, nn.Sequential(nn.Linear(out_dim + node_dim, out_dim), nn.ReLU(), nn.Linear(out_dim, out_dim))

    def forward(self, h_self, h_nb, e_nb, dt, mask):
        """``h_self [B, D]``, ``h_nb [B, K, D]``, ``e_nb [B, K, E]``, ``dt [B, K]`` elapsed time, ``mask [B, K]`` true for real neighbours."""
        B, K, _ = h_nb.shape
        q = self.q(torch.cat([h_self, self.time(torch.zeros(B, device=h_self.device))], -1)).view(B, self.heads, 1, -1)
        k, v = self.kv(torch.cat([h_nb, e_nb, self.time(dt)], -1)).chunk(2, -1)
        k, v = k.view(B, K, self.heads, -1).transpose(1, 2), v.view(B, K, self.heads, -1).transpose(1, 2)
        att = (q @ k.transpose(-1, -2)) / math.sqrt(k.shape[-1])
        att = att.masked_fill(~mask[:, None, None, :], -1e9).softmax(-1) * mask[:, None, None, :].any(-1, keepdim=True)
        agg = (att @ v).transpose(1, 2).reshape(B, -1)
        return self.out(torch.cat([agg, h_self], -1))


class ContinuousTimeGraphNetwork(nn.Module):
    """Event-stream model: every node keeps a memory updated by a GRU from the messages of its interactions (the memories
    of both endpoints, the edge feature and the time since the node's last update); embeddings come from temporal attention
    over the stored recent neighbours; a link decoder scores candidate interactions.  Events must be fed in time order."""

    def __init__(self, num_nodes: int, edge_dim: int, memory_dim: int = 32, time_dim: int = 16, embed_dim: int = 32, neighbors: int = 10):
        super().__init__()
        self.n, self.md, self.ed = num_nodes, memory_dim, edge_dim
        self.time = TimeEncoder(time_dim)
        self.node_emb = nn.Embedding(num_nodes, memory_dim)                         # static node features: the memory alone cannot tell untouched nodes apart
        self.gru = nn.GRUCell(2 * memory_dim + edge_dim + time_dim, memory_dim)
        self.attn = TemporalAttentionLayer(memory_dim, edge_dim, time_dim, embed_dim)
        self.decoder = nn.Sequential(nn.Linear(2 * embed_dim, embed_dim), nn.ReLU(), nn.Linear(embed_dim, 1))
        self.store = TemporalNeighborStore(neighbors)
        self.reset_state()

    def reset_state(self):
        self.memory = torch.zeros(self.n, self.md); self.last_update = torch.zeros(self.n); self.edge_feats: list[torch.Tensor] = []; self.store.reset()

    def detach_state(self): self.memory = self.memory.detach()
    def _state(self, nodes): return self.memory[nodes] + self.node_emb(nodes)

    def embed(self, nodes: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        K = self.store.k
        nb, dt, ef, mask = torch.zeros(len(nodes), K, dtype=torch.long), torch.zeros(len(nodes), K), torch.zeros(len(nodes), K, self.ed), torch.zeros(len(nodes), K, dtype=torch.bool)
        for i, (v, tv) in enumerate(zip(nodes.tolist(), t.tolist())):
            for j, (u, tu, eid) in enumerate(self.store.recent(v, tv)):
                nb[i, j], dt[i, j], ef[i, j], mask[i, j] = u, tv - tu, self.edge_feats[eid], True
        return self.attn(self._state(nodes), self._state(nb), ef, dt, mask)

    def score(self, src: torch.Tensor, dst: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        return self.decoder(torch.cat([self.embed(src, t), self.embed(dst, t)], -1)).squeeze(-1)

    def update(self, src: torch.Tensor, dst: torch.Tensor, t: torch.Tensor, feat: torch.Tensor):
        """Consumes a batch of events (after they have been scored): memory update for both endpoints, neighbour lists."""
        for a, b in ((src, dst), (dst, src)):
            msg = torch.cat([self._state(a), self._state(b), feat, self.time(t - self.last_update[a])], -1)
            new = self.gru(msg, self.memory[a])
            self.memory = self.memory.index_put((a,), new)                          # later events of the same node in the batch win
        self.last_update = self.last_update.index_put((torch.cat([src, dst]),), torch.cat([t, t]))
        for s, d, tt, f in zip(src.tolist(), dst.tolist(), t.tolist(), feat):
            self.edge_feats.append(f.detach()); self.store.insert(s, d, tt, len(self.edge_feats) - 1)


class GraphODE(nn.Module):
    """``dH/dt = f(H, A)`` integrated with fixed-step Runge-Kutta 4.  ``mode="heat"`` is linear diffusion ``-L H`` (no parameters,
    exact solution ``exp(-tL) H``); ``mode="gcn"`` uses a learned graph convolution as the vector field (a continuous-depth
    network whose depth is the integration time)."""

    def __init__(self, dim: int | None = None, mode: str = "heat", steps: int = 20):
        super().__init__()
        self.mode, self.steps = mode, steps
        if mode == "gcn":
            self.conv, self.gate = GCNConv(dim, dim), nn.Parameter(torch.tensor(0.0))

    @staticmethod
    def laplacian(edge_index, n):
        A = torch.zeros(n, n); A[edge_index[0], edge_index[1]] = 1.0; A = ((A + A.T) > 0).float()
        d = A.sum(1)
        dis = d.clamp_min(1e-12).rsqrt() * (d > 0)
        return torch.eye(n) - dis[:, None] * A * dis[None]

    def forward(self, h: torch.Tensor, edge_index: torch.Tensor, t: float = 1.0) -> torch.Tensor:
        L = self.laplacian(edge_index, h.shape[0]).to(h.dtype) if self.mode == "heat" else None
        f = (lambda x: -L @ x) if self.mode == "heat" else (lambda x: torch.sigmoid(self.gate) * torch.tanh(self.conv(x, edge_index)) - x * 0.1)
        dt = t / self.steps
        for _ in range(self.steps):
            k1 = f(h); k2 = f(h + 0.5 * dt * k1); k3 = f(h + 0.5 * dt * k2); k4 = f(h + dt * k3)
            h = h + dt / 6 * (k1 + 2 * k2 + 2 * k3 + k4)
        return h


# ================================================================================================ lottery tickets
class GraphLotteryTicket:
    """Iterative magnitude pruning for graph networks: each round trains the model (the caller's ``train`` function, which
    receives the model and the current edge mask), removes the smallest ``weight_rate`` of the surviving weights and the
    ``edge_rate`` least important surviving edges (importance = learned edge score when the model exposes ``edge_scores()``,
    else the product of endpoint embedding norms), rewinds the remaining weights to their initial values and repeats.  The
    result is a sparse sub-network and a sparse graph that train to the original accuracy from the original initialisation."""

    def __init__(self, model: nn.Module, edge_index: torch.Tensor, weight_rate: float = 0.2, edge_rate: float = 0.05):
        self.model, self.edge_index, self.wr, self.er = model, edge_index, weight_rate, edge_rate
        self.init_state = copy.deepcopy(model.state_dict())
        self.masks = {n: torch.ones_like(p, dtype=torch.bool) for n, p in model.named_parameters() if p.dim() >= 2}
        self.edge_mask = torch.ones(edge_index.shape[1], dtype=torch.bool)
        self.history = []

    def apply_masks(self):
        with torch.no_grad():
            for n, p in self.model.named_parameters():
                if n in self.masks:
                    p.mul_(self.masks[n])

    def masked_edges(self) -> torch.Tensor: return self.edge_index[:, self.edge_mask]
    def weight_sparsity(self) -> float: return 1 - sum(int(m.sum()) for m in self.masks.values()) / sum(m.numel() for m in self.masks.values())
    def edge_sparsity(self) -> float: return 1 - float(self.edge_mask.float().mean())

    def _prune_weights(self):
        alive = torch.cat([p.detach().abs()[self.masks[n]] for n, p in self.model.named_parameters() if n in self.masks])
        k = int(self.wr * alive.numel())
        if k:
            th = alive.kthvalue(k).values
            for n, p in self.model.named_parameters():
                if n in self.masks:
                    self.masks[n] &= p.detach().abs() > th

    def _prune_edges(self, importance: torch.Tensor):
        alive = self.edge_mask.nonzero().flatten()
        k = int(self.er * len(alive))
        if k:
            drop = alive[importance[alive].argsort()[:k]]
            self.edge_mask[drop] = False

    def round(self, train: Callable[[nn.Module, torch.Tensor, Callable[[], None]], float], edge_importance: Callable[[nn.Module, torch.Tensor], torch.Tensor] | None = None) -> dict:
        self.apply_masks()
        score = train(self.model, self.masked_edges(), self.apply_masks)
        self._prune_weights()
        if self.er:
            imp = edge_importance(self.model, self.edge_index) if edge_importance else torch.rand(self.edge_index.shape[1])
            self._prune_edges(imp)
        self.model.load_state_dict(self.init_state)                                 # rewind the survivors to their initial values
        self.apply_masks()
        rec = {"score": score, "weight_sparsity": self.weight_sparsity(), "edge_sparsity": self.edge_sparsity()}
        self.history.append(rec)
        return rec


# ================================================================================================ self-supervised pre-training
def augment_graph(x: torch.Tensor, edge_index: torch.Tensor, kind: str, ratio: float = 0.2, generator: torch.Generator | None = None):
    """``node_drop`` (removes nodes and their edges, re-indexing), ``edge_perturb`` (drops a share of edges and adds as many
    random ones), ``feature_mask`` (zeroes a share of feature columns), ``subgraph`` (keeps a random-walk neighbourhood)."""
    n = x.shape[0]
    if kind == "feature_mask":
        keep = torch.rand(x.shape[1], generator=generator) >= ratio
        return x * keep, edge_index
    if kind == "edge_perturb":
        m = edge_index.shape[1]
        keep = torch.rand(m, generator=generator) >= ratio
        extra = torch.randint(0, n, (2, int((~keep).sum())), generator=generator)
        return x, torch.cat([edge_index[:, keep], extra], 1)
    if kind in ("node_drop", "subgraph"):
        if kind == "node_drop":
            keep = torch.rand(n, generator=generator) >= ratio
        else:
            keep = torch.zeros(n, dtype=torch.bool)
            frontier = {int(torch.randint(0, n, (1,), generator=generator))}
            nbrs = defaultdict(list)
            for a, b in edge_index.T.tolist():
                nbrs[a].append(b); nbrs[b].append(a)
            target = max(1, int((1 - ratio) * n))
            while frontier and int(keep.sum()) < target:
                v = frontier.pop(); keep[v] = True
                frontier.update(u for u in nbrs[v] if not keep[u])
        if not keep.any():
            keep[0] = True
        new_id = torch.full((n,), -1, dtype=torch.long); new_id[keep] = torch.arange(int(keep.sum()))
        e = edge_index[:, keep[edge_index[0]] & keep[edge_index[1]]]
        return x[keep], new_id[e]
    raise ValueError(kind)


def nt_xent(z1: torch.Tensor, z2: torch.Tensor, temperature: float = 0.5) -> torch.Tensor:
    z = nn.functional.normalize(torch.cat([z1, z2]), dim=1)
    sim = z @ z.T / temperature
    n = len(z1)
    sim = sim.masked_fill(torch.eye(2 * n, dtype=torch.bool), -1e9)
    target = torch.cat([torch.arange(n, 2 * n), torch.arange(0, n)])
    return nn.functional.cross_entropy(sim, target)


class GraphEncoder(nn.Module):
    def __init__(self, in_dim: int, hidden: int = 32, layers: int = 2):
        super().__init__()
        self.convs = nn.ModuleList([GCNConv(in_dim if i == 0 else hidden, hidden) for i in range(layers)])
    def forward(self, x, edge_index):
        for i, c in enumerate(self.convs):
            x = c(x, edge_index)
            if i < len(self.convs) - 1:
                x = torch.relu(x)
        return x
    def graph_embedding(self, x, edge_index): return self.forward(x, edge_index).mean(0)


def pretrain_contrastive(encoder: GraphEncoder, graphs: Sequence[tuple[torch.Tensor, torch.Tensor]], steps: int = 100, lr: float = 1e-2, augmentations=("node_drop", "edge_perturb"), temperature: float = 0.5, generator: torch.Generator | None = None) -> list[float]:
    """Two augmented views of every graph; the views of one graph attract, those of different graphs repel."""
    proj = nn.Sequential(nn.Linear(encoder.convs[-1].lin.out_features, 32), nn.ReLU(), nn.Linear(32, 16))
    opt, hist = torch.optim.Adam(list(encoder.parameters()) + list(proj.parameters()), lr=lr), []
    for _ in range(steps):
        z1 = torch.stack([encoder.graph_embedding(*augment_graph(x, e, augmentations[0], generator=generator)) for x, e in graphs])
        z2 = torch.stack([encoder.graph_embedding(*augment_graph(x, e, augmentations[1], generator=generator)) for x, e in graphs])
        loss = nt_xent(proj(z1), proj(z2), temperature)
        opt.zero_grad(); loss.backward(); opt.step(); hist.append(float(loss.detach()))
    return hist


def pretrain_masked_features(encoder: GraphEncoder, x: torch.Tensor, edge_index: torch.Tensor, steps: int = 200, lr: float = 1e-2, mask_ratio: float = 0.3, generator: torch.Generator | None = None) -> list[float]:
    """Hides the features of random nodes behind a learned token and reconstructs them from the neighbourhood."""
    token = nn.Parameter(torch.zeros(x.shape[1]))
    head = nn.Linear(encoder.convs[-1].lin.out_features, x.shape[1])
    opt, hist = torch.optim.Adam(list(encoder.parameters()) + list(head.parameters()) + [token], lr=lr), []
    for _ in range(steps):
        m = torch.rand(x.shape[0], generator=generator) < mask_ratio
        if not m.any():
            continue
        xin = torch.where(m[:, None], token.expand_as(x), x)
        loss = nn.functional.mse_loss(head(encoder(xin, edge_index))[m], x[m])
        opt.zero_grad(); loss.backward(); opt.step(); hist.append(float(loss.detach()))
    return hist


class GraphPromptTuning(nn.Module):
    """Adapts a frozen pre-trained encoder to a task with a few parameters: a learnable prompt vector added to every node's
    features and a linear head."""

    def __init__(self, encoder: GraphEncoder, in_dim: int, num_classes: int):
        super().__init__()
        self.encoder = encoder
        for p in encoder.parameters():
            p.requires_grad_(False)
        self.prompt, self.head = nn.Parameter(torch.zeros(in_dim)), nn.Linear(encoder.convs[-1].lin.out_features, num_classes)
    def forward(self, x, edge_index): return self.head(self.encoder(x + self.prompt, edge_index))
    def trainable_parameters(self) -> int: return sum(p.numel() for p in self.parameters() if p.requires_grad)
