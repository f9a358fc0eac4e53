"""Graph models beyond message passing (``crates/torsh-graph/src/{classification,generative,diffusion,explainability,
quantum,neuromorphic,neural_operators,optimal_transport,matching,foundation,multimodal}.rs``): graph-level classifiers
and regressors, variational graph auto-encoders and a graph GAN, discrete denoising diffusion over adjacency matrices,
layer-wise relevance propagation and gradient attributions, quantum walks and a QAOA max-cut layer simulated as state
vectors, spiking graph networks and a liquid state machine, spectral graph neural operators and a DeepONet, a
physics-informed heat-equation GNN, Gromov-Wasserstein barycentres, siamese and cross-graph matching networks, a
foundation-model wrapper with task heads, and cross-modal attention.

All dense algebra is batched matrix products on the input's device; graphs are ``edge_index`` ``(2, E)`` tensors as in
``graph``."""
from __future__ import annotations

import math
from typing import Sequence

import torch
from torch import nn

from .graph import GCNConv, GATConv, global_add_pool, global_max_pool, global_mean_pool, scatter_add
from .graph_ext import gromov_wasserstein

__all__ = [
    "dense_adjacency", "normalized_laplacian", "GraphClassificationGCN", "GraphClassificationGAT", "GraphRegressor",
    "HierarchicalGraphClassifier", "MultiTaskGraphNetwork", "GraphVAE", "GraphGAN", "ConditionalGraphGenerator",
    "DiscreteGraphDiffusion", "GraphLRP", "GraphGradientAttribution", "QuantumWalk", "QuantumQAOA", "QuantumGraphLayer",
    "SpikingGraphNetwork", "LiquidStateMachine", "GraphFNO", "GraphDeepONet", "PhysicsInformedGNN", "GraphBarycenter",
    "SiameseGraphNetwork", "GraphMatchingNetwork", "GraphFoundationModel", "CrossModalGraphAttention", "MultiModalFusion",
]


def dense_adjacency(edge_index: torch.Tensor, n: int, symmetric: bool = True, dtype=torch.float32) -> torch.Tensor:
    a = torch.zeros(n, n, dtype=dtype, device=edge_index.device)
    a[edge_index[0], edge_index[1]] = 1
    return torch.maximum(a, a.T) if symmetric else a


def normalized_laplacian(adj: torch.Tensor) -> torch.Tensor:
    d = adj.sum(1).clamp(min=1e-12).rsqrt()
    return torch.eye(len(adj), dtype=adj.dtype, device=adj.device) - d[:, None] * adj * d[None]


# ================================================================================================ graph-level prediction
class _GraphEncoderBase(nn.Module):
    def __init__(self, convs: Sequence[nn.Module], readout: str = "mean+max"):
        super().__init__()
        self.convs, self.readout = nn.ModuleList(convs), readout

    def node_embeddings(self, x, edge_index):
        for c in self.convs:
            x = torch.relu(c(x, edge_index))
        return x

    def pool(self, h, batch, n_graphs):
        parts = {"mean": global_mean_pool, "max": global_max_pool, "sum": global_add_pool}
        return torch.cat([parts[p](h, batch, n_graphs) for p in self.readout.split("+")], 1)

    def embed(self, x, edge_index, batch=None):
        batch = torch.zeros(len(x), dtype=torch.long, device=x.device) if batch is None else batch
        return self.pool(self.node_embeddings(x, edge_index), batch, int(batch.max()) + 1)


class GraphClassificationGCN(_GraphEncoderBase):
    def __init__(self, in_dim: int, hidden: int, num_classes: int, layers: int = 3, readout: str = "mean+max", dropout: float = 0.0):
        super().__init__([GCNConv(in_dim if i == 0 else hidden, hidden) for i in range(layers)], readout)
        self.head = nn.Sequential(nn.Linear(hidden * len(readout.split("+")), hidden), nn.ReLU(), nn.Dropout(dropout), nn.Linear(hidden, num_classes))
    def forward(self, x, edge_index, batch=None): return self.head(self.embed(x, edge_index, batch))


class GraphClassificationGAT(_GraphEncoderBase):
    def __init__(self, in_dim: int, hidden: int, num_classes: int, layers: int = 2, heads: int = 4, readout: str = "mean"):
        super().__init__([GATConv(in_dim if i == 0 else hidden, hidden // heads, heads) for i in range(layers)], readout)
        self.head = nn.Linear(hidden * len(readout.split("+")), num_classes)
    def forward(self, x, edge_index, batch=None): return self.head(self.embed(x, edge_index, batch))


class GraphRegressor(GraphClassificationGCN):
    def __init__(self, in_dim: int, hidden: int, targets: int = 1, layers: int = 3, readout: str = "sum"):
        super().__init__(in_dim, hidden, targets, layers, readout)


class HierarchicalGraphClassifier(nn.Module):
    """Conv -> top-k pooling (score = projection on a learned vector, kept nodes gated by ``tanh(score)``) repeated per level;
    the readouts of all levels are summed before the classifier."""
    def __init__(self, in_dim: int, hidden: int, num_classes: int, levels: int = 2, ratio: float = 0.5):
        super().__init__()
        self.convs = nn.ModuleList(GCNConv(in_dim if i == 0 else hidden, hidden) for i in range(levels))
        self.scores = nn.ParameterList(nn.Parameter(torch.randn(hidden) / math.sqrt(hidden)) for _ in range(levels))
        self.ratio, self.head = ratio, nn.Linear(2 * hidden, num_classes)

    def forward(self, x, edge_index, batch=None):
        batch = torch.zeros(len(x), dtype=torch.long, device=x.device) if batch is None else batch
        g = int(batch.max()) + 1
        out = 0
        self.kept = []
        for conv, p in zip(self.convs, self.scores):
            x = torch.relu(conv(x, edge_index))
            s = x @ (p / p.norm())
            keep = torch.cat([(batch == b).nonzero().flatten()[s[batch == b].topk(max(1, math.ceil(self.ratio * int((batch == b).sum())))).indices] for b in range(g)])
            keep = keep.sort().values
            remap = torch.full((len(x),), -1, dtype=torch.long, device=x.device)
            remap[keep] = torch.arange(len(keep), device=x.device)
            x, batch = x[keep] * torch.tanh(s[keep])[:, None], batch[keep]
            ei = remap[edge_index]
            edge_index = ei[:, (ei >= 0).all(0)]
            self.kept.append(keep)
            out = out + torch.cat([global_mean_pool(x, batch, g), global_max_pool(x, batch, g)], 1)
        return self.head(out)


class MultiTaskGraphNetwork(nn.Module):
    """One shared encoder, one head per task (``node`` or ``graph`` level); ``loss`` weights the tasks by learned
    homoscedastic uncertainties ``exp(-s_t) L_t + s_t``."""
    def __init__(self, in_dim: int, hidden: int, tasks: dict[str, tuple[str, int]], layers: int = 2):
        super().__init__()
        self.encoder = _GraphEncoderBase([GCNConv(in_dim if i == 0 else hidden, hidden) for i in range(layers)], "mean")
        self.tasks = tasks
        self.heads = nn.ModuleDict({t: nn.Linear(hidden, out) for t, (_, out) in tasks.items()})
        self.log_vars = nn.ParameterDict({t: nn.Parameter(torch.zeros(())) for t in tasks})
    def forward(self, x, edge_index, batch=None) -> dict:
        h = self.encoder.node_embeddings(x, edge_index)
        batch = torch.zeros(len(x), dtype=torch.long, device=x.device) if batch is None else batch
        pooled = global_mean_pool(h, batch, int(batch.max()) + 1)
        return {t: self.heads[t](h if level == "node" else pooled) for t, (level, _) in self.tasks.items()}
    def loss(self, losses: dict[str, torch.Tensor]) -> torch.Tensor:
        return sum(torch.exp(-self.log_vars[t]) * l + self.log_vars[t] for t, l in losses.items())


# ================================================================================================ generative
class GraphVAE(nn.Module):
    """Variational graph auto-encoder: two GCN layers give ``mu`` and ``log sigma^2`` per node, edges are decoded as
    ``sigmoid(z_i . z_j)``; the loss re-weights the rare positive entries and adds the KL term."""
    def __init__(self, in_dim: int, hidden: int = 32, latent: int = 16):
        super().__init__()
        self.base, self.mu, self.logvar = GCNConv(in_dim, hidden), GCNConv(hidden, latent), GCNConv(hidden, latent)
    def encode(self, x, edge_index):
        h = torch.relu(self.base(x, edge_index))
        return self.mu(h, edge_index), self.logvar(h, edge_index).clamp(max=10)
    def decode(self, z): return z @ z.T
    def forward(self, x, edge_index):
        mu, lv = self.encode(x, edge_index)
        z = mu + torch.randn_like(mu) * torch.exp(0.5 * lv) if self.training else mu
        return self.decode(z), mu, lv
    def loss(self, x, edge_index):
        n = len(x)
        adj = dense_adjacency(edge_index, n, dtype=x.dtype) + torch.eye(n, dtype=x.dtype, device=x.device)
        logits, mu, lv = self(x, edge_index)
        pos_w = (n * n - adj.sum()) / adj.sum()
        rec = nn.functional.binary_cross_entropy_with_logits(logits, adj, pos_weight=pos_w)
        kl = -0.5 / n * (1 + lv - mu ** 2 - lv.exp()).sum(1).mean()
        return rec + kl
    @torch.no_grad()
    def sample(self, n: int, latent: int | None = None, threshold: float = 0.5) -> torch.Tensor:
        z = torch.randn(n, latent or self.mu.lin.out_features)
        return (torch.sigmoid(self.decode(z)) > threshold).float().fill_diagonal_(0)


class GraphGAN(nn.Module):
    """Generator: noise -> symmetric edge probabilities (MLP on the upper triangle); discriminator: permutation-invariant
    statistics of the soft adjacency (degree moments, triangle and edge densities) -> real / fake logit."""
    def __init__(self, n_nodes: int, noise: int = 16, hidden: int = 64):
        super().__init__()
        self.n, self.noise = n_nodes, noise
        self.iu = torch.triu_indices(n_nodes, n_nodes, 1)
        self.gen = nn.Sequential(nn.Linear(noise, hidden), nn.ReLU(), nn.Linear(hidden, hidden), nn.ReLU(), nn.Linear(hidden, self.iu.shape[1]))
        self.disc = nn.Sequential(nn.Linear(6, hidden), nn.LeakyReLU(0.2), nn.Linear(hidden, 1))
    def generate(self, batch: int, z: torch.Tensor | None = None) -> torch.Tensor:
        z = torch.randn(batch, self.noise) if z is None else z
        p = torch.sigmoid(self.gen(z))
        a = torch.zeros(len(z), self.n, self.n, dtype=p.dtype)
        a[:, self.iu[0], self.iu[1]] = p
        return a + a.transpose(1, 2)
    @staticmethod
    def statistics(a: torch.Tensor) -> torch.Tensor:
        n = a.shape[-1]
        deg = a.sum(-1)
        tri = torch.einsum("bij,bjk,bki->b", a, a, a) / 6
        return torch.stack([deg.mean(1) / n, deg.std(1) / n, deg.max(1).values / n, a.sum((1, 2)) / (n * (n - 1)), tri / math.comb(n, 3), (deg ** 2).mean(1) / n ** 2], 1)
    def discriminate(self, a: torch.Tensor) -> torch.Tensor: return self.disc(self.statistics(a)).squeeze(-1)
    def losses(self, real: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        fake = self.generate(len(real))
        bce = nn.functional.binary_cross_entropy_with_logits
        d = bce(self.discriminate(real), torch.ones(len(real))) + bce(self.discriminate(fake.detach()), torch.zeros(len(real)))
        return d, bce(self.discriminate(fake), torch.ones(len(real)))


class ConditionalGraphGenerator(GraphGAN):
    """The generator also sees a condition vector (target density, class, ...)."""
    def __init__(self, n_nodes: int, cond_dim: int, noise: int = 16, hidden: int = 64):
        super().__init__(n_nodes, noise + cond_dim, hidden)
        self.base_noise = noise
    def generate_conditioned(self, cond: torch.Tensor) -> torch.Tensor:
        return self.generate(len(cond), torch.cat([torch.randn(len(cond), self.base_noise), cond], 1))


class DiscreteGraphDiffusion(nn.Module):
    """Denoising diffusion over binary adjacency matrices.  Forward process: every edge slot is resampled towards the
    marginal density ``rho`` with the closed-form ``q(a_t = 1 | a_0) = abar_t a_0 + (1 - abar_t) rho``.  The denoiser (a
    GCN over the noisy graph with node degree and time features) predicts the clean edges; sampling walks the posterior."""
    def __init__(self, steps: int = 50, hidden: int = 32, rho: float = 0.1):
        super().__init__()
        self.T, self.rho = steps, rho
        betas = torch.linspace(1e-3, 0.25, steps)
        self.register_buffer("abar", torch.cumprod(1 - betas, 0))
        self.register_buffer("alpha", 1 - betas)
        self.c1, self.c2 = GCNConv(3, hidden), GCNConv(hidden, hidden)
        self.edge = nn.Sequential(nn.Linear(2 * hidden + 2, hidden), nn.ReLU(), nn.Linear(hidden, 1))
    def q_prob(self, a0: torch.Tensor, t: int) -> torch.Tensor: return self.abar[t] * a0 + (1 - self.abar[t]) * self.rho
    def q_sample(self, a0: torch.Tensor, t: int, generator=None) -> torch.Tensor:
        u = torch.rand(a0.shape, generator=generator)
        noisy = (torch.triu(u, 1) < torch.triu(self.q_prob(a0, t), 1)).to(a0.dtype)
        noisy = torch.triu(noisy, 1)
        return noisy + noisy.T
    def denoise_logits(self, at: torch.Tensor, t: int) -> torch.Tensor:
        n = len(at)
        ei = at.nonzero().T
        deg = at.sum(1, keepdim=True)
        feat = torch.cat([deg / n, torch.full((n, 1), t / self.T, dtype=at.dtype), torch.ones(n, 1, dtype=at.dtype)], 1)
        h = torch.relu(self.c2(torch.relu(self.c1(feat, ei)), ei))
        common = (at @ at) / n
        pair = torch.cat([(h[:, None] + h[None]).expand(n, n, -1), (h[:, None] * h[None]), at[..., None], common[..., None]], -1)
        logits = self.edge(pair).squeeze(-1)
        return (logits + logits.T) / 2
    def loss(self, a0: torch.Tensor, generator=None) -> torch.Tensor:
        t = int(torch.randint(0, self.T, (1,), generator=generator))
        at = self.q_sample(a0, t, generator)
        iu = torch.triu_indices(len(a0), len(a0), 1)
        return nn.functional.binary_cross_entropy_with_logits(self.denoise_logits(at, t)[iu[0], iu[1]], a0[iu[0], iu[1]])
    def posterior(self, at: torch.Tensor, p0: torch.Tensor, t: int) -> torch.Tensor:
        """``q(a_{t-1} = 1 | a_t, a_0 ~ Bernoulli(p0))`` for every slot."""
        if t == 0:
            return p0
        al, rho = self.alpha[t], self.rho
        def lik(prev):                                                # q(a_t | a_{t-1} = prev)
            p1 = al * prev + (1 - al) * rho
            return at * p1 + (1 - at) * (1 - p1)
        out = 0
        for a0, w in ((1.0, p0), (0.0, 1 - p0)):
            prior1 = self.abar[t - 1] * a0 + (1 - self.abar[t - 1]) * rho
            num = lik(1.0) * prior1
            out = out + w * num / (num + lik(0.0) * (1 - prior1))
        return out
    @torch.no_grad()
    def sample(self, n: int, generator=None) -> torch.Tensor:
        a = torch.triu((torch.rand(n, n, generator=generator) < self.rho).float(), 1)
        a = a + a.T
        for t in reversed(range(self.T)):
            p = self.posterior(a, torch.sigmoid(self.denoise_logits(a, t)), t)
            a = torch.triu((torch.rand(n, n, generator=generator) < p).float(), 1)
            a = a + a.T
        return a


# ================================================================================================ explanations
class GraphLRP:
    """Layer-wise relevance propagation (epsilon rule) through a stack of dense GCN layers ``H' = relu(A_hat H W)``:
    relevance of the chosen output logit is redistributed to input nodes and features; the total is conserved up to the
    bias and epsilon terms."""
    def __init__(self, weights: Sequence[torch.Tensor], eps: float = 1e-9): self.weights, self.eps = list(weights), eps
    @staticmethod
    def a_hat(adj: torch.Tensor) -> torch.Tensor:
        a = adj + torch.eye(len(adj), dtype=adj.dtype)
        d = a.sum(1).rsqrt()
        return d[:, None] * a * d[None]
    def forward(self, x, adj):
        ah, acts = self.a_hat(adj), [x]
        for i, w in enumerate(self.weights):
            z = ah @ acts[-1] @ w
            acts.append(torch.relu(z) if i < len(self.weights) - 1 else z)
        return acts, ah
    def explain(self, x: torch.Tensor, adj: torch.Tensor, node: int, target: int) -> dict:
        acts, ah = self.forward(x, adj)
        rel = torch.zeros_like(acts[-1])
        rel[node, target] = acts[-1][node, target]
        for w, h in zip(reversed(self.weights), reversed(acts[:-1])):
            # z[v, c] = sum_{u, f} ah[v, u] h[u, f] w[f, c]: share relevance in proportion to each contribution
            z = ah @ h @ w
            s = rel / (z + self.eps * torch.where(z >= 0, torch.ones_like(z), -torch.ones_like(z)))
            rel = h * (ah.T @ s @ w.T)
        return {"feature_relevance": rel, "node_relevance": rel.sum(1), "output": float(acts[-1][node, target])}


class GraphGradientAttribution:
    """Saliency, gradient x input and integrated gradients of a model ``f(x, edge_index) -> (N, C)`` with respect to node
    features, plus edge importance from the gradient of a soft edge mask."""
    def __init__(self, model): self.model = model
    def _grad(self, x, edge_index, node, target):
        x = x.clone().requires_grad_(True)
        self.model(x, edge_index)[node, target].backward()
        return x.grad
    def saliency(self, x, edge_index, node, target): return self._grad(x, edge_index, node, target).abs()
    def gradient_x_input(self, x, edge_index, node, target): return self._grad(x, edge_index, node, target) * x
    def integrated_gradients(self, x, edge_index, node, target, steps: int = 32, baseline=None):
        base = torch.zeros_like(x) if baseline is None else baseline
        total = sum(self._grad(base + (k + 0.5) / steps * (x - base), edge_index, node, target) for k in range(steps))
        return (x - base) * total / steps
    def edge_importance(self, dense_model, x, adj, node, target):
        mask = torch.ones_like(adj, requires_grad=True)
        dense_model(x, adj * mask)[node, target].backward()
        return (mask.grad * adj).abs()


# ================================================================================================ quantum (state-vector simulation)
class QuantumWalk:
    """Continuous-time quantum walk ``psi(t) = exp(-i A t) psi(0)`` via the eigendecomposition of the adjacency matrix."""
    def __init__(self, adj: torch.Tensor):
        self.w, self.v = torch.linalg.eigh(adj.double())
    def evolve(self, start: int | torch.Tensor, t: float) -> torch.Tensor:
        psi0 = torch.zeros(len(self.w), dtype=torch.complex128)
        if isinstance(start, int):
            psi0[start] = 1
        else:
            psi0 = start.to(torch.complex128)
        v = self.v.to(torch.complex128)
        return v @ (torch.exp(-1j * self.w * t) * (v.T @ psi0))
    def probabilities(self, start, t: float) -> torch.Tensor: return self.evolve(start, t).abs() ** 2
    def average_distribution(self, start: int, horizon: float, samples: int = 200) -> torch.Tensor:
        return torch.stack([self.probabilities(start, horizon * (k + 1) / samples) for k in range(samples)]).mean(0)
    def node_features(self, times: Sequence[float]) -> torch.Tensor:
        """Return probability of every node at the given times: a structural descriptor."""
        n = len(self.w)
        return torch.stack([torch.stack([self.probabilities(i, t)[i] for i in range(n)]) for t in times], 1)


class QuantumQAOA(nn.Module):
    """QAOA for max-cut, simulated exactly on ``2^n`` amplitudes (``n <= 16``).  Cost layer: phase ``exp(-i gamma C(z))``;
    mixer: ``RX(2 beta)`` on every qubit.  ``forward`` returns the expected cut, differentiable in the angles."""
    def __init__(self, edge_index: torch.Tensor, n: int, depth: int = 2):
        super().__init__()
        if n > 16:
            raise ValueError("state-vector simulation limited to 16 nodes")
        self.n, self.depth = n, depth
        z = torch.arange(2 ** n)
        bits = (z[:, None] >> torch.arange(n)[None]) & 1
        und = {tuple(sorted(e)) for e in edge_index.T.tolist() if e[0] != e[1]}
        self.register_buffer("cut", torch.stack([(bits[:, a] != bits[:, b]).double() for a, b in und]).sum(0))
        self.register_buffer("bits", bits)
        self.gamma, self.beta = nn.Parameter(torch.full((depth,), 0.4, dtype=torch.float64)), nn.Parameter(torch.full((depth,), 0.3, dtype=torch.float64))
    def state(self) -> torch.Tensor:
        n = self.n
        psi = torch.full((2 ** n,), 2 ** (-n / 2), dtype=torch.complex128)
        for g, b in zip(self.gamma, self.beta):
            psi = psi * torch.exp(-1j * g * self.cut)
            c, s = torch.cos(b).to(torch.complex128), (-1j * torch.sin(b))
            psi = psi.reshape([2] * n)
            for q in range(n):
                psi = psi.movedim(q, 0)
                psi = torch.stack([c * psi[0] + s * psi[1], s * psi[0] + c * psi[1]]).movedim(0, q)
            psi = psi.reshape(-1)
        return psi
    def forward(self) -> torch.Tensor: return (self.state().abs() ** 2 * self.cut).sum()
    def optimize(self, steps: int = 150, lr: float = 0.05) -> float:
        opt = torch.optim.Adam(self.parameters(), lr=lr)
        for _ in range(steps):
            opt.zero_grad()
            (-self()).backward()
            opt.step()
        return float(self())
    def best_assignment(self) -> tuple[torch.Tensor, float]:
        # qubit q is the axis q of the reshaped state, i.e. the bit of weight 2^(n-1-q)
        k = int((self.state().abs() ** 2).argmax())
        return self.bits[k], float(self.cut[k])
    def max_cut(self) -> float: return float(self.cut.max())


class QuantumGraphLayer(nn.Module):
    """Node features from quantum-walk return probabilities at learnable times, mixed with the input by a linear layer."""
    def __init__(self, in_dim: int, out_dim: int, n_times: int = 4):
        super().__init__()
        self.times = nn.Parameter(torch.linspace(0.5, 2.0, n_times))
        self.lin = nn.Linear(in_dim + n_times, out_dim)
    def forward(self, x, adj):
        w, v = torch.linalg.eigh(adj.double())
        # return amplitude of node i at time t: sum_k v[i,k]^2 exp(-i w_k t)
        phase = torch.exp(-1j * w[None, :, None] * self.times.double()[None, None, :])
        amp = ((v ** 2).to(torch.complex128)[:, :, None] * phase).sum(1)
        return self.lin(torch.cat([x, (amp.abs() ** 2).to(x.dtype)], 1))


# ================================================================================================ neuromorphic
class SpikingGraphNetwork(nn.Module):
    """Leaky integrate-and-fire neurons on the nodes: the input current is the projected feature plus spikes of the
    neighbours from the previous step through the normalised adjacency; rate-coded output over ``steps`` with a
    fast-sigmoid surrogate gradient."""
    def __init__(self, in_dim: int, hidden: int, out_dim: int, steps: int = 20, decay: float = 0.9, threshold: float = 1.0):
        super().__init__()
        self.inp, self.rec, self.out = nn.Linear(in_dim, hidden), nn.Linear(hidden, hidden, bias=False), nn.Linear(hidden, out_dim)
        self.steps, self.decay, self.th = steps, decay, threshold
    @staticmethod
    def _spike(v):
        soft = torch.sigmoid(4 * v)
        return (v > 0).to(v.dtype).detach() + soft - soft.detach()
    def forward(self, x, adj):
        a = GraphLRP.a_hat(adj.to(x.dtype))
        cur = self.inp(x)
        v = torch.zeros_like(cur)
        s = torch.zeros_like(cur)
        count = torch.zeros_like(cur)
        for _ in range(self.steps):
            v = self.decay * v + cur + a @ self.rec(s)
            s = self._spike(v - self.th)
            v = v - s * self.th
            count = count + s
        self.spike_rate = count / self.steps
        return self.out(self.spike_rate)


class LiquidStateMachine(nn.Module):
    """A fixed random recurrent reservoir whose connectivity is the graph; only the linear read-out is trained (ridge
    regression in closed form)."""
    def __init__(self, adj: torch.Tensor, in_dim: int, spectral_radius: float = 0.9, leak: float = 0.3, seed: int = 0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        w = adj.double() * torch.randn(adj.shape, generator=g, dtype=torch.float64)
        w = w * spectral_radius / torch.linalg.eigvals(w).abs().max().clamp(min=1e-12)
        self.register_buffer("w", w)
        self.register_buffer("w_in", torch.randn(len(adj), in_dim, generator=g, dtype=torch.float64))
        self.leak, self.readout = leak, None
    def states(self, u: torch.Tensor) -> torch.Tensor:
        x, out = torch.zeros(len(self.w), dtype=torch.float64), []
        for ut in u.double():
            x = (1 - self.leak) * x + self.leak * torch.tanh(self.w @ x + self.w_in @ ut)
            out.append(x)
        return torch.stack(out)
    def fit(self, u: torch.Tensor, y: torch.Tensor, ridge: float = 1e-6, washout: int = 20) -> "LiquidStateMachine":
        s = self.states(u)[washout:]
        s = torch.cat([s, torch.ones(len(s), 1, dtype=torch.float64)], 1)
        self.readout = torch.linalg.solve(s.T @ s + ridge * torch.eye(s.shape[1], dtype=torch.float64), s.T @ y.double()[washout:])
        return self
    def predict(self, u: torch.Tensor) -> torch.Tensor:
        s = self.states(u)
        return torch.cat([s, torch.ones(len(s), 1, dtype=torch.float64)], 1) @ self.readout


# ================================================================================================ neural operators
class GraphFNO(nn.Module):
    """Fourier neural operator on a graph: the graph Fourier basis is the lowest ``modes`` Laplacian eigenvectors; every
    layer multiplies the spectral coefficients by learned per-mode channel mixers and adds a pointwise linear path."""
    def __init__(self, in_dim: int, width: int, out_dim: int, modes: int = 16, layers: int = 3):
        super().__init__()
        self.lift, self.proj, self.modes = nn.Linear(in_dim, width), nn.Linear(width, out_dim), modes
        self.spectral = nn.ParameterList(nn.Parameter(torch.randn(modes, width, width) / width) for _ in range(layers))
        self.local = nn.ModuleList(nn.Linear(width, width) for _ in range(layers))
    def basis(self, adj: torch.Tensor) -> torch.Tensor: return torch.linalg.eigh(normalized_laplacian(adj))[1][:, :self.modes]
    def forward(self, x, adj, basis: torch.Tensor | None = None):
        u = self.basis(adj).to(x.dtype) if basis is None else basis
        h = self.lift(x)
        for w, loc in zip(self.spectral, self.local):
            coeff = u.T @ h
            h = torch.nn.functional.gelu(u @ torch.einsum("mc,mcd->md", coeff, w[: u.shape[1]]) + loc(h))
        return self.proj(h)


class GraphDeepONet(nn.Module):
    """Operator learning ``G(u)(y) = sum_k branch_k(u) trunk_k(y)``: the branch net reads the input function sampled on
    the graph's nodes, the trunk net reads query coordinates (node positions or spectral embeddings)."""
    def __init__(self, n_sensors: int, coord_dim: int, width: int = 64, basis: int = 32):
        super().__init__()
        self.branch = nn.Sequential(nn.Linear(n_sensors, width), nn.Tanh(), nn.Linear(width, basis))
        self.trunk = nn.Sequential(nn.Linear(coord_dim, width), nn.Tanh(), nn.Linear(width, basis), nn.Tanh())
        self.bias = nn.Parameter(torch.zeros(()))
    def forward(self, u: torch.Tensor, coords: torch.Tensor) -> torch.Tensor: return self.branch(u) @ self.trunk(coords).T + self.bias


class PhysicsInformedGNN(nn.Module):
    """Learns one explicit step of a diffusion process on a graph; the physics residual ``(u' - u) / dt + kappa L u``
    with a learnable ``kappa`` ties the prediction to the heat equation."""
    def __init__(self, hidden: int = 32, dt: float = 0.1):
        super().__init__()
        self.c1, self.c2, self.dt = GCNConv(1, hidden), GCNConv(hidden, 1), dt
        self.log_kappa = nn.Parameter(torch.zeros(()))
    def forward(self, u: torch.Tensor, edge_index: torch.Tensor) -> torch.Tensor:
        return u + self.dt * self.c2(torch.tanh(self.c1(u[:, None], edge_index)), edge_index).squeeze(1)
    def residual(self, u, u_next, lap) -> torch.Tensor: return (u_next - u) / self.dt + torch.exp(self.log_kappa) * (lap @ u)
    def loss(self, u, target, edge_index, lap, physics_weight: float = 1.0) -> torch.Tensor:
        pred = self(u, edge_index)
        return ((pred - target) ** 2).mean() + physics_weight * (self.residual(u, pred, lap) ** 2).mean()


# ================================================================================================ transport and matching
class GraphBarycenter:
    """Gromov-Wasserstein barycentre of structure matrices: alternate between coupling every input to the current
    barycentre and the closed-form update ``C = sum_s lambda_s T_s^T C_s T_s / (p p^T)``."""
    def __init__(self, size: int, iters: int = 10, reg: float = 0.01, seed: int = 0): self.size, self.iters, self.reg, self.seed = size, iters, reg, seed
    def fit(self, structures: Sequence[torch.Tensor], weights: Sequence[float] | None = None) -> torch.Tensor:
        lam = torch.tensor(weights or [1 / len(structures)] * len(structures), dtype=torch.float64)
        p = torch.full((self.size,), 1 / self.size, dtype=torch.float64)
        g = torch.Generator().manual_seed(self.seed)
        c = torch.rand(self.size, self.size, generator=g, dtype=torch.float64)
        c = (c + c.T) / 2
        self.couplings = []
        for _ in range(self.iters):
            ts = [gromov_wasserstein(cs.double(), c, reg=self.reg)[0] for cs in structures]
            c = sum(l * t.T @ cs.double() @ t for l, t, cs in zip(lam, ts, structures)) / (p[:, None] * p[None])
            self.couplings = ts
        self.structure = c
        return c


class SiameseGraphNetwork(nn.Module):
    """One encoder applied to both graphs; similarity = cosine of the pooled embeddings; contrastive loss with margin."""
    def __init__(self, in_dim: int, hidden: int = 32, layers: int = 2):
        super().__init__()
        self.enc = _GraphEncoderBase([GCNConv(in_dim if i == 0 else hidden, hidden) for i in range(layers)], "sum")
    def embed(self, x, edge_index): return self.enc.embed(x, edge_index)[0]
    def forward(self, g1, g2): return nn.functional.cosine_similarity(self.embed(*g1), self.embed(*g2), dim=0)
    def contrastive_loss(self, g1, g2, same: bool, margin: float = 0.5):
        d = 1 - self(g1, g2)
        return d ** 2 if same else torch.clamp(margin - d, min=0) ** 2


class GraphMatchingNetwork(nn.Module):
    """Cross-graph attention (Li et al.): every propagation step adds, to the within-graph message, the difference
    between a node and its attention-weighted match in the other graph, so that unmatched structure stands out."""
    def __init__(self, in_dim: int, hidden: int = 32, layers: int = 3):
        super().__init__()
        self.inp = nn.Linear(in_dim, hidden)
        self.msg = nn.ModuleList(nn.Linear(2 * hidden, hidden) for _ in range(layers))
        self.upd = nn.ModuleList(nn.GRUCell(2 * hidden, hidden) for _ in range(layers))
        self.gate, self.out = nn.Linear(hidden, hidden), nn.Linear(hidden, hidden)
    def _within(self, h, ei, lin): return scatter_add(lin(torch.cat([h[ei[0]], h[ei[1]]], 1)), ei[1], len(h))
    def forward(self, g1, g2) -> torch.Tensor:
        (x1, e1), (x2, e2) = g1, g2
        h1, h2 = self.inp(x1), self.inp(x2)
        for lin, gru in zip(self.msg, self.upd):
            att = h1 @ h2.T
            mu1 = h1 - torch.softmax(att, 1) @ h2
            mu2 = h2 - torch.softmax(att.T, 1) @ h1
            h1, h2 = gru(torch.cat([self._within(h1, e1, lin), mu1], 1), h1), gru(torch.cat([self._within(h2, e2, lin), mu2], 1), h2)
        self.attention = torch.softmax(h1 @ h2.T, 1)
        pool = lambda h: (torch.sigmoid(self.gate(h)) * self.out(h)).sum(0)
        return -(pool(h1) - pool(h2)).pow(2).sum()                    # similarity: negative squared distance


# ================================================================================================ foundation model and modalities
class GraphFoundationModel(nn.Module):
    """A shared encoder with pre-training objectives (masked feature reconstruction, edge prediction) and attachable task
    heads (``node``, ``graph``, ``link``, ``regression``); ``freeze_encoder`` supports linear probing."""
    def __init__(self, in_dim: int, hidden: int = 64, layers: int = 3):
        super().__init__()
        self.encoder = _GraphEncoderBase([GCNConv(in_dim if i == 0 else hidden, hidden) for i in range(layers)], "mean")
        self.mask_token = nn.Parameter(torch.zeros(in_dim))
        self.mlm_head = nn.Linear(hidden, in_dim)
        self.heads = nn.ModuleDict()
        self.hidden = hidden
    def encode(self, x, edge_index): return self.encoder.node_embeddings(x, edge_index)
    def add_head(self, name: str, kind: str, out_dim: int = 1):
        self.heads[name] = nn.Linear(2 * self.hidden if kind == "link" else self.hidden, out_dim)
        self.heads[name].kind = kind
        return self
    def freeze_encoder(self, frozen: bool = True):
        for p in self.encoder.parameters():
            p.requires_grad_(not frozen)
    def pretrain_loss(self, x, edge_index, mask_rate: float = 0.15, generator=None) -> dict:
        mask = torch.rand(len(x), generator=generator) < mask_rate
        if not bool(mask.any()):
            mask[0] = True
        h = self.encode(torch.where(mask[:, None], self.mask_token.expand_as(x), x), edge_index)
        mlm = ((self.mlm_head(h)[mask] - x[mask]) ** 2).mean()
        n, e = len(x), edge_index.shape[1]
        neg = torch.randint(0, n, (2, e), generator=generator)
        score = lambda ei: (h[ei[0]] * h[ei[1]]).sum(1)
        bce = nn.functional.binary_cross_entropy_with_logits
        link = bce(score(edge_index), torch.ones(e)) + bce(score(neg), torch.zeros(e))
        return {"masked_features": mlm, "structure": link, "total": mlm + link}
    def forward(self, name: str, x, edge_index, batch=None, pairs: torch.Tensor | None = None):
        h, head = self.encode(x, edge_index), self.heads[name]
        if head.kind == "node":
            return head(h)
        if head.kind == "link":
            return head(torch.cat([h[pairs[0]], h[pairs[1]]], 1)).squeeze(-1)
        batch = torch.zeros(len(x), dtype=torch.long) if batch is None else batch
        return head(global_mean_pool(h, batch, int(batch.max()) + 1))


class CrossModalGraphAttention(nn.Module):
    """Nodes carry several modalities; every modality attends over the others' projections of the same node and of its
    neighbours (mask = adjacency with self loops)."""
    def __init__(self, dims: dict[str, int], hidden: int = 32, heads: int = 4):
        super().__init__()
        self.proj = nn.ModuleDict({m: nn.Linear(d, hidden) for m, d in dims.items()})
        self.attn = nn.ModuleDict({m: nn.MultiheadAttention(hidden, heads, batch_first=True) for m in dims})
    def forward(self, feats: dict[str, torch.Tensor], adj: torch.Tensor) -> dict[str, torch.Tensor]:
        h = {m: self.proj[m](x) for m, x in feats.items()}
        n = len(adj)
        allowed = (adj + torch.eye(n, dtype=adj.dtype)) > 0
        out = {}
        for m in h:
            others = torch.cat([h[o] for o in h if o != m], 0)[None]
            mask = ~allowed.repeat(1, len(h) - 1)
            out[m] = h[m] + self.attn[m](h[m][None], others, others, attn_mask=mask)[0][0]
        return out


class MultiModalFusion(nn.Module):
    """``concat``, gated sum (softmax over per-modality scalar gates per node) or low-rank bilinear product; a missing
    modality (``None``) is skipped by the gated form."""
    def __init__(self, dims: dict[str, int], out_dim: int, mode: str = "gated"):
        super().__init__()
        self.mode = mode
        self.proj = nn.ModuleDict({m: nn.Linear(d, out_dim) for m, d in dims.items()})
        self.gate = nn.ModuleDict({m: nn.Linear(d, 1) for m, d in dims.items()})
        self.cat = nn.Linear(out_dim * len(dims), out_dim)
    def forward(self, feats: dict[str, torch.Tensor | None]) -> torch.Tensor:
        present = {m: x for m, x in feats.items() if x is not None}
        if self.mode == "concat":
            return self.cat(torch.cat([self.proj[m](feats[m]) for m in self.proj], 1))
        if self.mode == "bilinear":
            out = None
            for m, x in present.items():
                out = self.proj[m](x) if out is None else out * self.proj[m](x)
            return out
        gates = torch.softmax(torch.cat([self.gate[m](x) for m, x in present.items()], 1), 1)
        self.last_gates = dict(zip(present, gates.T))
        return sum(gates[:, i:i + 1] * self.proj[m](x) for i, (m, x) in enumerate(present.items()))
