"""Adaptive and graph-level quantisation (``crates/torsh-quantization/src``): a pattern language over traced graphs with
constraints and a rewriter that inserts fused quantised blocks (``pattern_matching/``, ``fusion.rs``), a run-time engine that
chooses precision per tensor from its statistics, keeps a bit-rate budget and reacts to degradation
(``realtime_adaptive/``), learned codecs with a shared codebook for weight compression (``neural_codecs.rs``), automatic
configuration under hardware constraints with a Pareto front (``auto_config.rs``) and annealing-based bit allocation
(``quantum_enhanced.rs``, ``quantum.rs``: the annealing schedule, without the quantum vocabulary)."""
from __future__ import annotations

import math
from collections import Counter, deque
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch
import torch.fx
from torch import nn

from .quantization import dequantize, quantize_per_channel, quantize_per_tensor, sqnr_db


# ================================================================================================ graph patterns
@dataclass
class GraphPattern:
    """A chain of node kinds (module class names or function names), optionally with alternatives (``"ReLU|ReLU6"``), that must be
    connected output-to-input with no other consumer in between; ``constraints`` are predicates on the matched nodes."""
    name: str
    chain: Sequence[str]
    constraints: Sequence[Callable[[list, dict], bool]] = ()
    priority: int = 0


COMMON_PATTERNS = [
    GraphPattern("conv_bn_relu", ("Conv2d", "BatchNorm2d", "ReLU|ReLU6"), priority=3), GraphPattern("conv_bn", ("Conv2d", "BatchNorm2d"), priority=2), GraphPattern("conv_relu", ("Conv2d", "ReLU|ReLU6"), priority=2),
    GraphPattern("linear_relu", ("Linear", "ReLU|GELU"), priority=2), GraphPattern("linear_bn", ("Linear", "BatchNorm1d"), priority=2), GraphPattern("add_relu", ("add", "ReLU|relu"), priority=1),
    GraphPattern("matmul_add", ("matmul", "add"), priority=1), GraphPattern("linear", ("Linear",), priority=0), GraphPattern("conv", ("Conv2d",), priority=0)]


class PatternMatcher:
    def __init__(self, patterns: Sequence[GraphPattern] = COMMON_PATTERNS): self.patterns, self.stats = sorted(patterns, key=lambda p: (-p.priority, -len(p.chain))), Counter()

    @staticmethod
    def _kind(node: torch.fx.Node, mods: dict) -> str:
        if node.op == "call_module":
            return type(mods[node.target]).__name__
        return getattr(node.target, "__name__", str(node.target)) if node.op in ("call_function", "call_method") else node.op

    def match(self, gm: torch.fx.GraphModule) -> list[dict]:
        """Non-overlapping matches, higher priority and longer chains first."""
        mods, used, out = dict(gm.named_modules()), set(), []
        nodes = list(gm.graph.nodes)
        for pat in self.patterns:
            for n in nodes:
                chain, cur = [n], n
                ok = self._kind(n, mods) in pat.chain[0].split("|") and n not in used
                for want in pat.chain[1:]:
                    if not ok:
                        break
                    users = list(cur.users)
                    ok = len(users) == 1 and self._kind(users[0], mods) in want.split("|") and users[0] not in used
                    if ok:
                        cur = users[0]; chain.append(cur)
                if ok and all(c(chain, mods) for c in pat.constraints):
                    used.update(chain); self.stats[pat.name] += 1
                    out.append({"pattern": pat.name, "nodes": [c.name for c in chain], "_nodes": chain})
        return sorted(out, key=lambda m: nodes.index(m["_nodes"][0]))

    def coverage(self, gm: torch.fx.GraphModule) -> dict:
        compute = [n for n in gm.graph.nodes if n.op in ("call_module", "call_function", "call_method")]
        matched = {x for m in self.match(gm) for x in m["nodes"]}
        return {"matched": len(matched), "compute_nodes": len(compute), "fraction": len(matched) / max(len(compute), 1), "unmatched": [n.name for n in compute if n.name not in matched]}


class FusedQuantBlock(nn.Module):
    """Folded conv / linear (+ batch norm) with optional activation: int8 weights per output channel, dynamic per-tensor
    activation quantisation, one requantisation at the end."""

    def __init__(self, layer: nn.Module, bn: nn.Module | None, act: nn.Module | None, bits: int = 8):
        super().__init__()
        w, b = layer.weight.detach().clone(), (layer.bias.detach().clone() if layer.bias is not None else torch.zeros(layer.weight.shape[0]))
        if bn is not None:
            scale = bn.weight.detach() / torch.sqrt(bn.running_var + bn.eps)
            w, b = w * scale.reshape(-1, *[1] * (w.dim() - 1)), (b - bn.running_mean) * scale + bn.bias.detach()
        q, qp = quantize_per_channel(w, 0, bits)
        self.register_buffer("qweight", q); self.register_buffer("scale", qp.scale.reshape(-1)); self.register_buffer("bias", b)
        self.bits, self.act, self.kind = bits, act, "conv" if isinstance(layer, nn.Conv2d) else "linear"
        self.conv_args = dict(stride=layer.stride, padding=layer.padding, dilation=layer.dilation, groups=layer.groups) if self.kind == "conv" else None

    def forward(self, x):
        amax = x.detach().abs().amax().clamp_min(1e-12)
        qmax = 2 ** (self.bits - 1) - 1
        xs = amax / qmax
        xq = (x / xs).round().clamp(-qmax - 1, qmax)                               # integer-valued activations
        wq = self.qweight.to(x.dtype)
        acc = nn.functional.conv2d(xq, wq, None, **self.conv_args) if self.kind == "conv" else nn.functional.linear(xq, wq)
        shape = (1, -1, 1, 1) if self.kind == "conv" else (-1,)
        y = acc * (xs * self.scale.to(x.dtype)).reshape(shape) + self.bias.to(x.dtype).reshape(shape)
        return self.act(y) if self.act is not None else y


def fuse_and_quantize(model: nn.Module, bits: int = 8, matcher: PatternMatcher | None = None) -> tuple[torch.fx.GraphModule, list[dict]]:
    """Traces the model (in eval mode), replaces every matched conv / linear pattern by one :class:`FusedQuantBlock` and
    returns the rewritten graph with the list of replacements."""
    model.eval()
    gm = torch.fx.symbolic_trace(model)
    mods = dict(gm.named_modules())
    done = []
    for m in (matcher or PatternMatcher()).match(gm):
        nodes = m["_nodes"]
        if nodes[0].op != "call_module" or not isinstance(mods[nodes[0].target], (nn.Conv2d, nn.Linear)):
            continue
        layer = mods[nodes[0].target]
        rest = [mods[n.target] for n in nodes[1:] if n.op == "call_module"]
        bn = next((r for r in rest if isinstance(r, (nn.BatchNorm1d, nn.BatchNorm2d))), None)
        act = next((r for r in rest if not isinstance(r, (nn.BatchNorm1d, nn.BatchNorm2d))), None)
        name = "fused_" + nodes[0].name
        gm.add_submodule(name, FusedQuantBlock(layer, bn, act, bits))
        with gm.graph.inserting_after(nodes[-1]):
            new = gm.graph.call_module(name, nodes[0].args)
        nodes[-1].replace_all_uses_with(new)
        for n in reversed(nodes):
            gm.graph.erase_node(n)
        done.append({"pattern": m["pattern"], "replaced": m["nodes"], "by": name})
    gm.graph.lint(); gm.recompile(); gm.delete_all_unused_submodules()
    return gm, done


# ================================================================================================ run-time adaptive engine
def tensor_features(x: torch.Tensor) -> dict:
    f = x.detach().float().flatten()
    std = float(f.std()) if f.numel() > 1 else 0.0
    mean = float(f.mean())
    z = (f - mean) / (std or 1.0)
    amax = float(f.abs().max())
    return {"mean": mean, "std": std, "abs_max": amax, "kurtosis": float((z ** 4).mean()) if std else 0.0, "sparsity": float((f == 0).float().mean()), "outlier_ratio": float((f.abs() > 4 * (std or 1.0)).float().mean()),
            "dynamic_range_db": 20 * math.log10(amax / max(float(f.abs()[f != 0].min()) if (f != 0).any() else 1e-12, 1e-12)) if amax else 0.0, "numel": f.numel()}


@dataclass
class AdaptiveQuantConfig:
    candidate_bits: Sequence[int] = (4, 6, 8)
    min_sqnr_db: float = 30.0
    target_mean_bits: float = 6.0
    clip_outliers: bool = True
    degradation_window: int = 20
    degradation_drop_db: float = 6.0


class AdaptiveQuantizationEngine:
    """Per call: measure the tensor, pick the smallest candidate width whose predicted SQNR meets the floor (uniform quantiser
    model: ``6.02 b + 4.77 - 20 log10(range / std)``, with the clipping range reduced when the tensor has heavy tails), quantise,
    measure the achieved SQNR and feed it back.  A rate controller raises or lowers the floor so that the running mean width
    approaches the target; a degradation detector flags a sustained drop against the history."""

    def __init__(self, cfg: AdaptiveQuantConfig | None = None):
        self.cfg = cfg or AdaptiveQuantConfig()
        self.floor, self.history, self.bits_used, self.bias_db, self.alerts = self.cfg.min_sqnr_db, deque(maxlen=200), deque(maxlen=200), 0.0, []

    def _clip(self, feats: dict) -> float:
        if self.cfg.clip_outliers and feats["kurtosis"] > 6 and feats["std"]:
            return min(feats["abs_max"], 6 * feats["std"])
        return feats["abs_max"]

    def predict_sqnr(self, feats: dict, bits: int) -> float:
        clip = self._clip(feats)
        return 6.02 * bits + 4.77 - 20 * math.log10(max(clip, 1e-12) / max(feats["std"], 1e-12)) + self.bias_db if feats["std"] else math.inf

    def choose_bits(self, feats: dict) -> int:
        for b in sorted(self.cfg.candidate_bits):
            if self.predict_sqnr(feats, b) >= self.floor:
                return b
        return max(self.cfg.candidate_bits)

    def quantize(self, x: torch.Tensor) -> dict:
        feats = tensor_features(x)
        bits, clip = self.choose_bits(feats), self._clip(feats)
        qmax = 2 ** (bits - 1) - 1
        scale = max(clip, 1e-12) / qmax
        q = (x / scale).round().clamp(-qmax - 1, qmax)
        deq = q * scale
        achieved = sqnr_db(x.float(), deq.float())
        predicted = self.predict_sqnr(feats, bits)
        if math.isfinite(achieved) and math.isfinite(predicted):
            self.bias_db += 0.1 * (achieved - predicted)                               # the model learns its own offset
        self.history.append(achieved); self.bits_used.append(bits)
        self._rate_control(); self._detect_degradation()
        return {"q": q.to(torch.int8 if bits <= 8 else torch.int16), "scale": scale, "bits": bits, "sqnr_db": achieved, "predicted_db": predicted, "dequantized": deq, "features": feats}

    def _rate_control(self):
        if len(self.bits_used) >= 10:
            mean_bits = sum(self.bits_used) / len(self.bits_used)
            self.floor += 0.5 * (self.cfg.target_mean_bits - mean_bits)               # too many bits -> relax the floor; too few -> tighten
            self.floor = min(max(self.floor, 10.0), 60.0)

    def _detect_degradation(self):
        w = self.cfg.degradation_window
        if len(self.history) >= 2 * w:
            h = list(self.history)
            old, new = sum(h[-2 * w:-w]) / w, sum(h[-w:]) / w
            if old - new > self.cfg.degradation_drop_db and (not self.alerts or self.alerts[-1]["at"] < len(h) - w):
                self.alerts.append({"at": len(h), "drop_db": old - new})

    def summary(self) -> dict:
        return {"mean_bits": sum(self.bits_used) / max(len(self.bits_used), 1), "mean_sqnr_db": sum(self.history) / max(len(self.history), 1), "floor_db": self.floor, "bits_histogram": dict(Counter(self.bits_used)), "alerts": len(self.alerts)}


# ================================================================================================ learned codec
class NeuralCodec(nn.Module):
    """Blocks of ``block`` weights are encoded to ``latent`` numbers, snapped to the nearest entry of a learned codebook and
    decoded; only the codebook indices (``log2(codebook)`` bits per block) and the small decoder are stored.  Trained with the
    reconstruction loss plus codebook and commitment terms (straight-through gradients)."""

    def __init__(self, block: int = 16, latent: int = 4, codebook: int = 64, hidden: int = 64, beta: float = 0.25):
        super().__init__()
        self.block, self.beta = block, beta
        self.enc = nn.Sequential(nn.Linear(block, hidden), nn.GELU(), nn.Linear(hidden, latent))
        self.dec = nn.Sequential(nn.Linear(latent, hidden), nn.GELU(), nn.Linear(hidden, block))
        self.codebook = nn.Parameter(torch.randn(codebook, latent) * 0.5)

    def _blocks(self, w): f = w.flatten(); pad = (-len(f)) % self.block; return nn.functional.pad(f, (0, pad)).view(-1, self.block), pad

    def forward(self, blocks):
        z = self.enc(blocks)
        idx = torch.cdist(z, self.codebook).argmin(1)
        zq = self.codebook[idx]
        out = self.dec(z + (zq - z).detach())
        loss = nn.functional.mse_loss(out, blocks) + nn.functional.mse_loss(zq, z.detach()) + self.beta * nn.functional.mse_loss(z, zq.detach())
        return out, idx, loss

    def fit(self, weights: Sequence[torch.Tensor], steps: int = 500, lr: float = 3e-3, batch: int = 1024, generator: torch.Generator | None = None) -> list[float]:
        data = torch.cat([self._blocks(w.detach().float())[0] for w in weights])
        self.norm = float(data.std()) or 1.0
        data = data / self.norm
        with torch.no_grad():                                                       # start the codebook on encoded data
            z = self.enc(data[torch.randperm(len(data), generator=generator)[:len(self.codebook)]])
            self.codebook[:len(z)] = z
        opt, hist = torch.optim.Adam(self.parameters(), lr=lr), []
        for _ in range(steps):
            b = data[torch.randint(len(data), (min(batch, len(data)),), generator=generator)]
            _, _, loss = self(b)
            opt.zero_grad(); loss.backward(); opt.step(); hist.append(float(loss.detach()))
        return hist

    @torch.no_grad()
    def compress(self, w: torch.Tensor) -> dict:
        blocks, pad = self._blocks(w.float())
        _, idx, _ = self(blocks / self.norm)
        bits = math.ceil(math.log2(len(self.codebook)))
        return {"indices": idx.to(torch.int16 if bits <= 15 else torch.int32), "shape": tuple(w.shape), "pad": pad, "payload_bits": bits * len(idx), "ratio": w.numel() * 32 / (bits * len(idx))}

    @torch.no_grad()
    def decompress(self, c: dict) -> torch.Tensor:
        flat = (self.dec(self.codebook[c["indices"].long()]) * self.norm).flatten()
        return flat[:len(flat) - c["pad"]].reshape(c["shape"]) if c["pad"] else flat.reshape(c["shape"])


# ================================================================================================ automatic configuration
@dataclass
class HardwareConstraints:
    memory_bytes: float = math.inf
    supported_bits: Sequence[int] = (4, 8, 16)
    int_speedup: dict = field(default_factory=lambda: {4: 3.0, 8: 2.0, 16: 1.0})       # throughput against 16-bit
    max_error_db: float = 25.0                                                         # lowest acceptable per-layer SQNR


class AutoConfigurator:
    """Measures every weight matrix at every supported width, then picks per layer the cheapest width whose SQNR clears the
    floor; if the model still exceeds the memory limit, layers are lowered in order of least damage per byte saved.  The
    ``objective`` weighs size against speed against accuracy when several configurations are admissible, and the explored
    configurations form a Pareto front."""

    def __init__(self, constraints: HardwareConstraints | None = None, objective: str = "balanced"): self.c, self.objective = constraints or HardwareConstraints(), objective

    def profile(self, model: nn.Module) -> dict:
        table = {}
        for name, p in model.named_parameters():
            if p.dim() < 2:
                continue
            row = {}
            for b in self.c.supported_bits:
                if b >= 16:
                    row[b] = {"sqnr_db": sqnr_db(p.detach().float(), p.detach().to(torch.bfloat16).float()), "bytes": p.numel() * 2}
                else:
                    q, qp = quantize_per_channel(p.detach().float(), 0, b)
                    row[b] = {"sqnr_db": sqnr_db(p.detach().float(), dequantize(q, qp)), "bytes": p.numel() * b / 8 + p.shape[0] * 4}
            table[name] = row
        return table

    def configure(self, model: nn.Module) -> dict:
        table = self.profile(model)
        bits = sorted(self.c.supported_bits)
        choice = {n: next((b for b in bits if row[b]["sqnr_db"] >= self.c.max_error_db), bits[-1]) for n, row in table.items()}
        if self.objective == "accuracy":
            choice = {n: max(b, 8) if 8 in bits else b for n, b in choice.items()}
        total = lambda ch: sum(table[n][b]["bytes"] for n, b in ch.items())
        relaxed = []
        while total(choice) > self.c.memory_bytes:
            best = None
            for n, b in choice.items():
                lower = [x for x in bits if x < b]
                if not lower:
                    continue
                nb = lower[-1]
                saved, damage = table[n][b]["bytes"] - table[n][nb]["bytes"], max(table[n][b]["sqnr_db"] - table[n][nb]["sqnr_db"], 1e-9)
                if best is None or damage / saved < best[0]:
                    best = (damage / saved, n, nb)
            if best is None:
                break
            choice[best[1]] = best[2]; relaxed.append(best[1])
        size = total(choice)
        speed = sum(table[n][b]["bytes"] for n, b in choice.items()) and sum(table[n][16 if 16 in bits else bits[-1]]["bytes"] for n in choice) / sum(table[n][16 if 16 in bits else bits[-1]]["bytes"] / self.c.int_speedup.get(b, 1.0) for n, b in choice.items())
        return {"bits": choice, "bytes": size, "fits": size <= self.c.memory_bytes, "estimated_speedup": speed, "min_sqnr_db": min(table[n][b]["sqnr_db"] for n, b in choice.items()), "relaxed_layers": relaxed, "table": table}

    def pareto_front(self, model: nn.Module) -> list[dict]:
        """Uniform configurations plus the mixed one, reduced to those not dominated in (bytes, worst SQNR)."""
        table = self.profile(model)
        cands = [{"name": f"uniform-{b}", "bytes": sum(r[b]["bytes"] for r in table.values()), "min_sqnr_db": min(r[b]["sqnr_db"] for r in table.values())} for b in self.c.supported_bits]
        mixed = self.configure(model)
        if not any(c["bytes"] == mixed["bytes"] and c["min_sqnr_db"] == mixed["min_sqnr_db"] for c in cands):      # a mixed result equal to a uniform one adds nothing
            cands.append({"name": "mixed", "bytes": mixed["bytes"], "min_sqnr_db": mixed["min_sqnr_db"]})
        return sorted([c for c in cands if not any(o["bytes"] <= c["bytes"] and o["min_sqnr_db"] >= c["min_sqnr_db"] and (o["bytes"] < c["bytes"] or o["min_sqnr_db"] > c["min_sqnr_db"]) for o in cands)], key=lambda c: c["bytes"])


# ================================================================================================ annealing-based bit allocation
def anneal_bit_allocation(sizes: Sequence[int], sensitivities: Sequence[float], budget_bits: float, choices: Sequence[int] = (2, 4, 8), steps: int = 4000, t0: float = 1.0, t1: float = 1e-3, schedule: str = "exponential", seed: int = 0) -> dict:
    """Minimises ``sum_i sensitivity_i 4^{-bits_i}`` (the noise power of a uniform quantiser) under ``sum size_i bits_i <=
    budget`` by simulated annealing over the discrete widths: a move changes one layer's width; infeasible states pay a
    penalty proportional to the overshoot; the temperature follows an exponential, linear or logarithmic schedule."""
    g = torch.Generator().manual_seed(seed)
    n = len(sizes)
    cost = lambda b: sum(s * 4.0 ** (-x) for s, x in zip(sensitivities, b))
    used = lambda b: sum(s * x for s, x in zip(sizes, b))
    scale = cost([min(choices)] * n) or 1.0
    energy = lambda b: cost(b) / scale + 10.0 * max(0.0, used(b) - budget_bits) / budget_bits
    cur = [min(choices)] * n
    e_cur = energy(cur)
    best, e_best = list(cur), e_cur
    rnd = torch.rand(steps, 2, generator=g).tolist(); pick = torch.randint(0, n, (steps,), generator=g).tolist()
    for k in range(steps):
        frac = k / max(steps - 1, 1)
        T = t0 * (t1 / t0) ** frac if schedule == "exponential" else t0 + (t1 - t0) * frac if schedule == "linear" else t0 / math.log(math.e + 50 * frac)
        i = pick[k]
        new = list(cur); new[i] = choices[int(rnd[k][0] * len(choices))]
        e_new = energy(new)
        if e_new <= e_cur or rnd[k][1] < math.exp(-(e_new - e_cur) / T):
            cur, e_cur = new, e_new
            if e_cur < e_best and used(cur) <= budget_bits:
                best, e_best = list(cur), e_cur
    return {"bits": best, "cost": cost(best), "used_bits": used(best), "feasible": used(best) <= budget_bits, "mean_bits": used(best) / sum(sizes)}
