"""Further evaluation tools (``crates/torsh-metrics/src/{statistical_tests,model_selection,uncertainty,explainability,
robustness,deep_learning,advanced_ml,reporting}.rs``): rank-based and multi-model significance tests with multiple
comparison corrections and effect sizes, small-sample information criteria, uncertainty decomposition for ensembles and
MC dropout, deletion / insertion faithfulness of attributions, robustness curves, continual-learning and recommendation
quality metrics, and report builders (Markdown / LaTeX).  Statistics follow scipy's definitions."""
from __future__ import annotations

import math
from typing import Callable, Sequence

import torch


def _t(x): return torch.as_tensor(x, dtype=torch.float64)


def _rank(x: torch.Tensor) -> torch.Tensor:
    """Average ranks (1-based) with ties sharing their mean rank."""
    order = x.argsort()
    ranks = torch.empty_like(x)
    ranks[order] = torch.arange(1, len(x) + 1, dtype=x.dtype)
    vals, inv, cnt = torch.unique(x, return_inverse=True, return_counts=True)
    sums = torch.zeros(len(vals), dtype=x.dtype).index_add_(0, inv, ranks)
    return (sums / cnt)[inv]


def _norm_sf(z: float) -> float: return 0.5 * math.erfc(z / math.sqrt(2))
def _chi2_sf(x: float, k: float) -> float: return float(torch.special.gammaincc(torch.tensor(k / 2, dtype=torch.float64), torch.tensor(x / 2, dtype=torch.float64)))


# ================================================================================================ tests
def mann_whitney_u(a, b) -> dict:
    """Two-sided, normal approximation with tie and continuity corrections."""
    a, b = _t(a), _t(b)
    n1, n2 = len(a), len(b)
    r = _rank(torch.cat([a, b]))
    u1 = float(r[:n1].sum()) - n1 * (n1 + 1) / 2
    u = min(u1, n1 * n2 - u1)
    _, cnt = torch.unique(torch.cat([a, b]), return_counts=True)
    n = n1 + n2
    sd = math.sqrt(n1 * n2 / 12 * ((n + 1) - float((cnt ** 3 - cnt).sum()) / (n * (n - 1))))
    z = (abs(u1 - n1 * n2 / 2) - 0.5) / sd if sd > 0 else 0.0
    return {"u": u1, "p_value": min(1.0, 2 * _norm_sf(z)), "effect_size": 1 - 2 * u / (n1 * n2)}


def kruskal_wallis(*groups) -> dict:
    gs = [_t(g) for g in groups]
    allv = torch.cat(gs)
    n, r = len(allv), _rank(allv)
    h, s = 0.0, 0
    for g in gs:
        h += float(r[s:s + len(g)].sum()) ** 2 / len(g); s += len(g)
    h = 12 / (n * (n + 1)) * h - 3 * (n + 1)
    _, cnt = torch.unique(allv, return_counts=True)
    h /= 1 - float((cnt ** 3 - cnt).sum()) / (n ** 3 - n)
    return {"statistic": h, "p_value": _chi2_sf(h, len(gs) - 1)}


def friedman_test(scores) -> dict:
    """``scores``: ``[datasets, models]``; ranks inside each row (higher score = better = rank 1 is not assumed: ranks ascend)."""
    x = _t(scores)
    n, k = x.shape
    r = torch.stack([_rank(row) for row in x])
    rbar = r.mean(0)
    ties = sum(float((c ** 3 - c).sum()) for c in (torch.unique(row, return_counts=True)[1] for row in x))
    stat = 12 * n / (k * (k + 1)) * float(((rbar - (k + 1) / 2) ** 2).sum()) / (1 - ties / (n * k * (k * k - 1)))
    return {"statistic": stat, "p_value": _chi2_sf(stat, k - 1), "mean_ranks": rbar}


_NEMENYI_Q05 = {2: 1.960, 3: 2.343, 4: 2.569, 5: 2.728, 6: 2.850, 7: 2.949, 8: 3.031, 9: 3.102, 10: 3.164}


def nemenyi_critical_difference(k: int, n: int) -> float: return _NEMENYI_Q05[k] * math.sqrt(k * (k + 1) / (6 * n))


def nemenyi_test(scores) -> dict:
    f = friedman_test(scores)
    k, n = len(f["mean_ranks"]), len(scores)
    cd = nemenyi_critical_difference(k, n)
    diff = (f["mean_ranks"][:, None] - f["mean_ranks"][None]).abs()
    return {"critical_difference": cd, "mean_ranks": f["mean_ranks"], "significant": diff > cd}


def five_by_two_cv_test(diffs) -> dict:
    """Dietterich's 5x2cv paired t test: ``diffs[i][j]`` is the score difference in fold ``j`` of replication ``i``."""
    d = _t(diffs)
    s2 = ((d - d.mean(1, keepdim=True)) ** 2).sum(1)
    t = float(d[0, 0] / torch.sqrt(s2.mean()))
    from scipy import stats
    return {"t": t, "p_value": float(2 * stats.t.sf(abs(t), 5))}


def multiple_comparison_correction(pvalues, method: str = "holm", alpha: float = 0.05) -> dict:
    p = _t(pvalues)
    m, order = len(p), p.argsort()
    adj = torch.empty_like(p)
    if method == "bonferroni":
        adj = (p * m).clamp(max=1)
    elif method == "holm":
        run = 0.0
        for i, idx in enumerate(order.tolist()):
            run = max(run, float(p[idx]) * (m - i)); adj[idx] = min(run, 1.0)
    elif method in ("fdr_bh", "benjamini_hochberg"):
        run = 1.0
        for i, idx in reversed(list(enumerate(order.tolist()))):
            run = min(run, float(p[idx]) * m / (i + 1)); adj[idx] = run
    else:
        raise ValueError(method)
    return {"adjusted": adj, "reject": adj < alpha}


def effect_size(a, b, kind: str = "cohen_d") -> float:
    a, b = _t(a), _t(b)
    if kind == "cliffs_delta":
        return float((torch.sign(a[:, None] - b[None])).mean())
    na, nb = len(a), len(b)
    sp = math.sqrt(((na - 1) * float(a.var()) + (nb - 1) * float(b.var())) / (na + nb - 2))
    d = float(a.mean() - b.mean()) / sp
    return d * (1 - 3 / (4 * (na + nb) - 9)) if kind == "hedges_g" else d


# ================================================================================================ information criteria
def aicc(log_likelihood: float, k: int, n: int) -> float: return 2 * k - 2 * log_likelihood + 2 * k * (k + 1) / max(n - k - 1, 1)
def hqic(log_likelihood: float, k: int, n: int) -> float: return -2 * log_likelihood + 2 * k * math.log(math.log(n))
def akaike_weights(scores) -> torch.Tensor: s = _t(scores); w = torch.exp(-0.5 * (s - s.min())); return w / w.sum()


# ================================================================================================ uncertainty
def uncertainty_decomposition(probs: torch.Tensor) -> dict:
    """``probs``: ``[members, samples, classes]`` from an ensemble or MC dropout.  Total (entropy of the mean) = aleatoric
    (mean entropy) + epistemic (mutual information between prediction and member)."""
    p = probs.double().clamp(min=1e-12)
    mean = p.mean(0)
    total = -(mean * mean.log()).sum(-1)
    alea = -(p * p.log()).sum(-1).mean(0)
    return {"total": total, "aleatoric": alea, "epistemic": total - alea, "variation_ratio": 1 - torch.stack([(p.argmax(-1) == c).double().mean(0) for c in range(p.shape[-1])]).max(0).values,
            "mean_prediction": mean}


def mc_dropout_predict(model: torch.nn.Module, x: torch.Tensor, samples: int = 20) -> torch.Tensor:
    """Softmax outputs with dropout layers active and everything else in eval mode: ``[samples, N, C]``."""
    was = model.training
    model.eval()
    for m in model.modules():
        if isinstance(m, (torch.nn.Dropout, torch.nn.Dropout1d, torch.nn.Dropout2d, torch.nn.Dropout3d)):
            m.train()
    with torch.no_grad():
        out = torch.stack([model(x).softmax(-1) for _ in range(samples)])
    model.train(was)
    return out


def prediction_interval_coverage(lower, upper, y) -> dict:
    lo, hi, y = _t(lower), _t(upper), _t(y)
    inside = (y >= lo) & (y <= hi)
    return {"coverage": float(inside.double().mean()), "mean_width": float((hi - lo).mean()), "winkler_miss": float((torch.where(y < lo, lo - y, torch.where(y > hi, y - hi, torch.zeros_like(y)))).mean())}


def selective_risk_curve(confidence, correct) -> dict:
    """Risk (error rate) among the most confident fraction, for every coverage; AURC is the area under it."""
    c, ok = _t(confidence), _t(correct)
    order = c.argsort(descending=True)
    err = (1 - ok[order]).cumsum(0) / torch.arange(1, len(c) + 1, dtype=torch.float64)
    return {"coverage": torch.arange(1, len(c) + 1, dtype=torch.float64) / len(c), "risk": err, "aurc": float(err.mean())}


# ================================================================================================ explainability / robustness
def deletion_insertion_curves(model_fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, attribution: torch.Tensor, steps: int = 10, baseline: float = 0.0) -> dict:
    """Deletes (or inserts) features in order of attributed importance and records the model's score; a faithful
    attribution has a low deletion AUC and a high insertion AUC."""
    order = attribution.flatten().argsort(descending=True)
    n = len(order)
    dele, ins = [float(model_fn(x))], [float(model_fn(torch.full_like(x, baseline)))]
    for s in range(1, steps + 1):
        k = int(round(n * s / steps))
        xd, xi = x.clone().flatten(), torch.full_like(x, baseline).flatten()
        xd[order[:k]] = baseline
        xi[order[:k]] = x.flatten()[order[:k]]
        dele.append(float(model_fn(xd.reshape(x.shape)))); ins.append(float(model_fn(xi.reshape(x.shape))))
    auc = lambda v: sum((a + b) / 2 for a, b in zip(v, v[1:])) / steps
    return {"deletion": dele, "insertion": ins, "deletion_auc": auc(dele), "insertion_auc": auc(ins)}


def attribution_sparsity(attribution: torch.Tensor) -> float:
    """Gini index of absolute attributions (0 = uniform, 1 = all mass on one feature)."""
    a = attribution.abs().flatten().double().sort().values
    n = len(a)
    return float(((2 * torch.arange(1, n + 1, dtype=torch.float64) - n - 1) * a).sum() / (n * a.sum().clamp(min=1e-300)))


def robustness_curve(model_fn: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor, y: torch.Tensor, noise_levels: Sequence[float], seed: int = 0) -> dict:
    """Accuracy under Gaussian input noise of growing standard deviation, with the area under the curve and the level
    at which accuracy first drops below half its clean value."""
    g = torch.Generator().manual_seed(seed)
    acc = [float((model_fn(x + s * torch.randn(x.shape, generator=g)).argmax(-1) == y).double().mean()) for s in noise_levels]
    half = next((s for s, a in zip(noise_levels, acc) if a < acc[0] / 2), None)
    return {"levels": list(noise_levels), "accuracy": acc, "auc": sum(acc) / len(acc), "breakdown_level": half}


def prediction_stability(preds: torch.Tensor) -> dict:
    """``preds``: ``[runs, samples]`` class predictions from re-trained models: share of samples all runs agree on and the
    mean pairwise agreement."""
    r = preds.shape[0]
    agree = (preds == preds[0:1]).all(0).double().mean()
    pair = torch.stack([(preds[i] == preds[j]).double().mean() for i in range(r) for j in range(i + 1, r)]).mean() if r > 1 else torch.tensor(1.0)
    return {"unanimous": float(agree), "pairwise_agreement": float(pair)}


# ================================================================================================ continual learning / recommendation
def continual_learning_metrics(acc: torch.Tensor, baseline: torch.Tensor | None = None) -> dict:
    """``acc[i, j]``: accuracy on task ``j`` after training task ``i``.  Average final accuracy, forgetting (best earlier
    minus final), backward transfer, and forward transfer against ``baseline[j]`` (accuracy of an untrained model)."""
    a = acc.double()
    t = a.shape[0]
    final = a[-1]
    forgetting = torch.stack([a[:-1, j].max() - final[j] for j in range(t - 1)]) if t > 1 else torch.zeros(0)
    bwt = torch.stack([final[j] - a[j, j] for j in range(t - 1)]).mean() if t > 1 else torch.tensor(0.0)
    fwt = torch.stack([a[j - 1, j] - baseline[j] for j in range(1, t)]).mean() if baseline is not None and t > 1 else None
    return {"average_accuracy": float(final.mean()), "forgetting": float(forgetting.mean()) if t > 1 else 0.0, "backward_transfer": float(bwt),
            "forward_transfer": float(fwt) if fwt is not None else None, "learning_accuracy": float(a.diagonal().mean())}


def recommendation_quality(recommended: Sequence[Sequence[int]], item_popularity: dict, item_features: torch.Tensor | None = None, catalog_size: int | None = None) -> dict:
    """Catalogue coverage, novelty (mean self-information of recommended items), intra-list diversity (mean pairwise
    cosine distance) and the Gini concentration of exposure."""
    total = sum(item_popularity.values())
    flat = [i for r in recommended for i in r]
    nov = sum(-math.log2(item_popularity.get(i, 1) / total) for i in flat) / max(len(flat), 1)
    out = {"coverage": len(set(flat)) / (catalog_size or len(item_popularity)), "novelty": nov}
    if item_features is not None:
        f = torch.nn.functional.normalize(item_features.double(), dim=1)
        div = []
        for r in recommended:
            if len(r) > 1:
                s = f[list(r)] @ f[list(r)].t()
                div.append(float((1 - s)[~torch.eye(len(r), dtype=torch.bool)].mean()))
        out["diversity"] = sum(div) / max(len(div), 1)
    exp = torch.zeros(catalog_size or (max(item_popularity) + 1), dtype=torch.float64)
    for i in flat:
        exp[i] += 1
    out["exposure_gini"] = attribution_sparsity(exp)
    return out


# ================================================================================================ reports
class ReportBuilder:
    """Collects named metric tables and renders Markdown or LaTeX (``booktabs``), bolding the best value per column."""

    def __init__(self, title: str = "Evaluation"): self.title, self.tables = title, []

    def add_table(self, name: str, rows: dict[str, dict[str, float]], higher_is_better: dict[str, bool] | None = None, fmt: str = "{:.3f}"):
        self.tables.append((name, rows, higher_is_better or {}, fmt))
        return self

    def _best(self, rows, col, hib): vals = {r: v[col] for r, v in rows.items() if col in v}; return (max if hib.get(col, True) else min)(vals, key=vals.get)

    def to_markdown(self) -> str:
        out = [f"# {self.title}", ""]
        for name, rows, hib, fmt in self.tables:
            cols = list(dict.fromkeys(c for v in rows.values() for c in v))
            out += [f"## {name}", "", "| model | " + " | ".join(cols) + " |", "|---|" + "---|" * len(cols)]
            for r, v in rows.items():
                out.append(f"| {r} | " + " | ".join((f"**{fmt.format(v[c])}**" if self._best(rows, c, hib) == r else fmt.format(v[c])) if c in v else "-" for c in cols) + " |")
            out.append("")
        return "\n".join(out)

    def to_latex(self) -> str:
        esc = lambda s: str(s).replace("_", r"\_").replace("%", r"\%").replace("&", r"\&")
        out = []
        for name, rows, hib, fmt in self.tables:
            cols = list(dict.fromkeys(c for v in rows.values() for c in v))
            out += [r"\begin{table}[t]", r"\centering", rf"\caption{{{esc(name)}}}", r"\begin{tabular}{l" + "r" * len(cols) + "}", r"\toprule", "model & " + " & ".join(map(esc, cols)) + r" \\", r"\midrule"]
            for r, v in rows.items():
                cells = [(rf"\textbf{{{fmt.format(v[c])}}}" if self._best(rows, c, hib) == r else fmt.format(v[c])) if c in v else "--" for c in cols]
                out.append(esc(r) + " & " + " & ".join(cells) + r" \\")
            out += [r"\bottomrule", r"\end{tabular}", r"\end{table}", ""]
        return "\n".join(out)
