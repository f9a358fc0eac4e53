"""Further evaluation metrics: classification (MCC, kappa, balanced accuracy, average precision, log loss, Brier), ranking
(MAP, MRR, precision / recall / hit rate at k), regression diagnostics, uncertainty calibration, time-series forecast
errors, model selection criteria and k-fold splits, distribution distances for generative models, streaming (online)
accumulators, and statistical tests for comparing models. Tensors in, Python floats / tensors out.
Reference: crates/torsh-metrics/src/{classification,ranking,regression_diagnostics,uncertainty,time_series,model_selection,
deep_learning,streaming,statistical_tests,statistics,sklearn_compat}.rs.
"""
from __future__ import annotations

import math

import torch

from .metrics import confusion_matrix


# ---- classification --------------------------------------------------------------------------------------------------
def matthews_corrcoef(pred, target, num_classes: int | None = None) -> float:
    c = confusion_matrix(pred, target, num_classes or int(max(pred.max(), target.max())) + 1).double()
    t, p, n, diag = c.sum(1), c.sum(0), c.sum(), c.diag().sum()
    den = torch.sqrt((n * n - (p * p).sum()) * (n * n - (t * t).sum()))
    return float((diag * n - (t * p).sum()) / den) if den > 0 else 0.0


def cohen_kappa(pred, target, num_classes: int | None = None) -> float:
    c = confusion_matrix(pred, target, num_classes or int(max(pred.max(), target.max())) + 1).double()
    n = c.sum()
    po, pe = c.diag().sum() / n, (c.sum(0) * c.sum(1)).sum() / (n * n)
    return float((po - pe) / (1 - pe)) if pe < 1 else 0.0


def balanced_accuracy(pred, target, num_classes: int | None = None) -> float:
    c = confusion_matrix(pred, target, num_classes or int(max(pred.max(), target.max())) + 1).double()
    support = c.sum(1)
    rec = c.diag()[support > 0] / support[support > 0]
    return float(rec.mean())


def average_precision(scores, target) -> float:
    """Area under the precision-recall curve as the step-wise sum used by scikit-learn."""
    order = torch.argsort(scores.double(), descending=True, stable=True)
    t, s = target[order].double(), scores[order].double()
    tp = t.cumsum(0)
    prec = tp / torch.arange(1, len(t) + 1, dtype=torch.float64)
    last_of_tie = torch.cat([s[1:] != s[:-1], torch.tensor([True])])       # evaluate at distinct thresholds only
    rec = tp[last_of_tie] / t.sum().clamp(min=1)
    prec = prec[last_of_tie]
    return float((torch.diff(rec, prepend=torch.zeros(1, dtype=torch.float64)) * prec).sum())


def log_loss(probs, target, eps: float = 1e-15) -> float:
    p = probs.double().clamp(eps, 1 - eps)
    if p.dim() == 1:
        t = target.double()
        return float(-(t * p.log() + (1 - t) * (1 - p).log()).mean())
    p = p / p.sum(-1, keepdim=True)
    return float(-p.gather(1, target.long()[:, None]).log().mean())


def brier_score(probs, target) -> float:
    return float(((probs.double() - target.double()) ** 2).mean())


# ---- ranking ---------------------------------------------------------------------------------------------------------
def precision_at_k(ranked_relevance, k: int) -> float:
    return float(ranked_relevance[:k].double().sum() / k)


def recall_at_k(ranked_relevance, k: int, total_relevant: int | None = None) -> float:
    tot = total_relevant if total_relevant is not None else int(ranked_relevance.sum())
    return float(ranked_relevance[:k].double().sum() / tot) if tot else 0.0


def hit_rate_at_k(ranked_relevance, k: int) -> float:
    return float(ranked_relevance[:k].any())


def reciprocal_rank(ranked_relevance) -> float:
    nz = ranked_relevance.nonzero()
    return 1.0 / (int(nz[0]) + 1) if len(nz) else 0.0


def mean_reciprocal_rank(queries) -> float:
    return sum(reciprocal_rank(q) for q in queries) / len(queries)


def average_precision_at_k(ranked_relevance, k: int | None = None) -> float:
    r = ranked_relevance[:k].double() if k else ranked_relevance.double()
    if r.sum() == 0:
        return 0.0
    prec = r.cumsum(0) / torch.arange(1, len(r) + 1, dtype=torch.float64)
    return float((prec * r).sum() / r.sum())


def mean_average_precision(queries, k: int | None = None) -> float:
    return sum(average_precision_at_k(q, k) for q in queries) / len(queries)


# ---- regression diagnostics --------------------------------------------------------------------------------------------
def adjusted_r2(pred, target, n_features: int) -> float:
    t = target.double()
    r2 = 1 - ((t - pred.double()) ** 2).sum() / ((t - t.mean()) ** 2).sum()
    n = t.numel()
    return float(1 - (1 - r2) * (n - 1) / (n - n_features - 1))


def mape(pred, target) -> float:
    return float(((target.double() - pred.double()).abs() / target.double().abs().clamp(min=1e-12)).mean())


def smape(pred, target) -> float:
    p, t = pred.double(), target.double()
    return float((2 * (p - t).abs() / (p.abs() + t.abs()).clamp(min=1e-12)).mean())


def explained_variance(pred, target) -> float:
    t, r = target.double(), target.double() - pred.double()
    return float(1 - r.var(unbiased=False) / t.var(unbiased=False))


def durbin_watson(residuals) -> float:
    r = residuals.double()
    return float((r[1:] - r[:-1]).pow(2).sum() / r.pow(2).sum())


def residual_diagnostics(pred, target) -> dict:
    r = target.double() - pred.double()
    z = (r - r.mean()) / r.std(unbiased=False).clamp(min=1e-12)
    return {"mean": float(r.mean()), "std": float(r.std()), "skewness": float((z ** 3).mean()), "excess_kurtosis": float((z ** 4).mean() - 3),
            "durbin_watson": durbin_watson(r), "max_abs": float(r.abs().max())}


# ---- uncertainty -----------------------------------------------------------------------------------------------------
def calibration_error(confidences, correct, n_bins: int = 15, norm: str = "l1") -> float:
    """Expected (l1) or maximum (max) calibration error over equal-width confidence bins."""
    conf, corr = confidences.double(), correct.double()
    edges = torch.linspace(0, 1, n_bins + 1, dtype=torch.float64)
    ece, mce = 0.0, 0.0
    for lo, hi in zip(edges[:-1], edges[1:]):
        m = (conf > lo) & (conf <= hi) if lo > 0 else (conf >= lo) & (conf <= hi)
        if m.any():
            gap = float((corr[m].mean() - conf[m].mean()).abs())
            ece += gap * float(m.double().mean())
            mce = max(mce, gap)
    return ece if norm == "l1" else mce


def interval_coverage(lower, upper, target) -> float:
    return float(((target >= lower) & (target <= upper)).double().mean())


def interval_sharpness(lower, upper) -> float:
    return float((upper - lower).double().mean())


def gaussian_nll(mean, var, target) -> float:
    v = var.double().clamp(min=1e-12)
    return float((0.5 * (torch.log(2 * math.pi * v) + (target.double() - mean.double()) ** 2 / v)).mean())


def predictive_entropy(probs) -> torch.Tensor:
    p = probs.double().clamp(min=1e-12)
    return -(p * p.log()).sum(-1)


def mutual_information(mc_probs) -> torch.Tensor:
    """BALD: entropy of the mean prediction minus the mean entropy, for ``[samples, N, C]`` Monte-Carlo predictions."""
    return predictive_entropy(mc_probs.mean(0)) - predictive_entropy(mc_probs).mean(0)


# ---- time series -----------------------------------------------------------------------------------------------------
def mase(pred, target, train, season: int = 1) -> float:
    scale = (train[season:].double() - train[:-season].double()).abs().mean()
    return float((target.double() - pred.double()).abs().mean() / scale.clamp(min=1e-12))


def directional_accuracy(pred, target) -> float:
    return float((torch.sign(pred[1:] - target[:-1]) == torch.sign(target[1:] - target[:-1])).double().mean())


def theil_u(pred, target) -> float:
    p, t = pred.double(), target.double()
    return float(torch.sqrt(((p - t) ** 2).mean()) / (torch.sqrt((p ** 2).mean()) + torch.sqrt((t ** 2).mean())))


# ---- model selection ---------------------------------------------------------------------------------------------------
def aic(log_likelihood: float, n_params: int) -> float:
    return 2 * n_params - 2 * log_likelihood


def bic(log_likelihood: float, n_params: int, n_samples: int) -> float:
    return n_params * math.log(n_samples) - 2 * log_likelihood


def k_fold_indices(n: int, k: int, shuffle: bool = True, seed: int = 0):
    """List of (train indices, validation indices); fold sizes differ by at most one."""
    idx = torch.randperm(n, generator=torch.Generator().manual_seed(seed)) if shuffle else torch.arange(n)
    sizes = [n // k + (1 if i < n % k else 0) for i in range(k)]
    out, s = [], 0
    for sz in sizes:
        val = idx[s:s + sz]
        out.append((torch.cat([idx[:s], idx[s + sz:]]), val))
        s += sz
    return out


def stratified_k_fold_indices(labels, k: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    folds = [[] for _ in range(k)]
    for c in labels.unique():
        members = (labels == c).nonzero().flatten()
        members = members[torch.randperm(len(members), generator=g)]
        for i, m in enumerate(members.tolist()):
            folds[i % k].append(m)
    allidx = set(range(len(labels)))
    return [(torch.tensor(sorted(allidx - set(f))), torch.tensor(sorted(f))) for f in folds]


# ---- generative-model distances ----------------------------------------------------------------------------------------
def frechet_distance(feat_a, feat_b) -> float:
    """|mu_a - mu_b|^2 + Tr(S_a + S_b - 2 (S_a S_b)^(1/2)) between Gaussians fitted to two feature sets (the FID formula)."""
    a, b = feat_a.double(), feat_b.double()
    mu_a, mu_b = a.mean(0), b.mean(0)
    sa, sb = torch.cov(a.T), torch.cov(b.T)
    ev = torch.linalg.eigvals(sa @ sb)
    tr_sqrt = ev.sqrt().real.sum()
    return float(((mu_a - mu_b) ** 2).sum() + sa.trace() + sb.trace() - 2 * tr_sqrt)


def inception_score(probs) -> float:
    p = probs.double().clamp(min=1e-12)
    py = p.mean(0, keepdim=True)
    return float(torch.exp((p * (p.log() - py.log())).sum(1).mean()))


# ---- streaming accumulators ----------------------------------------------------------------------------------------------
class RunningMoments:
    """Welford / Chan update of count, mean and variance over batches; ``merge`` combines two accumulators (ranks)."""

    def __init__(self):
        self.n, self.mean, self.m2 = 0, 0.0, 0.0

    def update(self, x):
        x = torch.as_tensor(x).double().flatten()
        nb = x.numel()
        if nb == 0:
            return self
        mb, m2b = float(x.mean()), float(((x - x.mean()) ** 2).sum())
        d = mb - self.mean
        tot = self.n + nb
        self.m2 += m2b + d * d * self.n * nb / tot
        self.mean += d * nb / tot
        self.n = tot
        return self

    def merge(self, o: "RunningMoments"):
        if o.n:
            d, tot = o.mean - self.mean, self.n + o.n
            self.m2 += o.m2 + d * d * self.n * o.n / tot
            self.mean += d * o.n / tot
            self.n = tot
        return self

    @property
    def variance(self): return self.m2 / (self.n - 1) if self.n > 1 else 0.0
    @property
    def std(self): return math.sqrt(self.variance)


class StreamingConfusion:
    def __init__(self, num_classes: int):
        self.c = torch.zeros(num_classes, num_classes, dtype=torch.long)

    def update(self, pred, target):
        k = self.c.shape[0]
        self.c += torch.bincount(target.long() * k + pred.long(), minlength=k * k).reshape(k, k)
        return self

    def accuracy(self) -> float: return float(self.c.diag().sum() / self.c.sum().clamp(min=1))

    def f1_macro(self) -> float:
        tp, fp, fn = self.c.diag().double(), self.c.sum(0).double() - self.c.diag(), self.c.sum(1).double() - self.c.diag()
        f1 = 2 * tp / (2 * tp + fp + fn).clamp(min=1)
        return float(f1.mean())


class StreamingAUC:
    """ROC AUC from per-class score histograms (fixed memory); exact up to ties within a bin."""

    def __init__(self, bins: int = 1024):
        self.bins = bins
        self.pos, self.neg = torch.zeros(bins, dtype=torch.float64), torch.zeros(bins, dtype=torch.float64)

    def update(self, scores, target):
        b = (scores.double().clamp(0, 1) * (self.bins - 1)).round().long()
        t = target.bool()
        self.pos += torch.bincount(b[t], minlength=self.bins)
        self.neg += torch.bincount(b[~t], minlength=self.bins)
        return self

    def compute(self) -> float:
        neg_below = self.neg.cumsum(0) - self.neg
        u = (self.pos * (neg_below + 0.5 * self.neg)).sum()
        return float(u / (self.pos.sum() * self.neg.sum()).clamp(min=1))


# ---- statistical tests -------------------------------------------------------------------------------------------------
def paired_t_test(a, b) -> dict:
    from ..special_functions import student_t_cdf
    d = a.double() - b.double()
    n = d.numel()
    t = float(d.mean() / (d.std() / math.sqrt(n)).clamp(min=1e-300))
    p = 2 * (1 - float(student_t_cdf(torch.tensor(abs(t)), float(n - 1))))
    return {"t": t, "df": n - 1, "p_value": p}


def mcnemar_test(correct_a, correct_b) -> dict:
    """Continuity-corrected McNemar chi-square on the discordant pairs of two classifiers' per-example correctness."""
    from ..special_functions import chi2_cdf
    b = int((correct_a.bool() & ~correct_b.bool()).sum())
    c = int((~correct_a.bool() & correct_b.bool()).sum())
    if b + c == 0:
        return {"statistic": 0.0, "p_value": 1.0, "b": b, "c": c}
    stat = (abs(b - c) - 1) ** 2 / (b + c)
    return {"statistic": stat, "p_value": 1 - float(chi2_cdf(torch.tensor(stat), 1.0)), "b": b, "c": c}


def wilcoxon_signed_rank(a, b) -> dict:
    """Normal approximation with tie and zero handling (zeros dropped, average ranks)."""
    from ..special_functions import norm_cdf
    d = (a.double() - b.double())
    d = d[d != 0]
    n = d.numel()
    if n == 0:
        return {"statistic": 0.0, "p_value": 1.0}
    order = d.abs().argsort()
    ranks = torch.empty(n, dtype=torch.float64)
    sorted_abs = d.abs()[order]
    i = 0
    while i < n:
        j = i
        while j + 1 < n and sorted_abs[j + 1] == sorted_abs[i]:
            j += 1
        ranks[order[i:j + 1]] = (i + j) / 2 + 1
        i = j + 1
    w_plus, w_minus = float(ranks[d > 0].sum()), float(ranks[d < 0].sum())
    w = min(w_plus, w_minus)
    mu, sigma = n * (n + 1) / 4, math.sqrt(n * (n + 1) * (2 * n + 1) / 24)
    z = (w - mu) / sigma
    return {"statistic": w, "z": z, "p_value": 2 * float(norm_cdf(torch.tensor(z)))}


def bootstrap_ci(values, stat=torch.mean, n_boot: int = 2000, alpha: float = 0.05, seed: int = 0) -> tuple:
    g = torch.Generator().manual_seed(seed)
    v = values.double()
    idx = torch.randint(0, len(v), (n_boot, len(v)), generator=g)
    stats = torch.stack([stat(v[i]) for i in idx])
    lo, hi = torch.quantile(stats, torch.tensor([alpha / 2, 1 - alpha / 2], dtype=torch.float64))
    return float(lo), float(hi)


def permutation_test(a, b, n_perm: int = 5000, seed: int = 0) -> float:
    """Two-sided p-value for a difference in means between two independent samples."""
    g = torch.Generator().manual_seed(seed)
    a, b = a.double(), b.double()
    obs = abs(float(a.mean() - b.mean()))
    pool, na = torch.cat([a, b]), len(a)
    count = 0
    for _ in range(n_perm):
        p = pool[torch.randperm(len(pool), generator=g)]
        count += abs(float(p[:na].mean() - p[na:].mean())) >= obs - 1e-15
    return (count + 1) / (n_perm + 1)


# ---- scikit-learn style scorers ----------------------------------------------------------------------------------------
def make_scorer(metric, greater_is_better: bool = True, needs_proba: bool = False):
    """``scorer(model, X, y)`` in scikit-learn's convention (higher is better after the sign flip)."""
    sign = 1.0 if greater_is_better else -1.0

    def scorer(model, X, y):
        with torch.no_grad():
            out = model(X)
        pred = out if needs_proba else (out.argmax(-1) if out.dim() > 1 else out)
        return sign * float(metric(pred, y))
    return scorer
