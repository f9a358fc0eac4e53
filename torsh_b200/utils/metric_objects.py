"""Stateful metric objects (``crates/torsh-metrics/src/{lib,classification,regression,ranking,clustering,uncertainty,
fairness,streaming,memory_efficient,statistics,statistical_tests,model_selection,advanced_ml,visualization,reporting}.rs``).

Every metric follows ``update(batch...)`` / ``compute()`` / ``reset()``.  The state is a small set of sufficient
statistics held as tensors on the device of the first batch (confusion counts, sums, sorted-score histograms), so an
evaluation loop accumulates with no host synchronisation per batch and reads one scalar back at the end; this is also what
makes the same objects serve as the streaming, chunked and data-parallel variants (``merge`` adds the states of two
ranks, ``sync`` all-reduces them over a process group).  Function-style implementations live in ``metrics``,
``metrics_ext`` and ``metrics_more``; the classes below reuse them where the metric is not decomposable."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch

from . import metrics as _m
from . import metrics_ext as _x
from . import metrics_more as _mm

__all__ = [
    "Metric", "MetricCollection", "Accuracy", "TopKAccuracy", "ConfusionMatrix", "Precision", "Recall", "F1Score",
    "MultiClassMetrics", "ThresholdMetrics", "MSE", "RMSE", "MAE", "MAPE", "SMAPE", "R2Score", "ExplainedVariance",
    "HuberLoss", "LogCoshLoss", "QuantileLoss", "NDCG", "MeanAveragePrecision", "MeanReciprocalRank", "PrecisionAtK",
    "RecallAtK", "F1AtK", "HitRateAtK", "RankingAUC", "Coverage", "Diversity", "Novelty", "SilhouetteScore",
    "DaviesBouldin", "CalinskiHarabasz", "AdjustedRandIndex", "NormalizedMutualInfo", "DunnIndex", "VMeasure", "Inertia",
    "Perplexity", "ExpectedCalibrationError", "MaximumCalibrationError", "BrierScore", "PredictionIntervalCoverage",
    "ReliabilityDiagram", "EntropyMeasures", "EnsembleUncertainty", "DemographicParity", "EqualizedOdds",
    "GroupCalibration", "IndividualFairness", "BiasAmplification", "FairnessMetrics", "StreamingAccuracy",
    "StreamingConfusionMatrix", "StreamingAUROC", "StreamingStats", "StreamingMetricCollection", "ChunkedEvaluator",
    "HypothesisTestResult", "PairedTTest", "McNemarTest", "WilcoxonTest", "FriedmanTest", "NemenyiTest",
    "MannWhitneyTest", "KruskalWallisTest", "FiveByTwoCVTest", "PermutationTest", "BootstrapCI", "EffectSize",
    "MultipleComparisonCorrection", "CrossValidator", "StabilityAnalyzer", "AIC", "AICc", "BIC", "HQIC",
    "MultiModelComparison", "FewShotMetrics", "MetaLearningMetrics", "DomainAdaptationMetrics",
    "ContinualLearningMetrics", "ConfusionMatrixPlot", "ROCCurvePlot", "PRCurvePlot", "LearningCurvePlot",
    "CalibrationCurvePlot", "FeatureImportancePlot", "MetricComparisonPlot", "LatexReportBuilder", "ExperimentTracker",
]


class Metric:
    """Base: subclasses declare their state in ``_init_state`` as tensors registered through ``_add``."""
    name = "metric"
    higher_is_better = True

    def __init__(self):
        self._state: dict[str, torch.Tensor] = {}
        self._defaults: dict[str, torch.Tensor] = {}
        self._init_state()

    def _init_state(self): ...

    def _add(self, key: str, value: torch.Tensor):
        self._defaults[key] = value.clone()
        self._state[key] = value.clone()

    def _acc(self, key: str, value: torch.Tensor):
        cur = self._state[key]
        if cur.device != value.device:
            cur = cur.to(value.device)
        self._state[key] = cur + value.to(cur.dtype)

    def reset(self):
        self._state = {k: v.clone() for k, v in self._defaults.items()}
        return self

    def merge(self, other: "Metric"):
        for k, v in other._state.items():
            self._state[k] = self._state[k] + v.to(self._state[k].device)
        return self

    def sync(self, group=None):
        """Sums the state over a process group (no-op outside ``torch.distributed``)."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            for v in self._state.values():
                dist.all_reduce(v, group=group)
        return self

    def update(self, *a, **k): raise NotImplementedError
    def compute(self): raise NotImplementedError

    def __call__(self, *a, **k):
        """Batch value: the metric of this batch alone, while still accumulating it."""
        saved = {k_: v.clone() for k_, v in self._state.items()}
        self.reset()
        self.update(*a, **k)
        out = self.compute()
        for k_, v in saved.items():
            self._state[k_] = self._state[k_] + v.to(self._state[k_].device)
        return out


class MetricCollection:
    """Named metrics updated with the same arguments; ``compute`` returns a flat dict (dict-valued metrics are prefixed)."""
    def __init__(self, metrics: dict[str, Metric] | Sequence[Metric]):
        self.metrics = dict(metrics) if isinstance(metrics, dict) else {type(m).__name__: m for m in metrics}

    def add(self, name: str, metric: Metric):
        self.metrics[name] = metric
        return self

    def update(self, *a, **k):
        for m in self.metrics.values():
            m.update(*a, **k)

    def compute(self) -> dict:
        out = {}
        for n, m in self.metrics.items():
            v = m.compute()
            if isinstance(v, dict):
                out.update({f"{n}/{k}": x for k, x in v.items()})
            else:
                out[n] = v
        return out

    def reset(self):
        for m in self.metrics.values():
            m.reset()

    def sync(self, group=None):
        for m in self.metrics.values():
            m.sync(group)
        return self


# ================================================================================================ classification
def _labels(pred: torch.Tensor, target: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    if pred.dim() > target.dim():
        return pred.argmax(-1)
    if pred.is_floating_point():
        return (pred > threshold).long()
    return pred


class Accuracy(Metric):
    name = "accuracy"
    def __init__(self, threshold: float = 0.5):
        self.threshold = threshold
        super().__init__()
    def _init_state(self):
        self._add("correct", torch.zeros((), dtype=torch.float64))
        self._add("total", torch.zeros((), dtype=torch.float64))
    def update(self, pred, target):
        lab = _labels(pred, target, self.threshold)
        self._acc("correct", (lab == target).sum())
        self._acc("total", torch.tensor(float(target.numel()), device=target.device))
    def compute(self) -> float: return float(self._state["correct"] / self._state["total"].clamp(min=1))


class TopKAccuracy(Accuracy):
    def __init__(self, k: int = 5):
        self.k = k
        super().__init__()
    def update(self, logits, target):
        hit = (logits.topk(self.k, -1).indices == target.unsqueeze(-1)).any(-1)
        self._acc("correct", hit.sum())
        self._acc("total", torch.tensor(float(target.numel()), device=target.device))


class ConfusionMatrix(Metric):
    """Rows are the true class, columns the predicted one."""
    name = "confusion_matrix"
    def __init__(self, num_classes: int, threshold: float = 0.5):
        self.num_classes, self.threshold = num_classes, threshold
        super().__init__()
    def _init_state(self): self._add("cm", torch.zeros(self.num_classes, self.num_classes, dtype=torch.float64))
    def update(self, pred, target): self._acc("cm", _m.confusion_matrix(_labels(pred, target, self.threshold), target, self.num_classes))
    def compute(self) -> torch.Tensor: return self._state["cm"].clone()
    def normalized(self, over: str = "true") -> torch.Tensor:
        cm = self._state["cm"]
        return cm / cm.sum(1 if over == "true" else 0, keepdim=True).clamp(min=1) if over in ("true", "pred") else cm / cm.sum().clamp(min=1)

    def per_class(self) -> dict:
        cm = self._state["cm"]
        tp = cm.diag()
        fp, fn = cm.sum(0) - tp, cm.sum(1) - tp
        tn = cm.sum() - tp - fp - fn
        prec, rec = tp / (tp + fp).clamp(min=1), tp / (tp + fn).clamp(min=1)
        return {"precision": prec, "recall": rec, "f1": 2 * prec * rec / (prec + rec).clamp(min=1e-12), "specificity": tn / (tn + fp).clamp(min=1), "support": cm.sum(1)}


class _PRF(ConfusionMatrix):
    which = "precision"
    def __init__(self, num_classes: int = 2, average: str = "macro", threshold: float = 0.5):
        self.average = average
        super().__init__(num_classes, threshold)

    def compute(self):
        pc = self.per_class()
        v, support = pc[self.which], pc["support"]
        if self.average == "none":
            return v
        if self.average == "binary":
            return float(v[1])
        if self.average == "micro":
            cm = self._state["cm"]
            return float(cm.diag().sum() / cm.sum().clamp(min=1))
        if self.average == "weighted":
            return float((v * support).sum() / support.sum().clamp(min=1))
        return float(v.mean())


class Precision(_PRF): which, name = "precision", "precision"
class Recall(_PRF): which, name = "recall", "recall"
class F1Score(_PRF): which, name = "f1", "f1"


class MultiClassMetrics(ConfusionMatrix):
    def compute(self) -> dict:
        cm, pc = self._state["cm"], self.per_class()
        n = cm.sum().clamp(min=1)
        po = cm.diag().sum() / n
        pe = (cm.sum(0) * cm.sum(1)).sum() / n ** 2
        t, p = cm.sum(1), cm.sum(0)
        cov = cm.diag().sum() * n - (t * p).sum()
        mcc = cov / (torch.sqrt((n ** 2 - (p ** 2).sum()) * (n ** 2 - (t ** 2).sum()))).clamp(min=1e-12)
        return {"accuracy": float(po), "balanced_accuracy": float(pc["recall"].mean()), "macro_precision": float(pc["precision"].mean()),
                "macro_recall": float(pc["recall"].mean()), "macro_f1": float(pc["f1"].mean()),
                "weighted_f1": float((pc["f1"] * pc["support"]).sum() / n), "cohen_kappa": float((po - pe) / (1 - pe).clamp(min=1e-12)), "mcc": float(mcc)}


class ThresholdMetrics(Metric):
    """Binary scores binned into ``bins`` equal-width score buckets (exact when scores take few values): ROC and
    precision-recall curves, their areas, and the threshold that maximises F1 or Youden's J, all from two histograms."""
    name = "threshold_metrics"
    def __init__(self, bins: int = 1000):
        self.bins = bins
        super().__init__()
    def _init_state(self):
        self._add("pos", torch.zeros(self.bins, dtype=torch.float64))
        self._add("neg", torch.zeros(self.bins, dtype=torch.float64))

    def update(self, scores, target):
        b = (scores.double().clamp(0, 1) * (self.bins - 1)).round().long().reshape(-1)
        t = target.reshape(-1).bool()
        self._acc("pos", torch.bincount(b[t], minlength=self.bins))
        self._acc("neg", torch.bincount(b[~t], minlength=self.bins))

    def _cum(self):
        pos, neg = self._state["pos"], self._state["neg"]
        tp = pos.flip(0).cumsum(0)                                   # predicted positive when score >= threshold, high to low
        fp = neg.flip(0).cumsum(0)
        return tp, fp, pos.sum(), neg.sum()

    def roc_curve(self):
        tp, fp, P, N = self._cum()
        z = torch.zeros(1, dtype=torch.float64, device=tp.device)
        return torch.cat([z, fp / N.clamp(min=1)]), torch.cat([z, tp / P.clamp(min=1)])

    def pr_curve(self):
        tp, fp, P, _ = self._cum()
        keep = (tp + fp) > 0
        return (tp / P.clamp(min=1))[keep], (tp / (tp + fp).clamp(min=1))[keep]

    def auroc(self) -> float:
        """Trapezoid over the binned curve; ties inside a bin count one half, as the rank statistic does."""
        fpr, tpr = self.roc_curve()
        return float(torch.trapezoid(tpr, fpr))

    def average_precision(self) -> float:
        rec, prec = self.pr_curve()
        prev = torch.cat([torch.zeros(1, dtype=torch.float64, device=rec.device), rec[:-1]])
        return float(((rec - prev) * prec).sum())

    def best_threshold(self, criterion: str = "f1") -> tuple[float, float]:
        tp, fp, P, N = self._cum()
        thr = torch.linspace(0, 1, self.bins, dtype=torch.float64).flip(0)
        if criterion == "f1":
            score = 2 * tp / (tp + fp + P).clamp(min=1)
        else:
            score = tp / P.clamp(min=1) - fp / N.clamp(min=1)
        i = int(score.argmax())
        return float(thr[i]), float(score[i])

    def compute(self) -> dict:
        return {"auroc": self.auroc(), "average_precision": self.average_precision(), "best_f1": self.best_threshold("f1")[1]}


# ================================================================================================ regression
class _SumMetric(Metric):
    """Mean of a per-element quantity."""
    higher_is_better = False
    def _init_state(self):
        self._add("sum", torch.zeros((), dtype=torch.float64))
        self._add("n", torch.zeros((), dtype=torch.float64))
    def _elem(self, p, t): raise NotImplementedError
    def update(self, pred, target):
        self._acc("sum", self._elem(pred.double(), target.double()).sum())
        self._acc("n", torch.tensor(float(target.numel()), device=target.device))
    def compute(self) -> float: return float(self._state["sum"] / self._state["n"].clamp(min=1))


class MSE(_SumMetric):
    name = "mse"
    def _elem(self, p, t): return (p - t) ** 2
class RMSE(MSE):
    name = "rmse"
    def compute(self) -> float: return math.sqrt(super().compute())
class MAE(_SumMetric):
    name = "mae"
    def _elem(self, p, t): return (p - t).abs()
class MAPE(_SumMetric):
    name = "mape"
    def _elem(self, p, t): return ((p - t) / t.abs().clamp(min=1e-12)).abs() * 100
class SMAPE(_SumMetric):
    name = "smape"
    def _elem(self, p, t): return 200 * (p - t).abs() / (p.abs() + t.abs()).clamp(min=1e-12)
class HuberLoss(_SumMetric):
    name = "huber"
    def __init__(self, delta: float = 1.0):
        self.delta = delta
        super().__init__()
    def _elem(self, p, t):
        r = (p - t).abs()
        return torch.where(r <= self.delta, 0.5 * r ** 2, self.delta * (r - 0.5 * self.delta))
class LogCoshLoss(_SumMetric):
    name = "log_cosh"
    def _elem(self, p, t):
        r = (p - t).abs()
        return r + torch.nn.functional.softplus(-2 * r) - math.log(2)
class QuantileLoss(_SumMetric):
    name = "pinball"
    def __init__(self, quantile: float = 0.5):
        self.q = quantile
        super().__init__()
    def _elem(self, p, t):
        d = t - p
        return torch.maximum(self.q * d, (self.q - 1) * d)


class R2Score(Metric):
    """From running sums of ``t``, ``t^2`` and squared residuals; ``adjusted(num_features)`` applies the usual correction."""
    name = "r2"
    def _init_state(self):
        for k in ("n", "st", "stt", "sse", "sr"):
            self._add(k, torch.zeros((), dtype=torch.float64))
    def update(self, pred, target):
        p, t = pred.double().reshape(-1), target.double().reshape(-1)
        self._acc("n", torch.tensor(float(len(t)), device=t.device))
        self._acc("st", t.sum()); self._acc("stt", (t * t).sum()); self._acc("sse", ((p - t) ** 2).sum()); self._acc("sr", (t - p).sum())
    def compute(self) -> float:
        s = self._state
        return float(1 - s["sse"] / (s["stt"] - s["st"] ** 2 / s["n"]).clamp(min=1e-300))
    def adjusted(self, num_features: int) -> float:
        n = float(self._state["n"])
        return 1 - (1 - self.compute()) * (n - 1) / (n - num_features - 1)


class ExplainedVariance(R2Score):
    name = "explained_variance"
    def compute(self) -> float:
        s = self._state
        var_res = s["sse"] / s["n"] - (s["sr"] / s["n"]) ** 2
        var_t = s["stt"] / s["n"] - (s["st"] / s["n"]) ** 2
        return float(1 - var_res / var_t.clamp(min=1e-300))


# ================================================================================================ ranking
class _QueryMetric(Metric):
    """Mean over queries of a per-query value; ``update(scores (Q, N), relevance (Q, N))`` (one query when 1-D)."""
    def __init__(self, k: int | None = None):
        self.k = k
        super().__init__()
    def _init_state(self):
        self._add("sum", torch.zeros((), dtype=torch.float64))
        self._add("n", torch.zeros((), dtype=torch.float64))
    def _per_query(self, rel_sorted: torch.Tensor, rel: torch.Tensor) -> torch.Tensor: raise NotImplementedError
    def update(self, scores, relevance):
        s, r = scores.reshape(-1, scores.shape[-1]).double(), relevance.reshape(-1, relevance.shape[-1]).double()
        order = s.argsort(dim=1, descending=True, stable=True)
        v = self._per_query(r.gather(1, order), r)
        self._acc("sum", v.sum())
        self._acc("n", torch.tensor(float(len(v)), device=v.device))
    def compute(self) -> float: return float(self._state["sum"] / self._state["n"].clamp(min=1))


def _topk(x: torch.Tensor, k: int | None) -> torch.Tensor: return x if k is None else x[:, :k]


class NDCG(_QueryMetric):
    name = "ndcg"
    def __init__(self, k: int | None = None, exponential: bool = True):
        self.exp = exponential
        super().__init__(k)
    def _dcg(self, r):
        r = _topk(r, self.k)
        gain = 2 ** r - 1 if self.exp else r
        return (gain / torch.log2(torch.arange(2, r.shape[1] + 2, dtype=torch.float64, device=r.device))).sum(1)
    def _per_query(self, rs, rel):
        ideal = self._dcg(rel.sort(1, descending=True).values)
        return torch.where(ideal > 0, self._dcg(rs) / ideal.clamp(min=1e-300), torch.zeros_like(ideal))


class MeanAveragePrecision(_QueryMetric):
    name = "map"
    def _per_query(self, rs, rel):
        hit = (_topk(rs, self.k) > 0).double()
        prec = hit.cumsum(1) / torch.arange(1, hit.shape[1] + 1, dtype=torch.float64, device=hit.device)
        denom = (rel > 0).sum(1).double()
        if self.k is not None:
            denom = denom.clamp(max=self.k)
        return (prec * hit).sum(1) / denom.clamp(min=1)


class MeanReciprocalRank(_QueryMetric):
    name = "mrr"
    def _per_query(self, rs, rel):
        hit = _topk(rs, self.k) > 0
        first = torch.where(hit.any(1), hit.double().argmax(1) + 1, torch.zeros(len(hit), dtype=torch.long, device=hit.device)).double()
        return torch.where(first > 0, 1 / first.clamp(min=1), torch.zeros_like(first))


class PrecisionAtK(_QueryMetric):
    name = "precision_at_k"
    def _per_query(self, rs, rel): return (_topk(rs, self.k) > 0).double().sum(1) / (self.k or rs.shape[1])
class RecallAtK(_QueryMetric):
    name = "recall_at_k"
    def _per_query(self, rs, rel): return (_topk(rs, self.k) > 0).double().sum(1) / (rel > 0).sum(1).double().clamp(min=1)
class F1AtK(_QueryMetric):
    name = "f1_at_k"
    def _per_query(self, rs, rel):
        p = (_topk(rs, self.k) > 0).double().sum(1) / (self.k or rs.shape[1])
        r = (_topk(rs, self.k) > 0).double().sum(1) / (rel > 0).sum(1).double().clamp(min=1)
        return 2 * p * r / (p + r).clamp(min=1e-12)
class HitRateAtK(_QueryMetric):
    name = "hit_rate_at_k"
    def _per_query(self, rs, rel): return (_topk(rs, self.k) > 0).any(1).double()
class RankingAUC(_QueryMetric):
    """Per-query probability that a relevant item is scored above an irrelevant one."""
    name = "ranking_auc"
    def _per_query(self, rs, rel):
        pos = (rs > 0).double()
        neg_before = (1 - pos).cumsum(1)
        n1, n0 = pos.sum(1), (1 - pos).sum(1)
        wrong = (pos * neg_before).sum(1)
        return torch.where((n1 > 0) & (n0 > 0), 1 - wrong / (n1 * n0).clamp(min=1), torch.full_like(n1, 0.5))


class Coverage(Metric):
    """Share of the catalogue that appears in any recommendation list."""
    name = "coverage"
    def __init__(self, catalog_size: int):
        self.catalog_size = catalog_size
        super().__init__()
    def _init_state(self): self._add("seen", torch.zeros(self.catalog_size, dtype=torch.float64))
    def update(self, recommended): self._acc("seen", torch.bincount(torch.as_tensor(recommended).reshape(-1), minlength=self.catalog_size))
    def compute(self) -> float: return float((self._state["seen"] > 0).double().mean())
    def gini(self) -> float:
        x = self._state["seen"].sort().values
        n = len(x)
        return float(((2 * torch.arange(1, n + 1, dtype=torch.float64) - n - 1) * x).sum() / (n * x.sum()).clamp(min=1e-300))


class Diversity(_SumMetric):
    """Mean pairwise cosine distance inside every recommendation list."""
    name, higher_is_better = "diversity", True
    def __init__(self, item_features: torch.Tensor):
        self.f = torch.nn.functional.normalize(item_features.double(), dim=1)
        super().__init__()
    def update(self, recommended):
        rec = torch.as_tensor(recommended)
        f = self.f[rec]
        sim = f @ f.transpose(1, 2)
        L = rec.shape[1]
        off = (sim.sum((1, 2)) - sim.diagonal(dim1=1, dim2=2).sum(1)) / (L * (L - 1))
        self._acc("sum", (1 - off).sum())
        self._acc("n", torch.tensor(float(len(rec))))


class Novelty(_SumMetric):
    """Mean self-information ``-log2 p(item)`` of recommended items under the popularity distribution."""
    name, higher_is_better = "novelty", True
    def __init__(self, item_popularity: torch.Tensor):
        p = item_popularity.double()
        self.info = -torch.log2((p / p.sum()).clamp(min=1e-300))
        super().__init__()
    def update(self, recommended):
        rec = torch.as_tensor(recommended).reshape(-1)
        self._acc("sum", self.info[rec].sum())
        self._acc("n", torch.tensor(float(len(rec))))


# ================================================================================================ clustering
class _ClusterMetric(Metric):
    """Not decomposable: batches are concatenated and the function applied at ``compute``."""
    fn: Callable = None
    def _init_state(self): self._a, self._b = [], []
    def reset(self):
        self._a, self._b = [], []
        return self
    def update(self, a, b):
        self._a.append(torch.as_tensor(a)); self._b.append(torch.as_tensor(b))
    def compute(self): return type(self).fn(torch.cat(self._a), torch.cat(self._b))
    def merge(self, other):
        self._a += other._a; self._b += other._b
        return self


def _cluster_fns():
    from .. import cluster as c
    return c


class SilhouetteScore(_ClusterMetric): fn = staticmethod(lambda x, l: _cluster_fns().silhouette_score(x, l))
class DaviesBouldin(_ClusterMetric):
    higher_is_better = False
    fn = staticmethod(lambda x, l: _cluster_fns().davies_bouldin(x, l))
class CalinskiHarabasz(_ClusterMetric): fn = staticmethod(lambda x, l: _cluster_fns().calinski_harabasz(x, l))
class DunnIndex(_ClusterMetric): fn = staticmethod(lambda x, l: _cluster_fns().dunn_index(x, l))
class Inertia(_ClusterMetric):
    higher_is_better = False
    fn = staticmethod(lambda x, l: _cluster_fns().inertia(x, l))
class AdjustedRandIndex(_ClusterMetric): fn = staticmethod(lambda a, b: _cluster_fns().adjusted_rand_index(a, b))
class NormalizedMutualInfo(_ClusterMetric): fn = staticmethod(lambda a, b: _cluster_fns().normalized_mutual_info(a, b))
class VMeasure(_ClusterMetric): fn = staticmethod(lambda a, b: _cluster_fns().homogeneity_completeness_v_measure(a, b)[2])


# ================================================================================================ language and uncertainty
class Perplexity(Metric):
    """``exp`` of the mean token negative log-likelihood; ``update(logits (.., V), targets (..), ignore_index)``."""
    name, higher_is_better = "perplexity", False
    def __init__(self, ignore_index: int = -100):
        self.ignore = ignore_index
        super().__init__()
    def _init_state(self):
        self._add("nll", torch.zeros((), dtype=torch.float64))
        self._add("n", torch.zeros((), dtype=torch.float64))
    def update(self, logits, target):
        lp = torch.log_softmax(logits.float(), -1).reshape(-1, logits.shape[-1])
        t = target.reshape(-1)
        keep = t != self.ignore
        self._acc("nll", -lp[keep].gather(1, t[keep, None]).sum())
        self._acc("n", keep.sum())
    def compute(self) -> float: return float(torch.exp(self._state["nll"] / self._state["n"].clamp(min=1)))


class ReliabilityDiagram(Metric):
    """Per-bin counts, summed confidence and summed correctness; the calibration errors and the curve come from these."""
    name = "reliability"
    def __init__(self, n_bins: int = 15):
        self.n_bins = n_bins
        super().__init__()
    def _init_state(self):
        for k in ("count", "conf", "acc"):
            self._add(k, torch.zeros(self.n_bins, dtype=torch.float64))
    def update(self, probs, target):
        if probs.dim() > target.dim():
            conf, pred = probs.max(-1)
            correct = (pred == target).double()
        else:
            conf, correct = probs, target.double()
        conf = conf.double().reshape(-1)
        b = (torch.ceil(conf * self.n_bins) - 1).clamp(0, self.n_bins - 1).long()
        self._acc("count", torch.bincount(b, minlength=self.n_bins))
        self._acc("conf", torch.bincount(b, weights=conf, minlength=self.n_bins))
        self._acc("acc", torch.bincount(b, weights=correct.reshape(-1), minlength=self.n_bins))
    def curve(self):
        c = self._state["count"].clamp(min=1)
        return self._state["conf"] / c, self._state["acc"] / c, self._state["count"]
    def compute(self) -> dict:
        conf, acc, n = self.curve()
        gap = (acc - conf).abs()
        w = n / n.sum().clamp(min=1)
        return {"ece": float((gap * w).sum()), "mce": float(gap[n > 0].max()) if bool((n > 0).any()) else 0.0}


class ExpectedCalibrationError(ReliabilityDiagram):
    name, higher_is_better = "ece", False
    def compute(self) -> float: return super().compute()["ece"]
class MaximumCalibrationError(ReliabilityDiagram):
    name, higher_is_better = "mce", False
    def compute(self) -> float: return super().compute()["mce"]


class BrierScore(_SumMetric):
    """Mean squared distance between the probability vector and the one-hot label (binary when probabilities are 1-D)."""
    name = "brier"
    def update(self, probs, target):
        if probs.dim() > target.dim():
            oh = torch.nn.functional.one_hot(target, probs.shape[-1]).double()
            self._acc("sum", ((probs.double() - oh) ** 2).sum())
        else:
            self._acc("sum", ((probs.double() - target.double()) ** 2).sum())
        self._acc("n", torch.tensor(float(target.numel()), device=target.device))


class PredictionIntervalCoverage(Metric):
    name = "picp"
    def _init_state(self):
        for k in ("inside", "width", "n"):
            self._add(k, torch.zeros((), dtype=torch.float64))
    def update(self, lower, upper, target):
        self._acc("inside", ((target >= lower) & (target <= upper)).sum())
        self._acc("width", (upper - lower).double().sum())
        self._acc("n", torch.tensor(float(target.numel()), device=target.device))
    def compute(self) -> dict:
        n = self._state["n"].clamp(min=1)
        return {"coverage": float(self._state["inside"] / n), "mean_width": float(self._state["width"] / n)}


class EntropyMeasures:
    @staticmethod
    def predictive_entropy(probs): return -(probs * probs.clamp(min=1e-12).log()).sum(-1)
    @staticmethod
    def normalized_entropy(probs): return EntropyMeasures.predictive_entropy(probs) / math.log(probs.shape[-1])
    @staticmethod
    def margin(probs):
        top = probs.topk(2, -1).values
        return top[..., 0] - top[..., 1]


class EnsembleUncertainty:
    """``probs (members, N, C)``: total = entropy of the mean, aleatoric = mean entropy, epistemic = their difference
    (the mutual information), plus the variation ratio."""
    @staticmethod
    def decompose(probs: torch.Tensor) -> dict:
        mean = probs.mean(0)
        total = EntropyMeasures.predictive_entropy(mean)
        alea = EntropyMeasures.predictive_entropy(probs).mean(0)
        votes = probs.argmax(-1)
        mode = votes.mode(0).values
        return {"total": total, "aleatoric": alea, "epistemic": total - alea, "variation_ratio": 1 - (votes == mode).double().mean(0)}


# ================================================================================================ fairness
class _GroupRates(Metric):
    """Per-group confusion counts of a binary classifier."""
    def __init__(self, num_groups: int = 2):
        self.g = num_groups
        super().__init__()
    def _init_state(self): self._add("c", torch.zeros(self.g, 2, 2, dtype=torch.float64))   # [group, true, pred]
    def update(self, pred, target, group):
        idx = group.reshape(-1) * 4 + target.reshape(-1).long() * 2 + pred.reshape(-1).long()
        self._acc("c", torch.bincount(idx, minlength=self.g * 4).view(self.g, 2, 2))
    def rates(self) -> dict:
        c = self._state["c"]
        n = c.sum((1, 2)).clamp(min=1)
        return {"positive_rate": c[:, :, 1].sum(1) / n, "tpr": c[:, 1, 1] / c[:, 1].sum(1).clamp(min=1), "fpr": c[:, 0, 1] / c[:, 0].sum(1).clamp(min=1),
                "ppv": c[:, 1, 1] / c[:, :, 1].sum(1).clamp(min=1), "accuracy": (c[:, 0, 0] + c[:, 1, 1]) / n}


class DemographicParity(_GroupRates):
    higher_is_better = False
    def compute(self) -> dict:
        r = self.rates()["positive_rate"]
        return {"difference": float(r.max() - r.min()), "ratio": float(r.min() / r.max().clamp(min=1e-12))}


class EqualizedOdds(_GroupRates):
    higher_is_better = False
    def compute(self) -> dict:
        r = self.rates()
        return {"tpr_gap": float(r["tpr"].max() - r["tpr"].min()), "fpr_gap": float(r["fpr"].max() - r["fpr"].min()),
                "difference": float(torch.maximum(r["tpr"].max() - r["tpr"].min(), r["fpr"].max() - r["fpr"].min()))}


class GroupCalibration(Metric):
    """Calibration error of every group and the largest gap between groups."""
    def __init__(self, num_groups: int = 2, n_bins: int = 10):
        self.diagrams = [ReliabilityDiagram(n_bins) for _ in range(num_groups)]
        super().__init__()
    def reset(self):
        for d in self.diagrams:
            d.reset()
        return self
    def update(self, probs, target, group):
        for g, d in enumerate(self.diagrams):
            m = group == g
            if bool(m.any()):
                d.update(probs[m], target[m])
    def compute(self) -> dict:
        e = [d.compute()["ece"] for d in self.diagrams]
        return {"ece_per_group": e, "gap": max(e) - min(e)}


class IndividualFairness:
    """Lipschitz view: similar individuals should get similar outputs.  ``evaluate`` reports the largest and mean ratio
    ``|f(x) - f(x')| / d(x, x')`` over sampled pairs and the share of pairs violating ``|df| <= L d``."""
    def __init__(self, lipschitz: float = 1.0, pairs: int = 10_000, seed: int = 0): self.L, self.pairs, self.seed = lipschitz, pairs, seed
    def evaluate(self, features: torch.Tensor, outputs: torch.Tensor) -> dict:
        g = torch.Generator().manual_seed(self.seed)
        n = len(features)
        i, j = torch.randint(0, n, (self.pairs,), generator=g), torch.randint(0, n, (self.pairs,), generator=g)
        keep = i != j
        i, j = i[keep], j[keep]
        d = (features[i] - features[j]).double().reshape(len(i), -1).norm(dim=1).clamp(min=1e-12)
        df = (outputs[i] - outputs[j]).double().reshape(len(i), -1).norm(dim=1)
        ratio = df / d
        return {"max_ratio": float(ratio.max()), "mean_ratio": float(ratio.mean()), "violation_rate": float((ratio > self.L).double().mean())}


class BiasAmplification:
    """How much the predicted label-group association exceeds the one in the data: mean over labels of
    ``P_pred(group* | label) - P_data(group* | label)`` where ``group*`` is the group over-represented for that label."""
    @staticmethod
    def compute(pred, target, group, num_classes: int, num_groups: int = 2) -> float:
        def assoc(lab):
            t = torch.bincount(lab * num_groups + group, minlength=num_classes * num_groups).view(num_classes, num_groups).double()
            return t / t.sum(1, keepdim=True).clamp(min=1)
        data, model = assoc(target), assoc(pred)
        star = data.argmax(1, keepdim=True)
        return float((model.gather(1, star) - data.gather(1, star)).mean())


class FairnessMetrics:
    """All group metrics in one pass."""
    def __init__(self, num_groups: int = 2): self.dp, self.eo = DemographicParity(num_groups), EqualizedOdds(num_groups)
    def update(self, pred, target, group):
        self.dp.update(pred, target, group); self.eo.update(pred, target, group)
    def compute(self) -> dict:
        r = self.dp.rates()
        return {"demographic_parity": self.dp.compute(), "equalized_odds": self.eo.compute(),
                "predictive_parity_gap": float(r["ppv"].max() - r["ppv"].min()), "accuracy_gap": float(r["accuracy"].max() - r["accuracy"].min())}


# ================================================================================================ streaming and chunked
StreamingAccuracy = Accuracy
StreamingConfusionMatrix = ConfusionMatrix
StreamingMetricCollection = MetricCollection


class StreamingAUROC(ThresholdMetrics):
    def compute(self) -> float: return self.auroc()


class StreamingStats(Metric):
    """Count, mean, variance (Chan's parallel update), min and max of a stream; ``merge`` combines two streams exactly."""
    def _init_state(self):
        self.n, self.mean, self.m2, self.lo, self.hi = 0, 0.0, 0.0, float("inf"), float("-inf")
    def reset(self):
        self._init_state()
        return self
    def _combine(self, n, mean, m2, lo, hi):
        tot = self.n + n
        if tot == 0:
            return
        d = mean - self.mean
        self.m2 += m2 + d * d * self.n * n / tot
        self.mean += d * n / tot
        self.n, self.lo, self.hi = tot, min(self.lo, lo), max(self.hi, hi)
    def update(self, x):
        x = torch.as_tensor(x).double().reshape(-1)
        if len(x):
            self._combine(len(x), float(x.mean()), float(((x - x.mean()) ** 2).sum()), float(x.min()), float(x.max()))
    def merge(self, other):
        self._combine(other.n, other.mean, other.m2, other.lo, other.hi)
        return self
    def compute(self) -> dict:
        return {"count": self.n, "mean": self.mean, "variance": self.m2 / (self.n - 1) if self.n > 1 else 0.0, "min": self.lo, "max": self.hi}


class ChunkedEvaluator:
    """Runs ``model`` over a dataset in chunks of ``chunk_size`` rows and feeds every output chunk to the metrics, so the
    peak memory is one chunk whatever the dataset size."""
    def __init__(self, metrics: MetricCollection | dict, chunk_size: int = 4096):
        self.metrics = metrics if isinstance(metrics, MetricCollection) else MetricCollection(metrics)
        self.chunk = chunk_size
    @torch.no_grad()
    def evaluate(self, model: Callable, inputs: torch.Tensor, targets: torch.Tensor) -> dict:
        self.metrics.reset()
        for lo in range(0, len(inputs), self.chunk):
            self.metrics.update(model(inputs[lo:lo + self.chunk]), targets[lo:lo + self.chunk])
        return self.metrics.compute()


# ================================================================================================ statistics
@dataclass
class HypothesisTestResult:
    statistic: float
    p_value: float
    significant: bool
    name: str = ""
    extra: dict = field(default_factory=dict)


def _wrap(name, res: dict, alpha: float) -> HypothesisTestResult:
    stat = next((res[k] for k in ("statistic", "t", "chi2", "u", "h", "w", "z", "f") if k in res), float("nan"))
    return HypothesisTestResult(float(stat), float(res["p_value"]), res["p_value"] < alpha, name, {k: v for k, v in res.items() if k != "p_value"})


class _Test:
    fn: Callable = None
    def __init__(self, alpha: float = 0.05): self.alpha = alpha
    def test(self, *a, **k) -> HypothesisTestResult: return _wrap(type(self).__name__, type(self).fn(*a, **k), self.alpha)


class PairedTTest(_Test): fn = staticmethod(_x.paired_t_test)
class McNemarTest(_Test): fn = staticmethod(_x.mcnemar_test)
class WilcoxonTest(_Test): fn = staticmethod(_x.wilcoxon_signed_rank)
class MannWhitneyTest(_Test): fn = staticmethod(_mm.mann_whitney_u)
class KruskalWallisTest(_Test): fn = staticmethod(_mm.kruskal_wallis)
class FriedmanTest(_Test): fn = staticmethod(_mm.friedman_test)
class FiveByTwoCVTest(_Test): fn = staticmethod(_mm.five_by_two_cv_test)
class PermutationTest(_Test):
    def test(self, a, b, n_perm: int = 5000, seed: int = 0) -> HypothesisTestResult:
        p = _x.permutation_test(a, b, n_perm, seed)
        return HypothesisTestResult(float(a.double().mean() - b.double().mean()), p, p < self.alpha, "PermutationTest")


class NemenyiTest:
    def __init__(self, alpha: float = 0.05): self.alpha = alpha
    def test(self, scores) -> dict: return _mm.nemenyi_test(scores)


class BootstrapCI:
    def __init__(self, n_boot: int = 1000, level: float = 0.95, seed: int = 0): self.n, self.level, self.seed = n_boot, level, seed
    def interval(self, metric: Callable, *arrays) -> dict:
        g = torch.Generator().manual_seed(self.seed)
        n = len(arrays[0])
        vals = torch.tensor([float(metric(*(a[idx] for a in arrays))) for idx in (torch.randint(0, n, (n,), generator=g) for _ in range(self.n))], dtype=torch.float64)
        lo, hi = torch.quantile(vals, torch.tensor([(1 - self.level) / 2, (1 + self.level) / 2], dtype=torch.float64)).tolist()
        return {"estimate": float(metric(*arrays)), "lower": lo, "upper": hi, "std_error": float(vals.std())}


class EffectSize:
    @staticmethod
    def compute(a, b, kind: str = "cohen_d"): return _mm.effect_size(a, b, kind)
class MultipleComparisonCorrection:
    def __init__(self, method: str = "holm"): self.method = method
    def correct(self, p_values, alpha: float = 0.05): return _mm.multiple_comparison_correction(p_values, self.method, alpha)


class CrossValidator:
    """K-fold (optionally stratified) evaluation of ``fit_score(train_idx, test_idx) -> float``."""
    def __init__(self, k: int = 5, stratified: bool = False, seed: int = 0): self.k, self.stratified, self.seed = k, stratified, seed
    def run(self, n_or_labels, fit_score: Callable) -> dict:
        folds = _x.stratified_k_fold_indices(n_or_labels, self.k, self.seed) if self.stratified else _x.k_fold_indices(int(n_or_labels), self.k, seed=self.seed)
        s = torch.tensor([float(fit_score(tr, te)) for tr, te in folds], dtype=torch.float64)
        se = float(s.std() / math.sqrt(len(s))) if len(s) > 1 else 0.0
        return {"scores": s.tolist(), "mean": float(s.mean()), "std": float(s.std()) if len(s) > 1 else 0.0, "ci95": (float(s.mean()) - 1.96 * se, float(s.mean()) + 1.96 * se)}


class StabilityAnalyzer:
    """Spread of a metric over repeated runs (seeds, resamples): coefficient of variation, range and the share of runs
    within ``tolerance`` of the median."""
    def __init__(self, tolerance: float = 0.01): self.tol = tolerance
    def analyze(self, values) -> dict:
        v = torch.as_tensor(values, dtype=torch.float64)
        med = v.median()
        return {"mean": float(v.mean()), "std": float(v.std()), "cv": float(v.std() / v.mean().abs().clamp(min=1e-12)), "range": float(v.max() - v.min()),
                "within_tolerance": float(((v - med).abs() <= self.tol).double().mean()), "stable": bool(((v - med).abs() <= self.tol).all())}


# ================================================================================================ model selection
class AIC:
    @staticmethod
    def compute(log_likelihood: float, k: int, n: int | None = None) -> float: return 2 * k - 2 * log_likelihood
class AICc:
    @staticmethod
    def compute(log_likelihood: float, k: int, n: int) -> float: return 2 * k - 2 * log_likelihood + 2 * k * (k + 1) / max(n - k - 1, 1)
class BIC:
    @staticmethod
    def compute(log_likelihood: float, k: int, n: int) -> float: return k * math.log(n) - 2 * log_likelihood
class HQIC:
    @staticmethod
    def compute(log_likelihood: float, k: int, n: int) -> float: return 2 * k * math.log(math.log(n)) - 2 * log_likelihood


class MultiModelComparison:
    """Ranks candidate models by a criterion; reports differences to the best, Akaike-style weights and evidence ratios."""
    def __init__(self, criterion: str = "aic"): self.criterion, self.models = criterion, {}
    def add(self, name: str, log_likelihood: float, k: int, n: int):
        self.models[name] = {"aic": AIC, "aicc": AICc, "bic": BIC, "hqic": HQIC}[self.criterion].compute(log_likelihood, k, n)
        return self
    def report(self) -> dict:
        best = min(self.models.values())
        delta = {m: v - best for m, v in self.models.items()}
        w = {m: math.exp(-0.5 * d) for m, d in delta.items()}
        z = sum(w.values())
        ranking = sorted(self.models, key=self.models.get)
        return {"ranking": ranking, "delta": delta, "weights": {m: v / z for m, v in w.items()}, "evidence_ratio": {m: w[ranking[0]] / max(w[m], 1e-300) for m in w}}


# ================================================================================================ advanced learning settings
class FewShotMetrics:
    """Episode accuracies -> mean and 95 % confidence interval (the usual way N-way K-shot results are reported)."""
    def __init__(self): self.acc = []
    def update(self, pred, target): self.acc.append(float((pred == target).double().mean()))
    def compute(self) -> dict:
        a = torch.tensor(self.acc, dtype=torch.float64)
        half = 1.96 * float(a.std()) / math.sqrt(len(a)) if len(a) > 1 else 0.0
        return {"episodes": len(a), "mean_accuracy": float(a.mean()), "ci95": half}


class MetaLearningMetrics:
    """Per task: loss before adaptation and after every inner step.  Reports the mean adaptation gain, the number of
    steps to reach ``fraction`` of the final gain, and the spread of post-adaptation loss across tasks."""
    def __init__(self): self.curves = []
    def update(self, losses_per_step: Sequence[float]): self.curves.append([float(v) for v in losses_per_step])
    def compute(self, fraction: float = 0.9) -> dict:
        c = torch.tensor(self.curves, dtype=torch.float64)
        gain = c[:, 0] - c[:, -1]
        mean_curve = c.mean(0)
        target = mean_curve[0] - fraction * (mean_curve[0] - mean_curve[-1])
        steps = int((mean_curve <= target).double().argmax())
        return {"adaptation_gain": float(gain.mean()), "steps_to_fraction": steps, "post_adaptation_std": float(c[:, -1].std()) if len(c) > 1 else 0.0,
                "tasks_improved": float((gain > 0).double().mean())}


class DomainAdaptationMetrics:
    """Source / target accuracy gap, linear-kernel and RBF maximum mean discrepancy between feature sets, and the proxy
    A-distance ``2 (1 - 2 err)`` of a least-squares domain classifier."""
    @staticmethod
    def mmd(a: torch.Tensor, b: torch.Tensor, kernel: str = "rbf", gamma: float | None = None) -> float:
        a, b = a.double(), b.double()
        if kernel == "linear":
            return float(((a.mean(0) - b.mean(0)) ** 2).sum())
        z = torch.cat([a, b])
        d2 = torch.cdist(z, z) ** 2
        gamma = gamma or 1.0 / float(d2[d2 > 0].median())
        K = torch.exp(-gamma * d2)
        n = len(a)
        return float(K[:n, :n].mean() + K[n:, n:].mean() - 2 * K[:n, n:].mean())

    @staticmethod
    def proxy_a_distance(a: torch.Tensor, b: torch.Tensor, seed: int = 0) -> float:
        g = torch.Generator().manual_seed(seed)
        z = torch.cat([a, b]).double()
        y = torch.cat([-torch.ones(len(a)), torch.ones(len(b))]).double()
        perm = torch.randperm(len(z), generator=g)
        tr, te = perm[: len(z) // 2], perm[len(z) // 2:]
        X = torch.cat([z, torch.ones(len(z), 1, dtype=torch.float64)], 1)
        w = torch.linalg.lstsq(X[tr], y[tr, None]).solution[:, 0]
        err = float(((X[te] @ w).sign() != y[te]).double().mean())
        return 2 * (1 - 2 * min(err, 0.5))

    @classmethod
    def compute(cls, src_feat, tgt_feat, src_acc: float, tgt_acc: float) -> dict:
        return {"accuracy_gap": src_acc - tgt_acc, "transfer_ratio": tgt_acc / max(src_acc, 1e-12), "mmd_rbf": cls.mmd(src_feat, tgt_feat),
                "mmd_linear": cls.mmd(src_feat, tgt_feat, "linear"), "proxy_a_distance": cls.proxy_a_distance(src_feat, tgt_feat)}


class ContinualLearningMetrics:
    """``acc[i][j]`` = accuracy on task ``j`` after training task ``i``."""
    @staticmethod
    def compute(acc_matrix) -> dict: return _mm.continual_learning_metrics(torch.as_tensor(acc_matrix, dtype=torch.float64))


# ================================================================================================ plots and reports
def _svg(width, height, body, title=""):
    head = f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" viewBox="0 0 {width} {height}" font-family="sans-serif" font-size="11">'
    ttl = f'<text x="{width / 2}" y="14" text-anchor="middle" font-size="13">{title}</text>' if title else ""
    return head + f'<rect width="{width}" height="{height}" fill="white"/>' + ttl + body + "</svg>"


class _LinePlot:
    title, xlabel, ylabel, diagonal = "", "x", "y", False
    W, H, M = 360, 300, 40

    def _render(self, series: dict[str, tuple], xlim=(0, 1), ylim=(0, 1)) -> str:
        W, H, M = self.W, self.H, self.M
        sx = lambda v: M + (v - xlim[0]) / max(xlim[1] - xlim[0], 1e-12) * (W - 2 * M)
        sy = lambda v: H - M - (v - ylim[0]) / max(ylim[1] - ylim[0], 1e-12) * (H - 2 * M)
        body = f'<rect x="{M}" y="{M}" width="{W - 2 * M}" height="{H - 2 * M}" fill="none" stroke="#888"/>'
        if self.diagonal:
            body += f'<line x1="{sx(xlim[0])}" y1="{sy(ylim[0])}" x2="{sx(xlim[1])}" y2="{sy(ylim[1])}" stroke="#bbb" stroke-dasharray="4"/>'
        colours = ["#1f77b4", "#d62728", "#2ca02c", "#9467bd", "#ff7f0e"]
        for i, (name, (xs, ys)) in enumerate(series.items()):
            pts = " ".join(f"{sx(float(a)):.1f},{sy(float(b)):.1f}" for a, b in zip(xs, ys))
            body += f'<polyline fill="none" stroke="{colours[i % 5]}" stroke-width="1.5" points="{pts}"/>'
            body += f'<text x="{W - M - 4}" y="{M + 14 + 13 * i}" text-anchor="end" fill="{colours[i % 5]}">{name}</text>'
        body += f'<text x="{W / 2}" y="{H - 8}" text-anchor="middle">{self.xlabel}</text><text x="12" y="{H / 2}" transform="rotate(-90 12 {H / 2})" text-anchor="middle">{self.ylabel}</text>'
        for v in (0, 0.5, 1):
            xv, yv = xlim[0] + v * (xlim[1] - xlim[0]), ylim[0] + v * (ylim[1] - ylim[0])
            body += f'<text x="{sx(xv)}" y="{H - M + 13}" text-anchor="middle">{xv:.3g}</text><text x="{M - 4}" y="{sy(yv) + 4}" text-anchor="end">{yv:.3g}</text>'
        return _svg(W, H, body, self.title)


class ROCCurvePlot(_LinePlot):
    title, xlabel, ylabel, diagonal = "ROC", "false positive rate", "true positive rate", True
    def render(self, curves: dict[str, ThresholdMetrics]) -> str:
        return self._render({f"{n} (AUC {m.auroc():.3f})": tuple(t.tolist() for t in m.roc_curve()) for n, m in curves.items()})


class PRCurvePlot(_LinePlot):
    title, xlabel, ylabel = "Precision-recall", "recall", "precision"
    def render(self, curves: dict[str, ThresholdMetrics]) -> str:
        return self._render({f"{n} (AP {m.average_precision():.3f})": tuple(t.tolist() for t in m.pr_curve()) for n, m in curves.items()})


class CalibrationCurvePlot(_LinePlot):
    title, xlabel, ylabel, diagonal = "Reliability", "confidence", "accuracy", True
    def render(self, diagrams: dict[str, ReliabilityDiagram]) -> str:
        out = {}
        for n, d in diagrams.items():
            conf, acc, cnt = d.curve()
            keep = cnt > 0
            out[f"{n} (ECE {d.compute()['ece']:.3f})"] = (conf[keep].tolist(), acc[keep].tolist())
        return self._render(out)


class LearningCurvePlot(_LinePlot):
    title, xlabel, ylabel = "Learning curve", "step", "value"
    def render(self, curves: dict[str, Sequence[float]]) -> str:
        hi = max(len(v) for v in curves.values()) - 1
        lo_y, hi_y = min(min(v) for v in curves.values()), max(max(v) for v in curves.values())
        return self._render({n: (list(range(len(v))), list(v)) for n, v in curves.items()}, (0, max(hi, 1)), (lo_y, hi_y if hi_y > lo_y else lo_y + 1))


class ConfusionMatrixPlot:
    def render(self, cm: torch.Tensor, labels: Sequence[str] | None = None, normalize: bool = True) -> str:
        k = len(cm)
        labels = labels or [str(i) for i in range(k)]
        shown = cm / cm.sum(1, keepdim=True).clamp(min=1) if normalize else cm / cm.max().clamp(min=1)
        cell, off = 44, 60
        body = ""
        for i in range(k):
            for j in range(k):
                v = float(shown[i, j])
                shade = int(255 - 200 * v)
                body += f'<rect x="{off + j * cell}" y="{off + i * cell}" width="{cell}" height="{cell}" fill="rgb({shade},{shade},255)" stroke="#fff"/>'
                body += f'<text x="{off + j * cell + cell / 2}" y="{off + i * cell + cell / 2 + 4}" text-anchor="middle" fill="{"#fff" if v > 0.6 else "#000"}">{int(cm[i, j])}</text>'
            body += f'<text x="{off - 6}" y="{off + i * cell + cell / 2 + 4}" text-anchor="end">{labels[i]}</text><text x="{off + i * cell + cell / 2}" y="{off - 6}" text-anchor="middle">{labels[i]}</text>'
        size = off + k * cell + 10
        return _svg(size, size, body, "Confusion matrix (rows: true)")


class _BarPlot:
    title = ""
    def render(self, values: dict[str, float]) -> str:
        items = sorted(values.items(), key=lambda kv: -abs(kv[1]))
        top = max(abs(v) for _, v in items) or 1.0
        body = ""
        for i, (n, v) in enumerate(items):
            y = 28 + i * 20
            body += f'<text x="118" y="{y + 12}" text-anchor="end">{n}</text><rect x="124" y="{y}" width="{abs(v) / top * 200:.1f}" height="14" fill="{"#1f77b4" if v >= 0 else "#d62728"}"/>'
            body += f'<text x="{128 + abs(v) / top * 200:.1f}" y="{y + 12}">{v:.4g}</text>'
        return _svg(400, 40 + 20 * len(items), body, self.title)


class FeatureImportancePlot(_BarPlot): title = "Feature importance"
class MetricComparisonPlot(_BarPlot): title = "Metric comparison"


class LatexReportBuilder:
    """Collects result rows and emits a ``booktabs`` table with the best value per column in bold."""
    def __init__(self, caption: str = "Results", label: str = "tab:results", precision: int = 3):
        self.caption, self.label, self.precision, self.rows, self.higher = caption, label, precision, {}, {}
    def add(self, model: str, metrics: dict[str, float], higher_is_better: dict[str, bool] | None = None):
        self.rows[model] = dict(metrics)
        self.higher.update(higher_is_better or {})
        return self
    def build(self) -> str:
        cols = sorted({k for r in self.rows.values() for k in r})
        best = {c: (max if self.higher.get(c, True) else min)(r[c] for r in self.rows.values() if c in r) for c in cols}
        esc = lambda s: s.replace("_", r"\_").replace("%", r"\%").replace("&", r"\&")
        lines = [r"\begin{table}[t]", r"\centering", rf"\caption{{{esc(self.caption)}}}", rf"\label{{{self.label}}}", r"\begin{tabular}{l" + "r" * len(cols) + "}", r"\toprule",
                 "Model & " + " & ".join(esc(c) for c in cols) + r" \\", r"\midrule"]
        for m, r in self.rows.items():
            cells = []
            for c in cols:
                if c not in r:
                    cells.append("--")
                    continue
                txt = f"{r[c]:.{self.precision}f}"
                cells.append(rf"\textbf{{{txt}}}" if r[c] == best[c] else txt)
            lines.append(esc(m) + " & " + " & ".join(cells) + r" \\")
        return "\n".join(lines + [r"\bottomrule", r"\end{tabular}", r"\end{table}"])


class ExperimentTracker:
    """Runs with parameters, per-step metrics and tags, kept in memory and written as one JSON file per run; ``best_run``
    picks by a metric's final (or best) value.  ``to_mlflow`` replays a run into an ``MLflowWriter`` directory."""
    def __init__(self, root=None):
        self.root, self.runs, self.active = root, {}, None

    def start_run(self, name: str, params: dict | None = None, tags: dict | None = None) -> str:
        rid = f"{len(self.runs):04d}-{name}"
        self.runs[rid] = {"name": name, "params": dict(params or {}), "tags": dict(tags or {}), "metrics": {}, "status": "running"}
        self.active = rid
        return rid

    def log_metric(self, key: str, value: float, step: int | None = None):
        hist = self.runs[self.active]["metrics"].setdefault(key, [])
        hist.append((len(hist) if step is None else step, float(value)))

    def log_metrics(self, values: dict, step: int | None = None):
        for k, v in values.items():
            self.log_metric(k, v, step)

    def end_run(self, status: str = "finished"):
        run = self.runs[self.active]
        run["status"] = status
        if self.root is not None:
            import json
            from pathlib import Path
            Path(self.root).mkdir(parents=True, exist_ok=True)
            (Path(self.root) / f"{self.active}.json").write_text(json.dumps(run, indent=1))
        self.active = None

    def best_run(self, metric: str, mode: str = "max", use: str = "last") -> str:
        pick = max if mode == "max" else min
        def val(r):
            h = [v for _, v in r["metrics"].get(metric, [])]
            if not h:
                return float("-inf") if mode == "max" else float("inf")
            return h[-1] if use == "last" else pick(h)
        return pick(self.runs, key=lambda rid: val(self.runs[rid]))

    def compare(self, metric: str) -> list[tuple[str, float]]:
        return sorted(((rid, r["metrics"][metric][-1][1]) for rid, r in self.runs.items() if metric in r["metrics"]), key=lambda kv: -kv[1])

    def to_mlflow(self, run_id: str, directory) -> None:
        w = _m.MLflowWriter(str(directory), run_name=self.runs[run_id]["name"])
        run = self.runs[run_id]
        for k, v in run["params"].items():
            w.log_param(k, v)
        for k, hist in run["metrics"].items():
            for step, v in hist:
                w.log_metric(k, v, step)
