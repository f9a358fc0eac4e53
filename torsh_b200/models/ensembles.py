"""Ensembles and model-file operations (``crates/torsh-models/src/ensembling.rs``, ``ensembling_advanced.rs``,
``crates/torsh-hub/src/model_ops.rs``): hard / soft / weighted voting, weights fitted on validation data, stacking with a
cross-validated meta-learner, bagging, snapshot ensembles, online adaptive weights, diversity measures, greedy ensemble
selection with size and gain estimates; state-dict comparison with shape and value differences, automatic loading by file
type and quantisation statistics."""
from __future__ import annotations

import copy
import math
from pathlib import Path
from typing import Callable, Sequence

import torch
from torch import nn


# ================================================================================================ combining predictions
def combine_predictions(probs: torch.Tensor, strategy: str = "soft", weights: torch.Tensor | None = None) -> torch.Tensor:
    """``probs [models, samples, classes]`` -> class probabilities.  ``soft`` averages probabilities, ``hard`` counts arg-max votes,
    ``weighted`` uses the given model weights, ``geometric`` averages log-probabilities, ``max`` takes the most confident model."""
    m = probs.shape[0]
    if strategy == "soft":
        return probs.mean(0)
    if strategy == "hard":
        votes = torch.nn.functional.one_hot(probs.argmax(-1), probs.shape[-1]).float()
        if weights is not None:
            votes = votes * weights.reshape(m, 1, 1)
        return votes.sum(0) / votes.sum(0).sum(-1, keepdim=True)
    if strategy == "weighted":
        w = (weights / weights.sum()).reshape(m, 1, 1)
        return (probs * w).sum(0)
    if strategy == "geometric":
        g = probs.clamp_min(1e-12).log().mean(0).exp()
        return g / g.sum(-1, keepdim=True)
    if strategy == "max":
        conf = probs.max(-1).values
        return probs[conf.argmax(0), torch.arange(probs.shape[1])]
    raise ValueError(strategy)


def fit_ensemble_weights(probs: torch.Tensor, targets: torch.Tensor, steps: int = 200, lr: float = 0.1) -> torch.Tensor:
    """Weights on the simplex minimising the validation negative log-likelihood of the weighted average."""
    theta = torch.zeros(probs.shape[0], requires_grad=True)
    opt = torch.optim.Adam([theta], lr=lr)
    for _ in range(steps):
        w = torch.softmax(theta, 0).reshape(-1, 1, 1)
        loss = torch.nn.functional.nll_loss((probs * w).sum(0).clamp_min(1e-12).log(), targets)
        opt.zero_grad(); loss.backward(); opt.step()
    return torch.softmax(theta.detach(), 0)


class StackingEnsemble:
    """Base models' out-of-fold probabilities train a meta-learner (multinomial logistic regression on the concatenated
    probabilities), so the meta-learner never sees predictions made on data a base model was trained on."""

    def __init__(self, make_models: Sequence[Callable[[], nn.Module]], train: Callable[[nn.Module, torch.Tensor, torch.Tensor], None], folds: int = 4, seed: int = 0): self.make, self.train, self.folds, self.seed = list(make_models), train, folds, seed

    def fit(self, x: torch.Tensor, y: torch.Tensor, meta_steps: int = 300) -> "StackingEnsemble":
        n, k = len(x), int(y.max()) + 1
        g = torch.Generator().manual_seed(self.seed)
        fold = torch.empty(n, dtype=torch.long); fold[torch.randperm(n, generator=g)] = torch.arange(n) % self.folds
        oof = torch.zeros(len(self.make), n, k)
        for mi, mk in enumerate(self.make):
            for f in range(self.folds):
                tr, te = fold != f, fold == f
                m = mk(); self.train(m, x[tr], y[tr]); m.eval()
                with torch.no_grad():
                    oof[mi, te] = m(x[te]).softmax(-1)
        self.meta = nn.Linear(len(self.make) * k, k)
        feats = oof.permute(1, 0, 2).reshape(n, -1)
        opt = torch.optim.Adam(self.meta.parameters(), lr=0.05, weight_decay=1e-3)
        for _ in range(meta_steps):
            loss = torch.nn.functional.cross_entropy(self.meta(feats), y)
            opt.zero_grad(); loss.backward(); opt.step()
        self.models = []
        for mk in self.make:                                                        # final base models on all the data
            m = mk(); self.train(m, x, y); m.eval(); self.models.append(m)
        self.oof_accuracy = [float((oof[i].argmax(-1) == y).float().mean()) for i in range(len(self.make))]
        return self

    @torch.no_grad()
    def predict_proba(self, x: torch.Tensor) -> torch.Tensor:
        feats = torch.stack([m(x).softmax(-1) for m in self.models], 1).reshape(len(x), -1)
        return self.meta(feats).softmax(-1)


def bagging(make_model: Callable[[], nn.Module], train: Callable, x: torch.Tensor, y: torch.Tensor, n_models: int = 5, sample_fraction: float = 1.0, seed: int = 0) -> tuple[list[nn.Module], list[torch.Tensor]]:
    """Models trained on bootstrap samples; also returns each model's out-of-bag indices (for an unbiased error estimate)."""
    g = torch.Generator().manual_seed(seed)
    models, oob = [], []
    for _ in range(n_models):
        idx = torch.randint(len(x), (int(sample_fraction * len(x)),), generator=g)
        m = make_model(); train(m, x[idx], y[idx]); m.eval(); models.append(m)
        mask = torch.ones(len(x), dtype=torch.bool); mask[idx] = False
        oob.append(mask.nonzero().flatten())
    return models, oob


@torch.no_grad()
def out_of_bag_accuracy(models: Sequence[nn.Module], oob: Sequence[torch.Tensor], x: torch.Tensor, y: torch.Tensor) -> float:
    k = int(y.max()) + 1
    votes = torch.zeros(len(x), k)
    for m, idx in zip(models, oob):
        votes[idx] += m(x[idx]).softmax(-1)
    seen = votes.sum(1) > 0
    return float((votes[seen].argmax(1) == y[seen]).float().mean())


class SnapshotEnsemble:
    """One training run with a cyclic cosine learning rate; the weights at the end of every cycle (a different local minimum)
    are kept and averaged at prediction time."""

    def __init__(self, model: nn.Module, cycles: int = 4, steps_per_cycle: int = 50, max_lr: float = 0.1): self.model, self.cycles, self.spc, self.max_lr, self.snapshots = model, cycles, steps_per_cycle, max_lr, []
    def lr_at(self, step: int) -> float: return 0.5 * self.max_lr * (1 + math.cos(math.pi * (step % self.spc) / self.spc))

    def fit(self, loss_fn: Callable[[nn.Module], torch.Tensor]) -> list[float]:
        opt, hist = torch.optim.SGD(self.model.parameters(), lr=self.max_lr, momentum=0.9), []
        for step in range(self.cycles * self.spc):
            for gp in opt.param_groups:
                gp["lr"] = self.lr_at(step)
            loss = loss_fn(self.model)
            opt.zero_grad(); loss.backward(); opt.step(); hist.append(float(loss.detach()))
            if (step + 1) % self.spc == 0:
                self.snapshots.append(copy.deepcopy(self.model.state_dict()))
        return hist

    @torch.no_grad()
    def predict_proba(self, x: torch.Tensor, last: int | None = None) -> torch.Tensor:
        keep, out = self.snapshots[-(last or len(self.snapshots)):], 0
        current = copy.deepcopy(self.model.state_dict())
        for s in keep:
            self.model.load_state_dict(s); out = out + self.model(x).softmax(-1)
        self.model.load_state_dict(current)
        return out / len(keep)


class OnlineAdaptiveEnsemble:
    """Multiplicative-weights (Hedge) combination: after each labelled example every model's weight is multiplied by
    ``exp(-eta * loss)``; the ensemble tracks the best model in hindsight and follows drift with ``forget``."""

    def __init__(self, n_models: int, eta: float = 0.5, forget: float = 0.0): self.w, self.eta, self.forget, self.cum_loss = torch.ones(n_models) / n_models, eta, forget, torch.zeros(n_models)
    def predict(self, probs: torch.Tensor) -> torch.Tensor: return (probs * self.w[:, None]).sum(0)
    def update(self, probs: torch.Tensor, target: int):
        loss = -probs[:, target].clamp_min(1e-12).log()
        self.cum_loss += loss
        w = self.w * torch.exp(-self.eta * loss)
        w = w / w.sum()
        self.w = (1 - self.forget) * w + self.forget / len(w)


# ================================================================================================ diversity and selection
def diversity_measures(preds: torch.Tensor, targets: torch.Tensor) -> dict:
    """``preds [models, samples]`` of class labels: mean pairwise disagreement, mean Yule's Q-statistic and correlation of the
    correctness indicators, and the double-fault rate."""
    m = preds.shape[0]
    c = (preds == targets).float()
    dis, qs, rho, df = [], [], [], []
    for i in range(m):
        for j in range(i + 1, m):
            n11, n00 = float((c[i] * c[j]).sum()), float(((1 - c[i]) * (1 - c[j])).sum())
            n10, n01 = float((c[i] * (1 - c[j])).sum()), float(((1 - c[i]) * c[j]).sum())
            dis.append(float((preds[i] != preds[j]).float().mean()))
            qs.append((n11 * n00 - n01 * n10) / (n11 * n00 + n01 * n10) if n11 * n00 + n01 * n10 else 0.0)
            den = math.sqrt((n11 + n10) * (n01 + n00) * (n11 + n01) * (n10 + n00))
            rho.append((n11 * n00 - n01 * n10) / den if den else 0.0)
            df.append(n00 / c.shape[1])
    mean = lambda v: sum(v) / len(v) if v else 0.0
    return {"disagreement": mean(dis), "q_statistic": mean(qs), "correlation": mean(rho), "double_fault": mean(df)}


def greedy_ensemble_selection(probs: torch.Tensor, targets: torch.Tensor, max_size: int | None = None, with_replacement: bool = True) -> dict:
    """Forward selection on validation data (Caruana): start from the best single model, repeatedly add the model (possibly
    again) that lowers the validation loss of the average most, stop when nothing helps.  The counts are the weights."""
    m = probs.shape[0]
    nll = lambda p: float(torch.nn.functional.nll_loss(p.clamp_min(1e-12).log(), targets))
    chosen, total = [], torch.zeros_like(probs[0])
    best_loss, trace = math.inf, []
    while max_size is None or len(chosen) < max_size:
        cands = [i for i in range(m) if with_replacement or i not in chosen]
        if not cands:
            break
        losses = {i: nll((total + probs[i]) / (len(chosen) + 1)) for i in cands}
        i = min(losses, key=losses.get)
        if losses[i] >= best_loss - 1e-9:
            break
        chosen.append(i); total = total + probs[i]; best_loss = losses[i]; trace.append(best_loss)
    counts = torch.bincount(torch.tensor(chosen), minlength=m).float()
    single = min(nll(probs[i]) for i in range(m))
    return {"members": chosen, "weights": counts / counts.sum(), "validation_loss": best_loss, "best_single_loss": single, "improvement": 1 - best_loss / single, "size": len(set(chosen)), "trace": trace}


def estimate_ensemble_gain(individual_accuracy: float, correlation: float, size: int) -> float:
    """Accuracy of a majority vote of ``size`` equally accurate binary classifiers whose errors have pairwise correlation
    ``correlation`` (the effective number of independent voters is ``size / (1 + (size - 1) rho)``)."""
    n_eff = max(1.0, size / (1 + (size - 1) * correlation))
    n = max(1, int(round(n_eff)))
    n = n if n % 2 else n + 1
    p = individual_accuracy
    return sum(math.comb(n, k) * p ** k * (1 - p) ** (n - k) for k in range(n // 2 + 1, n + 1))


def optimal_ensemble_size(individual_accuracy: float, correlation: float, max_size: int = 25, min_gain: float = 0.002) -> int:
    best, prev = 1, individual_accuracy
    for s in range(3, max_size + 1, 2):
        acc = estimate_ensemble_gain(individual_accuracy, correlation, s)
        if acc - prev < min_gain:
            break
        best, prev = s, acc
    return best


# ================================================================================================ model file operations
def compare_state_dicts(a: dict, b: dict, rtol: float = 1e-5, atol: float = 1e-8, top: int = 5) -> dict:
    """Keys only in one model, shape differences, and for tensors of equal shape the largest value differences."""
    only_a, only_b = sorted(set(a) - set(b)), sorted(set(b) - set(a))
    shape_diff, value_diff, identical = [], [], 0
    for k in sorted(set(a) & set(b)):
        if a[k].shape != b[k].shape:
            shape_diff.append({"name": k, "a": tuple(a[k].shape), "b": tuple(b[k].shape)})
        elif torch.allclose(a[k].double(), b[k].double(), rtol=rtol, atol=atol, equal_nan=True):
            identical += 1
        else:
            d = (a[k].double() - b[k].double()).abs()
            value_diff.append({"name": k, "max_abs": float(d.max()), "mean_abs": float(d.mean()), "relative": float(d.norm() / a[k].double().norm().clamp_min(1e-30)), "changed_fraction": float((d > atol).float().mean())})
    value_diff.sort(key=lambda r: -r["max_abs"])
    return {"only_in_a": only_a, "only_in_b": only_b, "shape_differences": shape_diff, "value_differences": value_diff[:top], "changed_tensors": len(value_diff), "identical_tensors": identical,
            "same_architecture": not only_a and not only_b and not shape_diff, "identical": not only_a and not only_b and not shape_diff and not value_diff}


def load_model_auto(path) -> dict:
    """State dict from ``.pt`` / ``.pth`` (pickle-free load), ``.safetensors``, ``.npz`` or the framework's own model-state formats,
    chosen by extension; raises with the list of supported types otherwise."""
    p = Path(path)
    ext = p.suffix.lower()
    if ext in (".pt", ".pth"):
        return torch.load(p, map_location="cpu", weights_only=True)
    if ext == ".safetensors":
        from .tooling import LazyModelLoader
        with LazyModelLoader(p) as ld:
            return {k: ld.get_tensor(k) for k in ld.tensor_names()}
    if ext == ".npz":
        import numpy as np
        return {k: torch.from_numpy(v) for k, v in np.load(p).items()}
    if ext in (".json", ".trsm"):
        from ..serialize import model_state as ms
        st = ms.load_json(str(p)) if ext == ".json" else ms.load_binary(str(p))
        return {k: torch.tensor(v["data"]).reshape(v["shape"]) for k, v in st["parameters"].items()}
    raise ValueError(f"unsupported model file type {ext!r}; supported: .pt .pth .safetensors .npz .json .trsm")


def quantization_stats(state: dict, bits: int = 8) -> dict:
    """What symmetric per-tensor quantisation to ``bits`` would do to every floating-point matrix: size, error and the
    tensors that suffer most."""
    rows, fp_bytes, q_bytes = [], 0, 0
    qmax = 2 ** (bits - 1) - 1
    for k, t in state.items():
        if not t.is_floating_point() or t.dim() < 2:
            fp_bytes += t.numel() * t.element_size(); q_bytes += t.numel() * t.element_size(); continue
        s = t.abs().max() / qmax
        dq = (t / s).round().clamp(-qmax - 1, qmax) * s if s > 0 else t
        err = float((dq - t).norm() / t.norm().clamp_min(1e-30))
        rows.append({"name": k, "relative_error": err, "range": float(t.abs().max()), "outlier_ratio": float((t.abs() > 6 * t.std()).float().mean())})
        fp_bytes += t.numel() * t.element_size(); q_bytes += t.numel() * bits / 8 + 4
    rows.sort(key=lambda r: -r["relative_error"])
    return {"tensors": len(rows), "size_bytes": fp_bytes, "quantized_bytes": q_bytes, "compression": fp_bytes / max(q_bytes, 1), "mean_relative_error": sum(r["relative_error"] for r in rows) / max(len(rows), 1), "worst": rows[:3]}
