"""Training / evaluation metrics and step logging.

Classification, regression and ranking metrics in the spirit of ``crates/torsh-metrics`` (accuracy, precision / recall /
F1, confusion matrix, top-k, ROC-AUC, MSE / MAE / R², perplexity, NDCG) and the JSONL step logger + Prometheus text
endpoint described for the distributed monitor (``crates/torsh-distributed/src/metrics.rs:33-760``,
``prometheus_exporter.rs:50-294``)."""
from __future__ import annotations

import json
import math
import threading
import time
from http.server import BaseHTTPRequestHandler, HTTPServer

import torch


def accuracy(pred: torch.Tensor, target: torch.Tensor) -> float:
    if pred.dim() > target.dim():
        pred = pred.argmax(-1)
    return (pred == target).float().mean().item()


def top_k_accuracy(logits: torch.Tensor, target: torch.Tensor, k: int = 5) -> float:
    return (logits.topk(k, -1).indices == target.unsqueeze(-1)).any(-1).float().mean().item()


def confusion_matrix(pred: torch.Tensor, target: torch.Tensor, num_classes: int) -> torch.Tensor:
    if pred.dim() > target.dim():
        pred = pred.argmax(-1)
    idx = target.reshape(-1) * num_classes + pred.reshape(-1)
    return torch.bincount(idx, minlength=num_classes * num_classes).view(num_classes, num_classes)


def precision_recall_f1(pred, target, num_classes: int, average: str = "macro"):
    cm = confusion_matrix(pred, target, num_classes).float()
    tp = cm.diag()
    prec = tp / cm.sum(0).clamp(min=1)
    rec = tp / cm.sum(1).clamp(min=1)
    f1 = 2 * prec * rec / (prec + rec).clamp(min=1e-12)
    if average == "micro":
        p = r = tp.sum() / cm.sum().clamp(min=1)
        return p.item(), r.item(), p.item()
    if average == "weighted":
        w = cm.sum(1) / cm.sum()
        return (prec * w).sum().item(), (rec * w).sum().item(), (f1 * w).sum().item()
    return prec.mean().item(), rec.mean().item(), f1.mean().item()


def roc_auc(scores: torch.Tensor, target: torch.Tensor) -> float:
    order = scores.argsort()
    ranks = torch.empty_like(order, dtype=torch.float)
    ranks[order] = torch.arange(1, len(scores) + 1, dtype=torch.float)
    pos = target.bool()
    n1, n0 = pos.sum().item(), (~pos).sum().item()
    if n1 == 0 or n0 == 0:
        return float("nan")
    return ((ranks[pos].sum() - n1 * (n1 + 1) / 2) / (n1 * n0)).item()


def mse(p, t): return torch.mean((p.float() - t.float()) ** 2).item()
def mae(p, t): return torch.mean((p.float() - t.float()).abs()).item()
def rmse(p, t): return math.sqrt(mse(p, t))


def r2_score(p, t) -> float:
    t = t.float()
    return (1 - ((p.float() - t) ** 2).sum() / ((t - t.mean()) ** 2).sum().clamp(min=1e-12)).item()


def perplexity(mean_cross_entropy: float) -> float:
    return math.exp(min(mean_cross_entropy, 50.0))


def ndcg_at_k(scores: torch.Tensor, relevance: torch.Tensor, k: int = 10) -> float:
    k = min(k, scores.numel())
    disc = 1.0 / torch.log2(torch.arange(2, k + 2, dtype=torch.float))
    dcg = (relevance[scores.topk(k).indices].float() * disc).sum()
    idcg = (relevance.float().topk(k).values * disc).sum()
    return (dcg / idcg.clamp(min=1e-12)).item()


class MetricsLogger:
    """One JSON object per step: loss, tokens/s or images/s, comm bandwidth, memory; optional Prometheus endpoint."""

    def __init__(self, path=None, rank: int = 0):
        self.path, self.rank, self.latest, self._srv = path, rank, {}, None
        self._f = open(path, "a") if path else None

    def log(self, step: int, **values):
        rec = {"step": step, "time": time.time(), "rank": self.rank, **values}
        if torch.cuda.is_available():
            rec["mem_allocated_gb"] = torch.cuda.memory_allocated() / 2 ** 30
            rec["mem_reserved_gb"] = torch.cuda.memory_reserved() / 2 ** 30
        self.latest = rec
        if self._f:
            self._f.write(json.dumps(rec) + "\n")
            self._f.flush()
        return rec

    def prometheus_text(self, prefix="torsh_train") -> str:
        return "".join(f"{prefix}_{k} {v}\n" for k, v in self.latest.items() if isinstance(v, (int, float)))

    def serve(self, port: int = 0, host: str = "127.0.0.1") -> int:
        logger = self

        class H(BaseHTTPRequestHandler):
            def do_GET(self):  # noqa: N802
                body = logger.prometheus_text().encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *a):
                pass

        self._srv = HTTPServer((host, port), H)
        threading.Thread(target=self._srv.serve_forever, daemon=True).start()
        return self._srv.server_address[1]

    def close(self):
        if self._srv:
            self._srv.shutdown()
        if self._f:
            self._f.close()


# ------------------------------------------------------------------------------------------------------------ fairness
def demographic_parity_difference(pred: torch.Tensor, group: torch.Tensor) -> float:
    """Largest gap between groups in the rate of positive predictions (``crates/torsh-metrics``: fairness)."""
    rates = [pred[group == g].float().mean().item() for g in group.unique()]
    return max(rates) - min(rates)


def equalized_odds_difference(pred: torch.Tensor, target: torch.Tensor, group: torch.Tensor) -> float:
    """Largest gap between groups in true-positive rate or false-positive rate."""
    gaps = []
    for label in (1, 0):
        rates = []
        for g in group.unique():
            m = (group == g) & (target == label)
            if m.any():
                rates.append(pred[m].float().mean().item())
        if rates:
            gaps.append(max(rates) - min(rates))
    return max(gaps) if gaps else 0.0


def disparate_impact_ratio(pred: torch.Tensor, group: torch.Tensor) -> float:
    rates = [pred[group == g].float().mean().item() for g in group.unique()]
    return min(rates) / max(max(rates), 1e-12)


# ------------------------------------------------------------------------------------------------- experiment writers
class MLflowWriter:
    """Writes the MLflow file-store layout without the mlflow package: ``<root>/<experiment_id>/<run_id>/`` with
    ``metrics/<key>`` (lines ``timestamp_ms value step``), ``params/<key>``, ``tags/<key>`` and ``meta.yaml`` files, which
    ``mlflow ui --backend-store-uri <root>`` reads."""

    def __init__(self, root: str, experiment: str = "0", run_name: str = "run"):
        import os
        import time
        import uuid
        self.run_id = uuid.uuid4().hex
        self.dir = os.path.join(root, experiment, self.run_id)
        for sub in ("metrics", "params", "tags", "artifacts"):
            os.makedirs(os.path.join(self.dir, sub), exist_ok=True)
        start = int(time.time() * 1000)
        with open(os.path.join(root, experiment, "meta.yaml"), "w") as f:
            f.write(f"artifact_location: {os.path.join(root, experiment)}\nexperiment_id: '{experiment}'\nlifecycle_stage: active\nname: Default\n")
        with open(os.path.join(self.dir, "meta.yaml"), "w") as f:
            f.write(f"artifact_uri: {os.path.join(self.dir, 'artifacts')}\nend_time: null\nexperiment_id: '{experiment}'\n"
                    f"lifecycle_stage: active\nrun_id: {self.run_id}\nrun_name: {run_name}\nstart_time: {start}\nstatus: 1\n")

    def _write(self, sub, key, text, mode):
        import os
        with open(os.path.join(self.dir, sub, key.replace("/", "_")), mode) as f:
            f.write(text)

    def log_param(self, key: str, value): self._write("params", key, str(value), "w")
    def set_tag(self, key: str, value): self._write("tags", key, str(value), "w")

    def log_metric(self, key: str, value: float, step: int = 0):
        import time
        self._write("metrics", key, f"{int(time.time() * 1000)} {float(value)} {int(step)}\n", "a")


class WandbOfflineWriter:
    """History and summary files in the layout of an offline W&B run directory (``wandb-history.jsonl``,
    ``wandb-summary.json``, ``config.yaml``) for later upload or inspection; needs no wandb package."""

    def __init__(self, root: str, project: str = "torsh", config: dict | None = None):
        import os
        import time
        self.dir = os.path.join(root, f"offline-run-{time.strftime('%Y%m%d_%H%M%S')}-{os.getpid()}", "files")
        os.makedirs(self.dir, exist_ok=True)
        self.summary, self._step = {}, 0
        with open(os.path.join(self.dir, "config.yaml"), "w") as f:
            f.write(f"wandb_project:\n  value: {project}\n")
            for k, v in (config or {}).items():
                f.write(f"{k}:\n  value: {v}\n")

    def log(self, metrics: dict, step: int | None = None):
        import json
        import os
        import time
        self._step = self._step + 1 if step is None else step
        rec = {**{k: float(v) for k, v in metrics.items()}, "_step": self._step, "_timestamp": time.time()}
        with open(os.path.join(self.dir, "wandb-history.jsonl"), "a") as f:
            f.write(json.dumps(rec) + "\n")
        self.summary.update(rec)
        with open(os.path.join(self.dir, "wandb-summary.json"), "w") as f:
            json.dump(self.summary, f)
