"""Services around the model hub (``crates/torsh-hub/src``): transfer control (``bandwidth.rs``, ``retry.rs``,
``download/``), cache management (``cache.rs``), model cards and search (``model_info.rs``, ``metadata.rs``,
``registry.rs``), usage analytics with A/B tests (``analytics.rs``), community records (``community.rs``), tenant quotas and
roles (``enterprise.rs``), imports from ONNX and TensorFlow-layout checkpoints (``onnx.rs``, ``tensorflow.rs``), and text /
SVG visualisation of models and metrics (``visualization.rs``).  Transfers work on local paths and ``file://`` URLs;
network schemes are refused, as in :mod:`torsh_b200.hub`."""
from __future__ import annotations

import hashlib
import json
import math
import os
import shutil
import time
from collections import Counter, defaultdict
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable, Iterable

import torch


# ================================================================================================ transfer control
class BandwidthLimiter:
    """Token bucket in bytes per second with a burst allowance; ``acquire(n)`` returns how long the caller must wait
    (and sleeps through ``sleep`` unless ``sleep=None``)."""

    def __init__(self, bytes_per_second: float, burst: float | None = None, clock=time.monotonic, sleep=time.sleep):
        self.rate, self.capacity, self.clock, self.sleep = bytes_per_second, burst or bytes_per_second, clock, sleep
        self.tokens, self.last, self.total_bytes, self.total_wait = self.capacity, clock(), 0, 0.0

    def acquire(self, n: int) -> float:
        now = self.clock()
        self.tokens = min(self.capacity, self.tokens + (now - self.last) * self.rate)
        self.last = now
        self.tokens -= n
        wait = max(0.0, -self.tokens / self.rate)
        self.total_bytes += n
        self.total_wait += wait
        if wait and self.sleep:
            self.sleep(wait)
        return wait

    def stats(self): return {"bytes": self.total_bytes, "waited_s": self.total_wait, "rate": self.rate}


class BandwidthLimitedReader:
    def __init__(self, fh, limiter: BandwidthLimiter, chunk: int = 1 << 16): self.fh, self.limiter, self.chunk = fh, limiter, chunk

    def read(self, n: int = -1) -> bytes:
        data = self.fh.read(self.chunk if n < 0 else min(n, self.chunk))
        if data:
            self.limiter.acquire(len(data))
        return data

    def __iter__(self):
        while chunk := self.read():
            yield chunk


class AdaptiveBandwidthLimiter(BandwidthLimiter):
    """Raises the rate by 10 % after every ``window`` clean chunks and halves it after an error (AIMD-like)."""

    def __init__(self, bytes_per_second, min_rate=1 << 14, max_rate=1 << 30, window=8, **kw):
        super().__init__(bytes_per_second, **kw)
        self.min_rate, self.max_rate, self.window, self._ok = min_rate, max_rate, window, 0

    def report(self, ok: bool):
        if ok:
            self._ok += 1
            if self._ok % self.window == 0:
                self.rate = min(self.max_rate, self.rate * 1.1)
        else:
            self._ok, self.rate = 0, max(self.min_rate, self.rate / 2)


class RetryPolicy:
    """Exponential back-off with jitter and a circuit breaker: after ``breaker_threshold`` consecutive failed calls the
    circuit opens for ``breaker_cooldown`` seconds and calls fail immediately."""

    def __init__(self, max_attempts=5, base_delay=0.5, max_delay=30.0, multiplier=2.0, jitter=0.1, retry_on=(IOError, TimeoutError), breaker_threshold=3, breaker_cooldown=60.0,
                 clock=time.monotonic, sleep=time.sleep, seed=0):
        self.max_attempts, self.base, self.max_delay, self.mult, self.jitter, self.retry_on = max_attempts, base_delay, max_delay, multiplier, jitter, retry_on
        self.thr, self.cooldown, self.clock, self.sleep = breaker_threshold, breaker_cooldown, clock, sleep
        self.failures, self.opened_at, self.attempts_log = 0, None, []
        self._rng = torch.Generator().manual_seed(seed)

    def delay(self, attempt: int) -> float:
        d = min(self.max_delay, self.base * self.mult ** attempt)
        return d * (1 + self.jitter * (2 * float(torch.rand((), generator=self._rng)) - 1))

    def call(self, fn: Callable, *a, **kw):
        if self.opened_at is not None:
            if self.clock() - self.opened_at < self.cooldown:
                raise ConnectionError("circuit open: recent calls kept failing")
            self.opened_at = None                                             # half-open: one trial call
        last = None
        for attempt in range(self.max_attempts):
            try:
                out = fn(*a, **kw)
                self.failures = 0
                self.attempts_log.append(attempt + 1)
                return out
            except self.retry_on as e:
                last = e
                if attempt + 1 < self.max_attempts:
                    self.sleep(self.delay(attempt))
        self.failures += 1
        self.attempts_log.append(self.max_attempts)
        if self.failures >= self.thr:
            self.opened_at = self.clock()
        raise last


def _sha256(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while chunk := f.read(1 << 20):
            h.update(chunk)
    return h.hexdigest()


class DownloadManager:
    """Resumable, verified copies from local paths or ``file://`` URLs: data goes to ``<dest>.part`` in chunks, an existing
    part file is continued from its length, the SHA-256 is checked before the rename, failures go through the retry policy."""

    def __init__(self, limiter: BandwidthLimiter | None = None, retry: RetryPolicy | None = None, chunk: int = 1 << 20):
        self.limiter, self.retry, self.chunk, self.metrics = limiter, retry or RetryPolicy(sleep=lambda s: None), chunk, []

    @staticmethod
    def _resolve(url: str) -> Path:
        if "://" in str(url) and not str(url).startswith("file://"):
            raise PermissionError(f"refusing {str(url).split(':')[0]}:// transfer: only local paths and file:// URLs are served")
        return Path(str(url)[7:] if str(url).startswith("file://") else url)

    def download(self, url, dest, sha256: str | None = None, opener: Callable | None = None) -> dict:
        src, dest = self._resolve(url), Path(dest)
        part = dest.with_suffix(dest.suffix + ".part")
        dest.parent.mkdir(parents=True, exist_ok=True)
        t0, attempts = time.perf_counter(), [0]

        def once():
            attempts[0] += 1
            done = part.stat().st_size if part.exists() else 0
            with (opener or open)(src, "rb") as f, open(part, "ab") as out:
                f.seek(done)
                while chunk := f.read(self.chunk):
                    if self.limiter:
                        self.limiter.acquire(len(chunk))
                    out.write(chunk)
            return done
        resumed_from = self.retry.call(once)
        if sha256 and _sha256(part) != sha256:
            part.unlink()
            raise IOError(f"{dest.name}: checksum mismatch, partial file removed")
        part.replace(dest)
        rec = {"url": str(url), "bytes": dest.stat().st_size, "resumed_from": resumed_from, "attempts": attempts[0], "seconds": time.perf_counter() - t0}
        self.metrics.append(rec)
        return rec


# ================================================================================================ cache
class CacheManager:
    """Directory cache with an index (size, checksum, last access): LRU eviction to ``max_bytes``, validation that finds
    corrupt or untracked files, age-based cleanup."""

    def __init__(self, root, max_bytes: int = 10 << 30, clock=time.time):
        self.root, self.max_bytes, self.clock = Path(root), max_bytes, clock
        self.root.mkdir(parents=True, exist_ok=True)
        self.index_path = self.root / "index.json"
        self.index = json.loads(self.index_path.read_text()) if self.index_path.exists() else {}
        self.hits = self.misses = 0

    def _save(self): self.index_path.write_text(json.dumps(self.index))

    def put(self, key: str, src) -> Path:
        dst = self.root / hashlib.sha256(key.encode()).hexdigest()[:32]
        shutil.copyfile(src, dst)
        self.index[key] = {"file": dst.name, "bytes": dst.stat().st_size, "sha256": _sha256(dst), "accessed": self.clock(), "created": self.clock()}
        self._evict(keep=key)
        self._save()
        return dst

    def get(self, key: str) -> Path | None:
        e = self.index.get(key)
        if e is None or not (self.root / e["file"]).exists():
            self.misses += 1
            return None
        e["accessed"] = self.clock()
        self.hits += 1
        self._save()
        return self.root / e["file"]

    def total_bytes(self): return sum(e["bytes"] for e in self.index.values())

    def _evict(self, keep=None):
        for k in sorted(self.index, key=lambda k: self.index[k]["accessed"]):
            if self.total_bytes() <= self.max_bytes:
                break
            if k != keep:
                self.remove(k)

    def remove(self, key):
        e = self.index.pop(key, None)
        if e:
            (self.root / e["file"]).unlink(missing_ok=True)

    def validate(self) -> dict:
        corrupt = [k for k, e in self.index.items() if not (self.root / e["file"]).exists() or _sha256(self.root / e["file"]) != e["sha256"]]
        tracked = {e["file"] for e in self.index.values()} | {"index.json"}
        return {"corrupt": corrupt, "untracked": sorted(p.name for p in self.root.iterdir() if p.name not in tracked), "entries": len(self.index)}

    def cleanup(self, max_age_s: float | None = None, remove_corrupt: bool = True) -> dict:
        v = self.validate()
        gone = list(v["corrupt"]) if remove_corrupt else []
        if max_age_s is not None:
            gone += [k for k, e in self.index.items() if self.clock() - e["accessed"] > max_age_s and k not in gone]
        freed = sum(self.index[k]["bytes"] for k in gone)
        for k in gone:
            self.remove(k)
        for name in v["untracked"]:
            (self.root / name).unlink()
        self._save()
        return {"removed": gone, "freed_bytes": freed, "untracked_removed": v["untracked"]}

    def stats(self): return {"entries": len(self.index), "bytes": self.total_bytes(), "hit_rate": self.hits / max(self.hits + self.misses, 1)}


# ================================================================================================ model cards and search
@dataclass
class ModelCard:
    name: str
    version: str = "1.0.0"
    task: str = ""
    architecture: str = ""
    license: str = ""
    description: str = ""
    tags: list = field(default_factory=list)
    metrics: dict = field(default_factory=dict)
    parameters: int = 0
    datasets: list = field(default_factory=list)
    languages: list = field(default_factory=list)
    limitations: str = ""

    def validate(self) -> list[str]:
        issues = []
        if not self.name or "/" in self.name.strip("/") and self.name.count("/") > 1:
            issues.append("name must be 'model' or 'owner/model'")
        parts = self.version.split(".")
        if len(parts) != 3 or not all(p.isdigit() for p in parts):
            issues.append("version must be MAJOR.MINOR.PATCH")
        issues += [f"{f} is empty" for f in ("task", "license", "description") if not getattr(self, f)]
        issues += [f"metric {k} is not a number" for k, v in self.metrics.items() if not isinstance(v, (int, float))]
        return issues

    def to_markdown(self) -> str:
        rows = "".join(f"| {k} | {v} |\n" for k, v in self.metrics.items())
        return (f"# {self.name}\n\n{self.description}\n\n- task: {self.task}\n- architecture: {self.architecture}\n- parameters: {self.parameters:,}\n- license: {self.license}\n"
                f"- tags: {', '.join(self.tags)}\n\n| metric | value |\n|---|---|\n{rows}" + (f"\n## Limitations\n\n{self.limitations}\n" if self.limitations else ""))

    @classmethod
    def from_model(cls, name, model: torch.nn.Module, **kw): return cls(name, architecture=type(model).__name__, parameters=sum(p.numel() for p in model.parameters()), **kw)


class ModelRegistry:
    """In-memory catalogue of cards with text search (name / description / tags, scored), filters and sorting."""

    def __init__(self): self.cards: dict[str, ModelCard] = {}
    def register(self, card: ModelCard):
        issues = card.validate()
        if issues:
            raise ValueError("; ".join(issues))
        self.cards[f"{card.name}@{card.version}"] = card
    def versions(self, name): return sorted((c.version for c in self.cards.values() if c.name == name), key=lambda v: tuple(map(int, v.split("."))))
    def latest(self, name): return self.cards[f"{name}@{self.versions(name)[-1]}"]

    def search(self, query: str = "", task: str | None = None, tags: Iterable[str] = (), license: str | None = None, max_parameters: int | None = None,
               min_metric: tuple[str, float] | None = None, sort_by: str = "relevance") -> list[ModelCard]:
        words = query.lower().split()
        out = []
        for c in self.cards.values():
            if task and c.task != task or license and c.license != license or max_parameters and c.parameters > max_parameters:
                continue
            if not set(tags) <= set(c.tags) or (min_metric and c.metrics.get(min_metric[0], -math.inf) < min_metric[1]):
                continue
            score = sum(3 * (w in c.name.lower()) + 2 * any(w in t.lower() for t in c.tags) + (w in c.description.lower()) for w in words)
            if words and score == 0:
                continue
            out.append((score, c))
        key = {"relevance": lambda t: -t[0], "parameters": lambda t: t[1].parameters, "name": lambda t: t[1].name}.get(sort_by) or (lambda t: -t[1].metrics.get(sort_by, -math.inf))
        return [c for _, c in sorted(out, key=key)]


# ================================================================================================ analytics
class AnalyticsManager:
    """Usage events (download / load / inference / error) per model and user, with summaries, trends and export."""

    def __init__(self, clock=time.time): self.events, self.clock = [], clock
    def record(self, kind: str, model: str, user: str = "", **data): self.events.append({"t": self.clock(), "kind": kind, "model": model, "user": user, **data})

    def summary(self, model: str | None = None) -> dict:
        ev = [e for e in self.events if model is None or e["model"] == model]
        lat = sorted(e["latency_ms"] for e in ev if "latency_ms" in e)
        return {"events": len(ev), "by_kind": dict(Counter(e["kind"] for e in ev)), "unique_users": len({e["user"] for e in ev if e["user"]}),
                "error_rate": sum(e["kind"] == "error" for e in ev) / max(len(ev), 1), "p50_latency_ms": lat[len(lat) // 2] if lat else None,
                "p95_latency_ms": lat[min(len(lat) - 1, int(0.95 * len(lat)))] if lat else None}

    def popular(self, k: int = 5, kind: str = "download"): return Counter(e["model"] for e in self.events if e["kind"] == kind).most_common(k)

    def trend(self, model: str, bucket_s: float = 86400.0, kind: str = "download") -> list[tuple[float, int]]:
        c = Counter(math.floor(e["t"] / bucket_s) * bucket_s for e in self.events if e["model"] == model and e["kind"] == kind)
        return sorted(c.items())

    def export(self, path): Path(path).write_text("\n".join(json.dumps(e) for e in self.events))


class ABTest:
    """Deterministic assignment of users to variants by hash and weight, metric collection per variant, and a two-sided
    z-test on conversion rates (or Welch test on means) to name a winner."""

    def __init__(self, name: str, variants: dict[str, float]):
        total = sum(variants.values())
        self.name, self.variants = name, {k: v / total for k, v in variants.items()}
        self.obs: dict[str, list] = {k: [] for k in variants}

    def assign(self, user: str) -> str:
        u = int(hashlib.sha256(f"{self.name}:{user}".encode()).hexdigest()[:12], 16) / 16 ** 12
        acc = 0.0
        for k, w in self.variants.items():
            acc += w
            if u < acc:
                return k
        return k

    def record(self, user: str, value: float): self.obs[self.assign(user)].append(float(value))

    def result(self, a: str, b: str, alpha: float = 0.05) -> dict:
        xa, xb = self.obs[a], self.obs[b]
        ma, mb = sum(xa) / len(xa), sum(xb) / len(xb)
        va = sum((v - ma) ** 2 for v in xa) / max(len(xa) - 1, 1)
        vb = sum((v - mb) ** 2 for v in xb) / max(len(xb) - 1, 1)
        z = (mb - ma) / math.sqrt(va / len(xa) + vb / len(xb) + 1e-30)
        p = math.erfc(abs(z) / math.sqrt(2))
        return {"mean": {a: ma, b: mb}, "n": {a: len(xa), b: len(xb)}, "z": z, "p_value": p, "significant": p < alpha, "winner": (b if z > 0 else a) if p < alpha else None,
                "lift": (mb - ma) / abs(ma) if ma else math.inf}


# ================================================================================================ community / enterprise
class CommunityManager:
    """Ratings (one per user, latest wins), threaded comments, badges from thresholds, and challenges with a leaderboard."""

    BADGES = [("popular", lambda s: s["downloads"] >= 1000), ("well_rated", lambda s: s["ratings"] >= 5 and s["mean_rating"] >= 4.5), ("discussed", lambda s: s["comments"] >= 10)]

    def __init__(self):
        self.ratings: dict[str, dict[str, int]] = defaultdict(dict)
        self.comments: dict[str, list] = defaultdict(list)
        self.downloads: Counter = Counter()
        self.challenges: dict[str, dict] = {}

    def rate(self, model, user, stars: int):
        if not 1 <= stars <= 5:
            raise ValueError("stars must be 1..5")
        self.ratings[model][user] = stars

    def comment(self, model, user, text, parent: int | None = None) -> int:
        if parent is not None and not 0 <= parent < len(self.comments[model]):
            raise KeyError(f"no comment {parent} on {model}")
        self.comments[model].append({"id": len(self.comments[model]), "user": user, "text": text, "parent": parent})
        return len(self.comments[model]) - 1

    def thread(self, model, root: int) -> list[dict]:
        out, frontier = [], [root]
        while frontier:
            cur = frontier.pop(0)
            out.append(self.comments[model][cur])
            frontier += [c["id"] for c in self.comments[model] if c["parent"] == cur]
        return out

    def stats(self, model):
        r = list(self.ratings[model].values())
        return {"ratings": len(r), "mean_rating": sum(r) / len(r) if r else 0.0, "comments": len(self.comments[model]), "downloads": self.downloads[model]}

    def badges(self, model): s = self.stats(model); return [name for name, rule in self.BADGES if rule(s)]

    def create_challenge(self, name, metric: str, higher_is_better=True, deadline: float | None = None): self.challenges[name] = {"metric": metric, "hib": higher_is_better, "deadline": deadline, "subs": []}

    def submit(self, challenge, user, model, score: float, now: float | None = None):
        c = self.challenges[challenge]
        if c["deadline"] is not None and (now if now is not None else time.time()) > c["deadline"]:
            raise PermissionError("the challenge is closed")
        c["subs"].append({"user": user, "model": model, "score": score})

    def leaderboard(self, challenge, k: int = 10):
        c = self.challenges[challenge]
        best: dict[str, dict] = {}
        for s in c["subs"]:
            if s["user"] not in best or (s["score"] > best[s["user"]]["score"]) == c["hib"]:
                best[s["user"]] = s
        return sorted(best.values(), key=lambda s: -s["score"] if c["hib"] else s["score"])[:k]


class EnterpriseManager:
    """Tenants with role-based permissions, storage and request quotas, and a compliance label per model that gates who may
    download it."""

    ROLES = {"viewer": {"read"}, "developer": {"read", "write"}, "admin": {"read", "write", "delete", "manage"}}
    LEVELS = ["public", "internal", "confidential", "restricted"]

    def __init__(self):
        self.tenants: dict[str, dict] = {}
        self.labels: dict[str, str] = {}

    def create_tenant(self, name, storage_quota: int = 1 << 30, monthly_requests: int = 100000): self.tenants[name] = {"users": {}, "quota": storage_quota, "used": 0, "req_quota": monthly_requests, "requests": 0, "clearance": {}}
    def add_user(self, tenant, user, role="viewer", clearance="internal"): self.tenants[tenant]["users"][user] = role; self.tenants[tenant]["clearance"][user] = clearance
    def label_model(self, model, level): assert level in self.LEVELS; self.labels[model] = level

    def authorize(self, tenant, user, action, model: str | None = None) -> bool:
        t = self.tenants.get(tenant)
        if t is None or user not in t["users"] or action not in self.ROLES[t["users"][user]]:
            return False
        if model is not None and self.LEVELS.index(self.labels.get(model, "public")) > self.LEVELS.index(t["clearance"][user]):
            return False
        return True

    def charge_storage(self, tenant, nbytes):
        t = self.tenants[tenant]
        if t["used"] + nbytes > t["quota"]:
            raise PermissionError(f"{tenant}: storage quota of {t['quota']} bytes exceeded")
        t["used"] += nbytes

    def charge_request(self, tenant):
        t = self.tenants[tenant]
        if t["requests"] >= t["req_quota"]:
            raise PermissionError(f"{tenant}: request quota spent")
        t["requests"] += 1

    def usage_report(self, tenant): t = self.tenants[tenant]; return {"storage": t["used"] / t["quota"], "requests": t["requests"] / t["req_quota"], "users": len(t["users"])}


# ================================================================================================ imports
def load_onnx_model(path_or_bytes):
    """An ONNX file as a callable evaluator (the package's own protobuf reader and operator set)."""
    from . import onnx_io
    return onnx_io.load_onnx(path_or_bytes)


def import_tensorflow_checkpoint(weights: dict, model: torch.nn.Module) -> dict:
    """Name and layout conversion of a TensorFlow-style ``{name: array}`` checkpoint into ``model``; returns the load report."""
    from .nn.tools import ModelConverter
    conv = ModelConverter()
    return conv.fit(model, conv.from_tensorflow({k: torch.as_tensor(v) for k, v in weights.items()}))


# ================================================================================================ visualisation
def model_tree(model: torch.nn.Module, max_depth: int = 3) -> str:
    """Indented module tree with parameter counts."""
    lines = []
    def walk(m, name, depth):
        n = sum(p.numel() for p in m.parameters())
        lines.append(f"{'  ' * depth}{name or type(m).__name__}: {type(m).__name__} ({n:,})")
        if depth < max_depth:
            for cn, c in m.named_children():
                walk(c, cn, depth + 1)
    walk(model, "", 0)
    return "\n".join(lines)


def sparkline(values) -> str:
    bars, v = "▁▂▃▄▅▆▇█", list(values)
    lo, hi = min(v), max(v)
    return "".join(bars[int((x - lo) / (hi - lo) * 7) if hi > lo else 0] for x in v)


def line_chart_svg(series: dict[str, list[float]], width: int = 480, height: int = 240, title: str = "") -> str:
    """Multi-series line chart as stand-alone SVG text (axes, polylines, legend)."""
    pad = 36
    allv = [v for s in series.values() for v in s]
    lo, hi, n = min(allv), max(allv), max(len(s) for s in series.values())
    sx, sy = (width - 2 * pad) / max(n - 1, 1), (height - 2 * pad) / ((hi - lo) or 1.0)
    colors = ["#1f77b4", "#d62728", "#2ca02c", "#9467bd", "#ff7f0e"]
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}">', f'<text x="{width / 2}" y="16" text-anchor="middle">{title}</text>',
             f'<line x1="{pad}" y1="{height - pad}" x2="{width - pad}" y2="{height - pad}" stroke="black"/>', f'<line x1="{pad}" y1="{pad}" x2="{pad}" y2="{height - pad}" stroke="black"/>',
             f'<text x="4" y="{pad + 4}" font-size="10">{hi:.3g}</text>', f'<text x="4" y="{height - pad}" font-size="10">{lo:.3g}</text>']
    for i, (name, s) in enumerate(series.items()):
        pts = " ".join(f"{pad + k * sx:.1f},{height - pad - (v - lo) * sy:.1f}" for k, v in enumerate(s))
        parts.append(f'<polyline fill="none" stroke="{colors[i % 5]}" points="{pts}"/>')
        parts.append(f'<text x="{width - pad - 80}" y="{pad + 12 * i}" font-size="10" fill="{colors[i % 5]}">{name}</text>')
    return "\n".join(parts + ["</svg>"])


def compare_models(a: torch.nn.Module, b: torch.nn.Module) -> dict:
    """Structural and weight comparison of two modules with the same parameter names."""
    sa, sb = dict(a.named_parameters()), dict(b.named_parameters())
    shared = [k for k in sa if k in sb and sa[k].shape == sb[k].shape]
    diff = {k: float((sa[k].detach() - sb[k].detach()).norm() / sa[k].detach().norm().clamp(min=1e-12)) for k in shared}
    return {"only_in_a": sorted(set(sa) - set(sb)), "only_in_b": sorted(set(sb) - set(sa)), "shape_mismatch": sorted(k for k in sa if k in sb and sa[k].shape != sb[k].shape),
            "relative_difference": diff, "identical": sorted(k for k, v in diff.items() if v == 0), "most_changed": sorted(diff, key=diff.get, reverse=True)[:5]}
