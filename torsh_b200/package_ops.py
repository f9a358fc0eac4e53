"""Package operations around :class:`torsh_b200.hub.Package` (the operational half of ``crates/torsh-package``):

* delta patches between two package versions with block-level binary diffs (``delta.rs``);
* compression choice per resource from measured ratios (``compression.rs``), de-duplication and size report
  (``optimization.rs``), structural diagnostics (``diagnostics.rs``);
* lazily loaded resources with a memory budget and LRU eviction (``lazy_resources.rs``);
* audit log with a hash chain (``audit.rs``), usage metrics with alert thresholds (``monitoring.rs``);
* backups with retention and verification (``backup.rs``), storage back ends (``storage.rs``), mirrors with health-based
  selection and fail-over (``mirror.rs``), replication with quorum writes and conflict resolution (``replication.rs``);
* static vulnerability scan of packaged code and dependency advisories (``vulnerability.rs``), restricted execution of
  packaged code (``sandbox.rs``), lineage / provenance / compliance records (``governance.rs``);
* import / export of other model package layouts (``format_compat.rs``).
"""
from __future__ import annotations

import ast
import builtins
import bz2
import hashlib
import io
import json
import lzma
import time
import zipfile
import zlib
from collections import OrderedDict
from dataclasses import dataclass
from pathlib import Path

from .hub import Package
from .package_resolver import Requirement, Version


def _sha(b: bytes) -> str:
    return hashlib.sha256(b).hexdigest()


# ================================================================================================ delta patches
def _binary_diff(old: bytes, new: bytes, block: int = 64) -> list:
    """Copy / insert operations: blocks of ``old`` are indexed by content; ``new`` is scanned greedily, extending each
    match as far as it goes."""
    index: dict[bytes, int] = {}
    for off in range(0, max(len(old) - block + 1, 0), block):
        index.setdefault(old[off:off + block], off)
    ops, lit, i = [], bytearray(), 0
    while i < len(new):
        src = index.get(new[i:i + block]) if i + block <= len(new) else None
        if src is None:
            lit.append(new[i])
            i += 1
            continue
        n = block
        while src + n < len(old) and i + n < len(new) and old[src + n] == new[i + n]:
            n += 1
        if lit:
            ops.append(("insert", bytes(lit)))
            lit = bytearray()
        ops.append(("copy", src, n))
        i += n
    if lit:
        ops.append(("insert", bytes(lit)))
    return ops


def _apply_diff(old: bytes, ops: list) -> bytes:
    out = bytearray()
    for op in ops:
        out += old[op[1]:op[1] + op[2]] if op[0] == "copy" else op[1]
    return bytes(out)


@dataclass
class DeltaPatch:
    name: str
    from_version: str
    to_version: str
    operations: list                     # ("add", file, bytes) | ("delete", file) | ("modify", file, diff ops) | ("replace", file, bytes)
    target_hashes: dict
    dependencies: dict

    def size(self) -> int:
        n = 0
        for op in self.operations:
            if op[0] in ("add", "replace"):
                n += len(op[2])
            elif op[0] == "modify":
                n += sum(len(o[1]) if o[0] == "insert" else 16 for o in op[2])
        return n

    def save(self, path, level: int = 6):
        def enc(op):
            if op[0] in ("add", "replace"):
                return [op[0], op[1], op[2].hex()]
            if op[0] == "modify":
                return [op[0], op[1], [[o[0], o[1].hex()] if o[0] == "insert" else list(o) for o in op[2]]]
            return list(op)
        body = json.dumps({**{k: getattr(self, k) for k in ("name", "from_version", "to_version", "target_hashes", "dependencies")},
                           "operations": [enc(o) for o in self.operations]}).encode()
        Path(path).write_bytes(zlib.compress(body, level))

    @classmethod
    def load(cls, path) -> "DeltaPatch":
        d = json.loads(zlib.decompress(Path(path).read_bytes()))
        def dec(op):
            if op[0] in ("add", "replace"):
                return (op[0], op[1], bytes.fromhex(op[2]))
            if op[0] == "modify":
                return (op[0], op[1], [("insert", bytes.fromhex(o[1])) if o[0] == "insert" else tuple(o) for o in op[2]])
            return tuple(op)
        return cls(d["name"], d["from_version"], d["to_version"], [dec(o) for o in d["operations"]], d["target_hashes"], d["dependencies"])


def create_patch(old: Package, new: Package, max_diff_ratio: float = 0.8, block: int = 64) -> DeltaPatch:
    """A file whose diff would exceed ``max_diff_ratio`` of its new size is shipped whole."""
    ops = []
    for k in sorted(set(old.files) - set(new.files)):
        ops.append(("delete", k))
    for k, v in sorted(new.files.items()):
        if k not in old.files:
            ops.append(("add", k, v))
        elif old.files[k] != v:
            diff = _binary_diff(old.files[k], v, block)
            cost = sum(len(o[1]) if o[0] == "insert" else 16 for o in diff)
            ops.append(("modify", k, diff) if cost <= max_diff_ratio * max(len(v), 1) else ("replace", k, v))
    return DeltaPatch(new.name, old.version, new.version, ops, {k: _sha(v) for k, v in new.files.items()}, dict(new.dependencies))


def apply_patch(old: Package, patch: DeltaPatch, verify: bool = True) -> Package:
    if (old.name, old.version) != (patch.name, patch.from_version):
        raise ValueError(f"patch is for {patch.name} {patch.from_version}, not {old.name} {old.version}")
    out = Package(patch.name, patch.to_version, dict(patch.dependencies))
    out.files = dict(old.files)
    for op in patch.operations:
        if op[0] == "delete":
            out.files.pop(op[1])
        elif op[0] in ("add", "replace"):
            out.files[op[1]] = op[2]
        else:
            out.files[op[1]] = _apply_diff(old.files[op[1]], op[2])
    if verify:
        bad = [k for k, v in out.files.items() if _sha(v) != patch.target_hashes.get(k)] + sorted(set(patch.target_hashes) - set(out.files))
        if bad:
            raise IOError(f"patched package does not match its target hashes: {bad}")
    return out


# ================================================================================================ compression / optimisation
_CODECS = {"none": (lambda b, l: b, lambda b: b), "zlib": (lambda b, l: zlib.compress(b, l), zlib.decompress),
           "bz2": (lambda b, l: bz2.compress(b, max(1, min(l, 9))), bz2.decompress),
           "lzma": (lambda b, l: lzma.compress(b, preset=max(0, min(l, 9))), lzma.decompress)}


def compress_data(data: bytes, algorithm: str = "zlib", level: int = 6) -> bytes:
    return _CODECS[algorithm][0](data, level)


def decompress_data(data: bytes, algorithm: str) -> bytes:
    return _CODECS[algorithm][1](data)


class AdvancedCompressor:
    """Strategy ``fast`` / ``balanced`` / ``best`` / ``adaptive``; adaptive tries every codec on a sample and keeps the one
    with the best ratio that is worth it (below ``min_threshold`` bytes or above ``min_ratio`` nothing is compressed)."""

    LEVEL = {"fast": 1, "balanced": 6, "best": 9, "adaptive": 6}

    def __init__(self, strategy: str = "adaptive", min_threshold: int = 64, min_ratio: float = 0.95, sample: int = 1 << 16):
        self.strategy, self.min_threshold, self.min_ratio, self.sample = strategy, min_threshold, min_ratio, sample
        self.stats: dict[str, dict] = {}

    def algorithm_for_resource(self, name: str, data: bytes) -> str:
        if len(data) < self.min_threshold or name.endswith((".zip", ".gz", ".xz", ".png", ".jpg", ".zst")):
            return "none"
        if self.strategy != "adaptive":
            return {"fast": "zlib", "balanced": "zlib", "best": "lzma"}[self.strategy]
        sample = data[:self.sample]
        best = min(("zlib", "bz2", "lzma"), key=lambda a: len(compress_data(sample, a, 6)))
        return best if len(compress_data(sample, best, 6)) <= self.min_ratio * len(sample) else "none"

    def compress_resource(self, name: str, data: bytes) -> tuple[str, bytes]:
        algo = self.algorithm_for_resource(name, data)
        out = compress_data(data, algo, self.LEVEL[self.strategy])
        s = self.stats.setdefault(algo, {"count": 0, "in": 0, "out": 0})
        s["count"], s["in"], s["out"] = s["count"] + 1, s["in"] + len(data), s["out"] + len(out)
        return algo, out

    def overall_ratio(self): return sum(s["out"] for s in self.stats.values()) / max(sum(s["in"] for s in self.stats.values()), 1)
    def space_saved(self): return sum(s["in"] - s["out"] for s in self.stats.values())
    def most_used_algorithm(self): return max(self.stats, key=lambda a: self.stats[a]["count"]) if self.stats else None

    @staticmethod
    def benchmark_algorithms(data: bytes) -> dict:
        out = {}
        for a in ("zlib", "bz2", "lzma"):
            t0 = time.perf_counter()
            c = compress_data(data, a, 6)
            t1 = time.perf_counter()
            assert decompress_data(c, a) == data
            out[a] = {"ratio": len(c) / max(len(data), 1), "compress_s": t1 - t0, "decompress_s": time.perf_counter() - t1}
        return out


class PackageOptimizer:
    def analyze(self, pkg: Package) -> dict:
        by_hash: dict[str, list] = {}
        for k, v in pkg.files.items():
            by_hash.setdefault(_sha(v), []).append(k)
        dup = {h: ks for h, ks in by_hash.items() if len(ks) > 1}
        comp = AdvancedCompressor()
        compressible = {k: len(comp.compress_resource(k, v)[1]) / max(len(v), 1) for k, v in pkg.files.items() if len(v) >= 256}
        return {"total_bytes": sum(map(len, pkg.files.values())),
                "duplicate_groups": list(dup.values()), "duplicate_bytes": sum(len(pkg.files[ks[0]]) * (len(ks) - 1) for ks in dup.values()),
                "compressible": {k: r for k, r in compressible.items() if r < 0.8}, "estimated_compressed_bytes": sum(s["out"] for s in comp.stats.values())}

    def optimize(self, pkg: Package) -> tuple[Package, dict]:
        """Keeps one copy of identical files; the others become entries of ``ALIASES.json`` (alias -> kept file)."""
        out, seen, aliases = Package(pkg.name, pkg.version, dict(pkg.dependencies)), {}, {}
        for k, v in sorted(pkg.files.items()):
            h = _sha(v)
            if h in seen:
                aliases[k] = seen[h]
            else:
                seen[h] = k
                out.files[k] = v
        if aliases:
            out.files["ALIASES.json"] = json.dumps(aliases, sort_keys=True).encode()
        return out, aliases


def resolve_alias(pkg: Package, name: str) -> bytes:
    if name in pkg.files:
        return pkg.files[name]
    return pkg.files[json.loads(pkg.files["ALIASES.json"])[name]]


def diagnose(pkg: Package) -> dict:
    """Structural checks: manifest fields, version syntax, empty or oversized files, code that does not parse, missing model."""
    issues = []
    try:
        Version.parse(pkg.version)
    except Exception:
        issues.append({"severity": "error", "category": "manifest", "message": f"version {pkg.version!r} is not semantic"})
    if not pkg.name or not pkg.name.replace("-", "_").replace(".", "_").isidentifier():
        issues.append({"severity": "error", "category": "manifest", "message": f"bad package name {pkg.name!r}"})
    for k, v in pkg.files.items():
        if not v:
            issues.append({"severity": "warning", "category": "resource", "message": f"{k} is empty"})
        if k.startswith("code/") and k.endswith(".py"):
            try:
                ast.parse(v.decode())
            except (SyntaxError, UnicodeDecodeError) as e:
                issues.append({"severity": "error", "category": "code", "message": f"{k} does not parse: {e}"})
        if ".." in Path(k).parts or k.startswith("/"):
            issues.append({"severity": "error", "category": "security", "message": f"{k} escapes the package root"})
    if not any(k.endswith((".trsm", ".safetensors", ".trsh", ".onnx")) for k in pkg.files):
        issues.append({"severity": "info", "category": "resource", "message": "package holds no model or tensor file"})
    worst = max((["info", "warning", "error"].index(i["severity"]) for i in issues), default=-1)
    return {"health": ["healthy", "healthy", "degraded", "broken"][worst + 1], "issues": issues,
            "statistics": {"files": len(pkg.files), "bytes": sum(map(len, pkg.files.values()))}}


# ================================================================================================ lazy resources
class LazyResourceManager:
    """Reads members of a saved package on first use, within ``memory_limit`` bytes (LRU or largest-first eviction)."""

    def __init__(self, path, memory_limit: int = 1 << 30, eviction: str = "lru"):
        self.path, self.limit, self.eviction = Path(path), memory_limit, eviction
        with zipfile.ZipFile(self.path) as z:
            self.sizes = {i.filename: i.file_size for i in z.infolist() if i.filename not in ("MANIFEST.json", "SIGNATURE", "SIGNATURE.ed25519")}
        self.cache: OrderedDict[str, bytes] = OrderedDict()
        self.loads = 0

    def is_loaded(self, name): return name in self.cache
    def memory_usage(self): return sum(map(len, self.cache.values()))
    def loaded_resources(self): return list(self.cache)

    def get_resource(self, name: str) -> bytes:
        if name in self.cache:
            self.cache.move_to_end(name)
            return self.cache[name]
        with zipfile.ZipFile(self.path) as z:
            data = z.read(name)
        self.loads += 1
        self.cache[name] = data
        while self.memory_usage() > self.limit and len(self.cache) > 1:
            victim = next(iter(self.cache)) if self.eviction == "lru" else max((k for k in self.cache if k != name), key=lambda k: len(self.cache[k]))
            self.cache.pop(victim)
        return data

    def stream(self, name: str, chunk_size: int = 1 << 16):
        with zipfile.ZipFile(self.path) as z, z.open(name) as f:
            while chunk := f.read(chunk_size):
                yield chunk

    def preload(self, names): return [len(self.get_resource(n)) for n in names]
    def evict_all_cache(self): self.cache.clear()


# ================================================================================================ audit / monitoring
class AuditLogger:
    """Append-only JSON-lines log; every record carries the hash of the previous one, so :meth:`validate` finds edits,
    deletions and re-ordering."""

    def __init__(self, path=None):
        self.path, self.events, self.listeners = Path(path) if path else None, [], []
        if self.path and self.path.exists():
            self.events = [json.loads(ln) for ln in self.path.read_text().splitlines() if ln]

    def log(self, event_type: str, resource: str = "", user: str = "", result: str = "success", severity: str = "info", **metadata) -> dict:
        prev = self.events[-1]["hash"] if self.events else "0" * 64
        ev = {"seq": len(self.events), "time": time.time(), "type": event_type, "resource": resource, "user": user, "result": result,
              "severity": severity, "metadata": metadata, "prev": prev}
        ev["hash"] = _sha(json.dumps(ev, sort_keys=True).encode())
        self.events.append(ev)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(ev, sort_keys=True) + "\n")
        for fn in self.listeners:
            fn(ev)
        return ev

    def log_download(self, resource, user=""): return self.log("download", resource, user)
    def log_upload(self, resource, user=""): return self.log("upload", resource, user)
    def log_access_denied(self, resource, user=""): return self.log("access_denied", resource, user, "denied", "warning")
    def log_security_violation(self, resource, detail, user=""): return self.log("security_violation", resource, user, "failure", "critical", detail=detail)
    def add_listener(self, fn): self.listeners.append(fn)

    def query(self, event_type=None, user=None, severity=None, since: float | None = None):
        return [e for e in self.events if (event_type is None or e["type"] == event_type) and (user is None or e["user"] == user)
                and (severity is None or e["severity"] == severity) and (since is None or e["time"] >= since)]

    def validate(self) -> list[int]:
        bad, prev = [], "0" * 64
        for i, e in enumerate(self.events):
            body = {k: v for k, v in e.items() if k != "hash"}
            if e.get("prev") != prev or e.get("seq") != i or _sha(json.dumps(body, sort_keys=True).encode()) != e.get("hash"):
                bad.append(i)
            prev = e.get("hash")
        return bad

    def get_statistics(self):
        by = {}
        for e in self.events:
            by[e["type"]] = by.get(e["type"], 0) + 1
        return {"events": len(self.events), "by_type": by, "denied": sum(e["result"] == "denied" for e in self.events)}


class MetricsCollector:
    def __init__(self, max_points: int = 1000):
        self.max_points, self.series, self.packages, self.users, self.thresholds, self.alerts = max_points, {}, {}, {}, {}, []

    def record_metric(self, name: str, value: float, t: float | None = None):
        s = self.series.setdefault(name, [])
        s.append((t if t is not None else time.time(), float(value)))
        del s[:-self.max_points]
        th = self.thresholds.get(name)
        if th and ((th["kind"] == "above" and value > th["value"]) or (th["kind"] == "below" and value < th["value"])):
            self.alerts.append({"metric": name, "value": value, "severity": th["severity"], "threshold": th["value"]})

    def _bump(self, table, key, field_, n=1):
        table.setdefault(key, {"downloads": 0, "uploads": 0, "errors": 0, "bytes": 0})[field_] += n

    def record_download(self, package, user="", size=0):
        self._bump(self.packages, package, "downloads"); self._bump(self.packages, package, "bytes", size); self._bump(self.users, user, "downloads")
        self.record_metric("downloads", 1)

    def record_upload(self, package, user="", size=0):
        self._bump(self.packages, package, "uploads"); self._bump(self.users, user, "uploads")

    def record_error(self, package, user=""):
        self._bump(self.packages, package, "errors")
        p = self.packages[package]
        self.record_metric("error_rate", p["errors"] / max(p["downloads"] + p["uploads"] + p["errors"], 1))

    def set_alert_threshold(self, metric, value, kind="above", severity="warning"): self.thresholds[metric] = {"value": value, "kind": kind, "severity": severity}
    def get_active_alerts(self): return list(self.alerts)
    def clear_alerts(self): self.alerts.clear()
    def get_package_stats(self, package): return self.packages.get(package)

    def get_time_series(self, name):
        v = [x for _, x in self.series.get(name, [])]
        return {"count": len(v), "min": min(v, default=None), "max": max(v, default=None), "mean": sum(v) / len(v) if v else None}

    def generate_report(self):
        top = sorted(self.packages.items(), key=lambda kv: -kv[1]["downloads"])[:5]
        return {"packages": len(self.packages), "users": len(self.users), "top_packages": [k for k, _ in top], "alerts": len(self.alerts)}


# ================================================================================================ storage / backup / mirrors / replication
class MemoryStorage:
    def __init__(self): self.objects, self.stats = {}, {"puts": 0, "gets": 0, "bytes_in": 0, "bytes_out": 0}
    def put(self, key, data: bytes): self.objects[key] = bytes(data); self.stats["puts"] += 1; self.stats["bytes_in"] += len(data)
    def get(self, key) -> bytes: self.stats["gets"] += 1; self.stats["bytes_out"] += len(self.objects[key]); return self.objects[key]
    def exists(self, key): return key in self.objects
    def delete(self, key): self.objects.pop(key, None)
    def list(self, prefix=""): return sorted(k for k in self.objects if k.startswith(prefix))
    def get_metadata(self, key): return {"size": len(self.objects[key]), "sha256": _sha(self.objects[key])}
    def copy(self, src, dst): self.put(dst, self.objects[src])


class LocalStorage(MemoryStorage):
    """Objects as files under ``root`` (keys may contain ``/``); writes go through a temporary file and a rename."""

    def __init__(self, root):
        super().__init__()
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)

    def _p(self, key):
        p = (self.root / key).resolve()
        if self.root.resolve() not in p.parents:
            raise PermissionError(f"key {key!r} escapes the storage root")
        return p

    def put(self, key, data):
        p = self._p(key)
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_suffix(p.suffix + ".tmp")
        tmp.write_bytes(data)
        tmp.replace(p)
        self.stats["puts"] += 1; self.stats["bytes_in"] += len(data)

    def get(self, key): d = self._p(key).read_bytes(); self.stats["gets"] += 1; self.stats["bytes_out"] += len(d); return d
    def exists(self, key): return self._p(key).is_file()
    def delete(self, key): self._p(key).unlink(missing_ok=True)
    def list(self, prefix=""): return sorted(str(p.relative_to(self.root)) for p in self.root.rglob("*") if p.is_file() and str(p.relative_to(self.root)).startswith(prefix))
    def get_metadata(self, key): d = self._p(key).read_bytes(); return {"size": len(d), "sha256": _sha(d)}
    def copy(self, src, dst): self.put(dst, self.get(src))


def _pkg_bytes(pkg: Package) -> bytes:
    buf = io.BytesIO()
    pkg.save(buf)
    return buf.getvalue()


class BackupManager:
    """Full or incremental (files changed since the previous backup of that package) backups into a storage back end, with
    ``keep_last`` / ``keep_days`` retention, verification against recorded hashes, and restore that replays the chain."""

    def __init__(self, storage, strategy: str = "full"):
        self.storage, self.strategy = storage, strategy
        self.index: list[dict] = json.loads(storage.get("backups/index.json")) if storage.exists("backups/index.json") else []

    def _flush(self): self.storage.put("backups/index.json", json.dumps(self.index).encode())

    def create_backup(self, pkg: Package, now: float | None = None) -> dict:
        prev = next((b for b in reversed(self.index) if b["name"] == pkg.name), None)
        incremental = self.strategy == "incremental" and prev is not None
        hashes = {k: _sha(v) for k, v in pkg.files.items()}
        stored = {k: v for k, v in pkg.files.items() if not incremental or prev["hashes"].get(k) != hashes[k]}
        bid = f"{pkg.name}-{pkg.version}-{len(self.index)}"
        blob = zlib.compress(json.dumps({k: v.hex() for k, v in stored.items()}).encode())
        self.storage.put(f"backups/{bid}.bin", blob)
        meta = {"id": bid, "name": pkg.name, "version": pkg.version, "time": now if now is not None else time.time(), "hashes": hashes,
                "dependencies": pkg.dependencies, "parent": prev["id"] if incremental else None, "blob_sha256": _sha(blob), "stored_files": sorted(stored)}
        self.index.append(meta)
        self._flush()
        return meta

    def list_backups(self, name=None): return [b for b in self.index if name is None or b["name"] == name]

    def verify_backup(self, bid: str) -> dict:
        meta = next(b for b in self.index if b["id"] == bid)
        ok = self.storage.exists(f"backups/{bid}.bin") and _sha(self.storage.get(f"backups/{bid}.bin")) == meta["blob_sha256"]
        return {"id": bid, "valid": ok}

    def restore_backup(self, bid: str) -> Package:
        chain, meta = [], next(b for b in self.index if b["id"] == bid)
        cur = meta
        while cur is not None:
            chain.append(cur)
            cur = next((b for b in self.index if b["id"] == cur["parent"]), None) if cur["parent"] else None
        files: dict[str, bytes] = {}
        for b in reversed(chain):
            if not self.verify_backup(b["id"])["valid"]:
                raise IOError(f"backup {b['id']} is missing or corrupt")
            files.update({k: bytes.fromhex(v) for k, v in json.loads(zlib.decompress(self.storage.get(f"backups/{b['id']}.bin"))).items()})
        pkg = Package(meta["name"], meta["version"], dict(meta["dependencies"]))
        pkg.files = {k: files[k] for k in meta["hashes"]}
        if any(_sha(v) != meta["hashes"][k] for k, v in pkg.files.items()):
            raise IOError("restored files do not match the recorded hashes")
        return pkg

    def apply_retention_policy(self, keep_last: int | None = None, keep_days: float | None = None, now: float | None = None) -> list[str]:
        """Never removes a backup that a kept incremental backup still depends on."""
        now = now if now is not None else time.time()
        keep = set()
        for name in {b["name"] for b in self.index}:
            mine = [b for b in self.index if b["name"] == name]
            kept = mine[-keep_last:] if keep_last else list(mine)
            if keep_days is not None:
                kept = [b for b in kept if now - b["time"] <= keep_days * 86400] or mine[-1:]
            for b in kept:
                while b is not None and b["id"] not in keep:
                    keep.add(b["id"])
                    b = next((p for p in self.index if p["id"] == b["parent"]), None) if b["parent"] else None
        gone = [b["id"] for b in self.index if b["id"] not in keep]
        for bid in gone:
            self.storage.delete(f"backups/{bid}.bin")
        self.index = [b for b in self.index if b["id"] in keep]
        self._flush()
        return gone


@dataclass
class Mirror:
    name: str
    storage: object
    priority: int = 0
    weight: float = 1.0
    region: str = ""
    requests: int = 0
    errors: int = 0
    latency_ms: float = 0.0
    available: bool = True

    @property
    def error_rate(self): return self.errors / max(self.requests, 1)
    @property
    def health(self): return "offline" if not self.available else "unhealthy" if self.error_rate > 0.5 else "degraded" if self.error_rate > 0.1 else "healthy"
    def score(self): return self.weight * (1 - self.error_rate) / (1 + self.latency_ms / 100) + 0.01 * self.priority


class MirrorManager:
    """Selection strategies ``priority`` / ``score`` / ``round_robin`` / ``region``; ``fetch`` fails over down the list and
    records every error, marking a mirror offline after ``max_failures`` consecutive errors."""

    def __init__(self, strategy: str = "score", max_failures: int = 3):
        self.mirrors: dict[str, Mirror] = {}
        self.strategy, self.max_failures, self._rr, self._consecutive, self.failovers = strategy, max_failures, 0, {}, 0

    def add_mirror(self, m: Mirror): self.mirrors[m.name] = m
    def remove_mirror(self, name): self.mirrors.pop(name, None)
    def get_healthy_mirrors(self): return [m for m in self.mirrors.values() if m.health in ("healthy", "degraded")]

    def ranked(self, region: str = "") -> list[Mirror]:
        """Healthy and degraded mirrors in strategy order, then unhealthy ones as a last resort; offline ones never."""
        return self._ordered(self.get_healthy_mirrors(), region) + [m for m in self.mirrors.values() if m.health == "unhealthy"]

    def _ordered(self, ms, region):
        if self.strategy == "priority":
            return sorted(ms, key=lambda m: -m.priority)
        if self.strategy == "round_robin":
            self._rr += 1
            return ms[self._rr % len(ms):] + ms[:self._rr % len(ms)] if ms else []
        if self.strategy == "region":
            return sorted(ms, key=lambda m: (m.region != region, -m.score()))
        return sorted(ms, key=lambda m: -m.score())

    def select_mirror(self, region: str = "") -> Mirror | None:
        r = self._ordered(self.get_healthy_mirrors(), region)
        return r[0] if r else None

    def fetch(self, key: str, region: str = "") -> tuple[str, bytes]:
        for i, m in enumerate(self.ranked(region)):
            m.requests += 1
            t0 = time.perf_counter()
            try:
                data = m.storage.get(key)
            except Exception:
                m.errors += 1
                self._consecutive[m.name] = self._consecutive.get(m.name, 0) + 1
                if self._consecutive[m.name] >= self.max_failures:
                    m.available = False
                self.failovers += 1
                continue
            self._consecutive[m.name] = 0
            m.latency_ms = 0.8 * m.latency_ms + 0.2 * (time.perf_counter() - t0) * 1e3
            return m.name, data
        raise IOError(f"no mirror could serve {key!r}")

    def sync(self, source, keys=None) -> dict:
        """Copies what each mirror lacks (or holds with another hash) from ``source``."""
        copied = {}
        for m in self.mirrors.values():
            for k in keys or source.list():
                if not m.storage.exists(k) or m.storage.get_metadata(k)["sha256"] != source.get_metadata(k)["sha256"]:
                    m.storage.put(k, source.get(k))
                    copied[m.name] = copied.get(m.name, 0) + 1
        return copied


class ReplicationManager:
    """Writes a versioned object to every reachable node and succeeds when ``consistency`` (``one`` / ``quorum`` / ``all``)
    nodes acknowledged; reads take the newest version among a read quorum; ``synchronize`` repairs stale or missing
    replicas and reports conflicts (same version, different content), settled by ``last_write_wins`` or ``highest_hash``."""

    def __init__(self, consistency: str = "quorum", conflict_resolution: str = "last_write_wins"):
        self.nodes: dict[str, dict] = {}
        self.consistency, self.resolution, self.conflicts = consistency, conflict_resolution, []

    def add_node(self, name, storage): self.nodes[name] = {"storage": storage, "online": True}
    def remove_node(self, name): self.nodes.pop(name)
    def set_online(self, name, online: bool): self.nodes[name]["online"] = online
    def _need(self): n = len(self.nodes); return {"one": 1, "quorum": n // 2 + 1, "all": n}[self.consistency]

    def _read(self, node, key):
        st = node["storage"]
        if not node["online"] or not st.exists(key):
            return None
        rec = json.loads(st.get(key))
        return rec

    def replicate_package(self, key: str, data: bytes, now: float | None = None) -> dict:
        cur = [r for n in self.nodes.values() if (r := self._read(n, key))]
        version = 1 + max((r["version"] for r in cur), default=0)
        rec = json.dumps({"version": version, "time": now if now is not None else time.time(), "sha256": _sha(data), "data": data.hex()}).encode()
        acks = []
        for name, n in self.nodes.items():
            if n["online"]:
                n["storage"].put(key, rec)
                acks.append(name)
        ok = len(acks) >= self._need()
        return {"status": "committed" if ok else "failed", "version": version, "acks": acks, "needed": self._need()}

    def get_package(self, key: str) -> bytes:
        recs = [r for n in self.nodes.values() if (r := self._read(n, key))]
        if len(recs) < min(self._need(), len(self.nodes)) or not recs:
            raise IOError(f"read of {key!r} reached {len(recs)} replicas, {self._need()} needed")
        return bytes.fromhex(max(recs, key=lambda r: (r["version"], r["time"]))["data"])

    def synchronize(self, key: str) -> dict:
        recs = {name: r for name, n in self.nodes.items() if (r := self._read(n, key))}
        if not recs:
            return {"repaired": [], "conflicts": 0}
        top = max(r["version"] for r in recs.values())
        heads = {name: r for name, r in recs.items() if r["version"] == top}
        distinct = {r["sha256"] for r in heads.values()}
        if len(distinct) > 1:
            self.conflicts.append({"key": key, "version": top, "hashes": sorted(distinct)})
        pick = max(heads.values(), key=(lambda r: r["time"]) if self.resolution == "last_write_wins" else (lambda r: r["sha256"]))
        blob, repaired = json.dumps(pick).encode(), []
        for name, n in self.nodes.items():
            if n["online"] and (name not in recs or recs[name]["version"] < top or recs[name]["sha256"] != pick["sha256"]):
                n["storage"].put(key, blob)
                repaired.append(name)
        return {"repaired": repaired, "conflicts": int(len(distinct) > 1)}

    def health_check(self): return {name: ("online" if n["online"] else "offline") for name, n in self.nodes.items()}


# ================================================================================================ security
_RISKY_CALLS = {"eval": ("high", "evaluates a string as code"), "exec": ("high", "executes a string as code"),
                "compile": ("medium", "compiles source at run time"), "__import__": ("medium", "dynamic import"),
                "os.system": ("critical", "runs a shell command"), "os.popen": ("critical", "runs a shell command"),
                "subprocess.run": ("high", "starts a process"), "subprocess.Popen": ("high", "starts a process"),
                "subprocess.call": ("high", "starts a process"), "subprocess.check_output": ("high", "starts a process"),
                "pickle.load": ("high", "unpickling runs arbitrary code"), "pickle.loads": ("high", "unpickling runs arbitrary code"),
                "marshal.loads": ("high", "loads code objects"), "ctypes.CDLL": ("high", "loads a native library"),
                "socket.socket": ("medium", "opens a network socket"), "urllib.request.urlopen": ("medium", "network access"),
                "shutil.rmtree": ("medium", "removes directory trees")}
_SEV_W = {"low": 1, "medium": 3, "high": 7, "critical": 15}


def _dotted(node) -> str:
    parts = []
    while isinstance(node, ast.Attribute):
        parts.append(node.attr)
        node = node.value
    if isinstance(node, ast.Name):
        parts.append(node.id)
    return ".".join(reversed(parts))


class VulnerabilityScanner:
    """Walks the syntax tree of packaged Python sources for risky calls, looks for embedded secrets and pickled payloads,
    and matches dependencies against an advisory list ``[{package, affected (specifier), id, severity}]``.
    Policies: ``lenient`` reports high and above, ``standard`` medium and above, ``strict`` everything."""

    FLOOR = {"lenient": 7, "standard": 3, "strict": 1}

    def __init__(self, policy: str = "standard", advisories: list | None = None):
        self.policy, self.advisories = policy, advisories or []

    def scan(self, pkg: Package) -> dict:
        issues = []
        add = lambda sev, kind, comp, msg, **kw: issues.append({"severity": sev, "type": kind, "component": comp, "message": msg, **kw})
        for k, v in pkg.files.items():
            if k.endswith(".py"):
                try:
                    tree = ast.parse(v.decode())
                except (SyntaxError, UnicodeDecodeError):
                    add("medium", "unparseable_code", k, "source does not parse")
                    continue
                for node in ast.walk(tree):
                    if isinstance(node, ast.Call) and (name := _dotted(node.func)) in _RISKY_CALLS:
                        sev, why = _RISKY_CALLS[name]
                        add(sev, "risky_call", k, f"{name}: {why}", line=node.lineno)
                    if isinstance(node, ast.Assign) and isinstance(node.value, ast.Constant) and isinstance(node.value.value, str):
                        names = [t.id.lower() for t in node.targets if isinstance(t, ast.Name)]
                        if any(s in n for n in names for s in ("password", "secret", "api_key", "token")) and len(node.value.value) >= 8:
                            add("high", "embedded_secret", k, f"literal assigned to {names[0]}", line=node.lineno)
            elif v[:2] == b"\x80\x04" or v[:2] == b"\x80\x05" or k.endswith((".pkl", ".pickle")):
                add("high", "pickled_payload", k, "pickle data runs code when loaded")
            if ".." in Path(k).parts or k.startswith("/"):
                add("critical", "path_traversal", k, "member path escapes the package root")
        for dep, spec in pkg.dependencies.items():
            for adv in self.advisories:
                if adv["package"] != dep:
                    continue
                pinned = spec.lstrip("=^~>< ")
                try:
                    hit = Requirement(adv["affected"]).matches(Version.parse(pinned))
                except Exception:
                    hit = False
                if hit:
                    add(adv.get("severity", "high"), "vulnerable_dependency", dep, f"{dep} {pinned} is affected by {adv['id']}", advisory=adv["id"])
        issues = [i for i in issues if _SEV_W[i["severity"]] >= self.FLOOR[self.policy]]
        count = lambda s: sum(i["severity"] == s for i in issues)
        return {"issues": issues, "critical": count("critical"), "high": count("high"), "medium": count("medium"), "low": count("low"),
                "risk_score": min(100, sum(_SEV_W[i["severity"]] for i in issues)), "passed": count("critical") + count("high") == 0}


class SandboxViolation(Exception):
    pass


class Sandbox:
    """Runs packaged source with a reduced set of builtins, an import allow-list, a file policy for ``open`` and an
    instruction budget (``sys.settrace`` line events).  This limits honest code to what a package declares; it is not a
    security boundary against hostile code, which needs a separate process."""

    SAFE_BUILTINS = ("abs all any bool bytes callable chr dict divmod enumerate filter float format frozenset getattr hasattr hash "
                     "int isinstance issubclass iter len list map max min next object ord pow print range repr reversed round set "
                     "setattr slice sorted str sum tuple type zip Exception ValueError TypeError KeyError IndexError RuntimeError "
                     "StopIteration ArithmeticError ZeroDivisionError AttributeError NotImplementedError __build_class__ __name__ "
                     "True False None property staticmethod classmethod super").split()

    def __init__(self, allowed_imports=("math", "json", "torch", "numpy"), read_paths=(), write_paths=(), max_lines: int = 2_000_000):
        self.allowed, self.read_paths, self.write_paths, self.max_lines = set(allowed_imports), [Path(p).resolve() for p in read_paths], [Path(p).resolve() for p in write_paths], max_lines
        self.violations: list[dict] = []

    def _violate(self, kind, detail):
        self.violations.append({"type": kind, "detail": detail})
        raise SandboxViolation(f"{kind}: {detail}")

    def can_read(self, p): return any(r == Path(p).resolve() or r in Path(p).resolve().parents for r in self.read_paths + self.write_paths)
    def can_write(self, p): return any(r == Path(p).resolve() or r in Path(p).resolve().parents for r in self.write_paths)

    def _globals(self):
        def imp(name, globals=None, locals=None, fromlist=(), level=0):
            if name.split(".")[0] not in self.allowed:
                self._violate("import", name)
            return builtins.__import__(name, globals, locals, fromlist, level)

        def opn(path, mode="r", *a, **kw):
            if any(c in mode for c in "wax+"):
                if not self.can_write(path):
                    self._violate("file_write", str(path))
            elif not self.can_read(path):
                self._violate("file_read", str(path))
            return builtins.open(path, mode, *a, **kw)
        b = {k: getattr(builtins, k) for k in self.SAFE_BUILTINS if hasattr(builtins, k)}
        b.update({"__import__": imp, "open": opn, "__build_class__": builtins.__build_class__})
        return {"__builtins__": b, "__name__": "sandboxed"}

    def execute(self, source: str, entry: str | None = None, *args):
        import sys
        g, budget = self._globals(), [self.max_lines]

        def tracer(frame, event, arg):
            if event == "line":
                budget[0] -= 1
                if budget[0] < 0:
                    self._violate("cpu_budget", f"more than {self.max_lines} lines executed")
            return tracer
        code = compile(source, "<sandboxed>", "exec")
        old = sys.gettrace()
        sys.settrace(tracer)
        t0 = time.perf_counter()
        try:
            exec(code, g)
            value = g[entry](*args) if entry else None
        finally:
            sys.settrace(old)
        return {"value": value, "lines_executed": self.max_lines - budget[0], "seconds": time.perf_counter() - t0, "violations": list(self.violations)}

    def execute_package_module(self, pkg: Package, module_name: str, entry: str | None = None, *args):
        return self.execute(pkg.files[f"code/{module_name.replace('.', '/')}.py"].decode(), entry, *args)


# ================================================================================================ governance
class LineageTracker:
    """Directed lineage between package versions (``derived_from`` / ``fine_tuned_from`` / ``quantized_from`` / ...),
    provenance and transformation records, and compliance checks with a report."""

    def __init__(self):
        self.edges: list[dict] = []
        self.provenance: dict[str, dict] = {}
        self.transformations: dict[str, list] = {}
        self.compliance: dict[str, dict] = {}

    def add_lineage(self, child: str, parent: str, relation: str = "derived_from", **metadata):
        if child == parent or child in self.get_ancestors(parent):
            raise ValueError(f"lineage {child} -> {parent} would close a cycle")
        self.edges.append({"child": child, "parent": parent, "relation": relation, "metadata": metadata})

    def _walk(self, start, src, dst):
        seen, stack = [], [start]
        while stack:
            cur = stack.pop()
            for e in self.edges:
                if e[src] == cur and e[dst] not in seen:
                    seen.append(e[dst])
                    stack.append(e[dst])
        return seen

    def get_ancestors(self, pkg): return self._walk(pkg, "child", "parent")
    def get_descendants(self, pkg): return self._walk(pkg, "parent", "child")
    def record_provenance(self, pkg, source: str, creator: str, **info): self.provenance[pkg] = {"source": source, "creator": creator, "time": time.time(), **info}
    def get_provenance(self, pkg): return self.provenance.get(pkg)
    def record_transformation(self, pkg, kind: str, **params): self.transformations.setdefault(pkg, []).append({"kind": kind, "params": params})
    def set_compliance(self, pkg, license: str, level: str = "internal", pii: bool = False, tags=()): self.compliance[pkg] = {"license": license, "level": level, "pii": pii, "tags": list(tags)}

    def generate_compliance_report(self, pkg: str, allowed_licenses=("apache-2.0", "mit", "bsd-3-clause")) -> dict:
        issues = []
        for p in [pkg] + self.get_ancestors(pkg):
            c = self.compliance.get(p)
            if c is None:
                issues.append({"severity": "warning", "package": p, "message": "no compliance record"})
                continue
            if c["license"].lower() not in allowed_licenses:
                issues.append({"severity": "error", "package": p, "message": f"license {c['license']} is not on the allow-list"})
            if c["pii"] and p != pkg and not (self.compliance.get(pkg) or {}).get("pii"):
                issues.append({"severity": "error", "package": p, "message": "ancestor holds personal data but the package is not marked so"})
            if p not in self.provenance:
                issues.append({"severity": "info", "package": p, "message": "no provenance record"})
        return {"package": pkg, "compliant": not any(i["severity"] == "error" for i in issues), "issues": issues, "ancestors": self.get_ancestors(pkg)}

    def export_to_dot(self) -> str:
        return "digraph lineage {\n" + "".join(f'  "{e["parent"]}" -> "{e["child"]}" [label="{e["relation"]}"];\n' for e in self.edges) + "}"

    def export_to_json(self) -> str: return json.dumps({"edges": self.edges, "provenance": self.provenance, "transformations": self.transformations, "compliance": self.compliance}, sort_keys=True)

    def get_statistics(self):
        nodes = {e["child"] for e in self.edges} | {e["parent"] for e in self.edges}
        return {"packages": len(nodes), "edges": len(self.edges), "roots": sorted(n for n in nodes if not self.get_ancestors(n))}


# ================================================================================================ other package layouts
class FormatCompatibilityManager:
    """Converts between this package layout and three directory / archive layouts other tools read:
    ``pytorch`` (a zip with ``data.pt`` written by ``torch.save`` of a state dict plus ``extra/manifest.json``),
    ``huggingface`` (``config.json`` + ``model.safetensors``) and ``mlflow`` (``MLmodel`` YAML + ``data/model.safetensors``
    + ``requirements.txt``)."""

    supported_formats = ("pytorch", "huggingface", "mlflow")

    @staticmethod
    def _state(pkg: Package) -> dict:
        from .serialize import model_state as ms
        name = next(k for k in pkg.files if k.endswith(".trsm"))
        st = ms.decode_binary(pkg.files[name])
        return st

    def export_package(self, pkg: Package, fmt: str, out_dir) -> Path:
        import torch
        from .serialize import model_state as ms
        out = Path(out_dir)
        out.mkdir(parents=True, exist_ok=True)
        st = self._state(pkg)
        tensors = {k: torch.tensor(v["data"], dtype=torch.float32).reshape(v["shape"]) for k, v in st["parameters"].items()}
        if fmt == "pytorch":
            p = out / f"{pkg.name}.pt.zip"
            buf = io.BytesIO()
            torch.save(tensors, buf)
            with zipfile.ZipFile(p, "w") as z:
                z.writestr("data.pt", buf.getvalue())
                z.writestr("extra/manifest.json", json.dumps(pkg.manifest()))
            return p
        if fmt in ("huggingface", "mlflow"):
            d = out if fmt == "huggingface" else out / "data"
            d.mkdir(parents=True, exist_ok=True)
            ms.save_safetensors(st, d / "model.safetensors")
            if fmt == "huggingface":
                (out / "config.json").write_text(json.dumps({"model_type": st.get("metadata", {}).get("architecture", pkg.name), "torsh_package": pkg.name, "version": pkg.version, **(st.get("config") or {})}))
            else:
                (out / "MLmodel").write_text(f"artifact_path: model\nflavors:\n  torsh_b200:\n    model_data: data/model.safetensors\n    package: {pkg.name}\n    version: {pkg.version}\n")
                (out / "requirements.txt").write_text("".join(f"{k}{v if v[:1] in '=<>~^' else '==' + v}\n" for k, v in pkg.dependencies.items()))
            return out
        raise ValueError(f"unknown format {fmt!r}; supported: {self.supported_formats}")

    def import_package(self, path, fmt: str, name: str | None = None, version: str = "0.1.0") -> Package:
        import torch
        from .serialize import model_state as ms
        path = Path(path)
        if fmt == "pytorch":
            with zipfile.ZipFile(path) as z:
                loaded = torch.load(io.BytesIO(z.read("data.pt")), weights_only=True)
                tensors = {k: {"shape": list(v.shape), "dtype": "f32", "data": v.float().reshape(-1).tolist(), "requires_grad": True} for k, v in loaded.items()}
                man = json.loads(z.read("extra/manifest.json")) if "extra/manifest.json" in z.namelist() else {}
            name, version = name or man.get("name", path.stem), man.get("version", version)
        elif fmt == "huggingface":
            cfg = json.loads((path / "config.json").read_text())
            tensors = ms.load_safetensors(path / "model.safetensors")["parameters"]
            name, version = name or cfg.get("torsh_package", path.name), cfg.get("version", version)
        elif fmt == "mlflow":
            import yaml
            ml = yaml.safe_load((path / "MLmodel").read_text())["flavors"]["torsh_b200"]
            tensors = ms.load_safetensors(path / ml["model_data"])["parameters"]
            name, version = name or ml["package"], str(ml.get("version", version))
        else:
            raise ValueError(f"unknown format {fmt!r}; supported: {self.supported_formats}")
        pkg = Package(name, version)
        st = {"parameters": dict(tensors), "config": {}, "metadata": ms._meta(name)}
        pkg.files["model.trsm"] = ms.encode_binary(st)
        return pkg
