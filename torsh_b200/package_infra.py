"""Package infrastructure (``crates/torsh-package/src``): installation plans with rollback (``dependency_installer.rs``), lock files
with content hashes and drift reports (``dependency_lockfile.rs``), an edge cache network with regional routing and
invalidation (``cdn.rs``), an object-store interface with multipart uploads, signed URLs and versioning over a directory
(``cloud_storage.rs``), RFC 5424 syslog records (``syslog_integration.rs``) and segmented, indexed, tamper-evident audit
storage with retention (``audit_storage.rs``).  Network services are modelled on local directories and sockets: nothing here
needs a network."""
from __future__ import annotations

import base64
import hashlib
import hmac
import json
import os
import shutil
import socket
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Sequence

from .package_resolver import PackageIndex, Requirement, Version, resolve


# ================================================================================================ lock file
class Lockfile:
    """Pinned versions with the hash of each artefact and the requirement set they were resolved from."""

    def __init__(self, packages: dict[str, dict], roots: dict[str, str]): self.packages, self.roots = packages, roots

    @classmethod
    def generate(cls, index: PackageIndex, roots: dict[str, str], artefacts: Callable[[str, str], bytes]) -> "Lockfile":
        res = resolve(index, roots)
        pk = {}
        for name, ver in sorted(res.items()):
            deps = index.releases[name][Version.parse(str(ver))]
            pk[name] = {"version": str(ver), "sha256": hashlib.sha256(artefacts(name, str(ver))).hexdigest(), "dependencies": {k: str(v) for k, v in deps.items()}}
        return cls(pk, dict(roots))

    def dumps(self) -> str:
        body = {"lock_version": 1, "roots": self.roots, "packages": self.packages}
        body["content_hash"] = hashlib.sha256(json.dumps({"roots": self.roots, "packages": self.packages}, sort_keys=True).encode()).hexdigest()
        return json.dumps(body, indent=1, sort_keys=True)

    @classmethod
    def loads(cls, text: str) -> "Lockfile":
        d = json.loads(text)
        want = hashlib.sha256(json.dumps({"roots": d["roots"], "packages": d["packages"]}, sort_keys=True).encode()).hexdigest()
        if d.get("content_hash") != want:
            raise ValueError("lock file was edited by hand: content hash does not match")
        return cls(d["packages"], d["roots"])

    def is_current(self, roots: dict[str, str]) -> bool: return roots == self.roots

    def verify(self, artefacts: Callable[[str, str], bytes]) -> list[str]:
        return [n for n, p in self.packages.items() if hashlib.sha256(artefacts(n, p["version"])).hexdigest() != p["sha256"]]

    def diff(self, other: "Lockfile") -> dict:
        a, b = self.packages, other.packages
        return {"added": sorted(set(b) - set(a)), "removed": sorted(set(a) - set(b)), "changed": {n: (a[n]["version"], b[n]["version"]) for n in sorted(set(a) & set(b)) if a[n]["version"] != b[n]["version"]}}


# ================================================================================================ installer
class InstallError(RuntimeError):
    pass


class DependencyInstaller:
    """Installs locked packages into ``target/<name>-<version>/`` in dependency order; every artefact is checked against the
    lock's hash; a failure removes what this run installed (the directory is left as it was)."""

    def __init__(self, target, artefacts: Callable[[str, str], bytes]): self.target, self.fetch, self.log = Path(target), artefacts, []

    def plan(self, lock: Lockfile) -> list[str]:
        order, seen = [], set()
        def visit(n, stack=()):
            if n in stack:
                raise InstallError(f"dependency cycle: {' -> '.join(stack + (n,))}")
            if n in seen or n not in lock.packages:
                return
            for d in sorted(lock.packages[n]["dependencies"]):
                visit(d, stack + (n,))
            seen.add(n); order.append(n)
        for n in sorted(lock.packages):
            visit(n)
        return order

    def installed(self) -> dict[str, str]:
        out = {}
        if self.target.exists():
            for d in self.target.iterdir():
                if d.is_dir() and (d / ".installed").exists():
                    name, _, ver = d.name.rpartition("-")
                    out[name] = ver
        return out

    def install(self, lock: Lockfile, post_install: Callable[[str, Path], None] | None = None) -> dict:
        self.target.mkdir(parents=True, exist_ok=True)
        have, done, skipped = self.installed(), [], []
        try:
            for name in self.plan(lock):
                p = lock.packages[name]
                if have.get(name) == p["version"]:
                    skipped.append(name); continue
                data = self.fetch(name, p["version"])
                if hashlib.sha256(data).hexdigest() != p["sha256"]:
                    raise InstallError(f"{name} {p['version']}: artefact hash differs from the lock file")
                dest = self.target / f"{name}-{p['version']}"
                dest.mkdir(exist_ok=True)
                done.append(dest)
                (dest / "payload.bin").write_bytes(data)
                if post_install:
                    post_install(name, dest)
                (dest / ".installed").write_text(p["sha256"])
                if name in have:                                                   # an upgrade replaces the old version
                    shutil.rmtree(self.target / f"{name}-{have[name]}", ignore_errors=True)
                self.log.append(("installed", name, p["version"]))
        except Exception as e:
            for d in done:
                shutil.rmtree(d, ignore_errors=True)
            self.log.append(("rolled_back", [d.name for d in done]))
            raise InstallError(str(e)) from e
        return {"installed": [d.name for d in done], "skipped": skipped}

    def uninstall_unlisted(self, lock: Lockfile) -> list[str]:
        gone = []
        for name, ver in self.installed().items():
            if name not in lock.packages:
                shutil.rmtree(self.target / f"{name}-{ver}"); gone.append(name)
        return sorted(gone)


# ================================================================================================ CDN
@dataclass
class EdgeNode:
    name: str
    region: str
    latency_ms: dict                                                                 # client region -> latency
    capacity: int = 1 << 20
    cache: "OrderedDict[str, tuple[bytes, float]]" = field(default_factory=OrderedDict)
    used: int = 0
    hits: int = 0
    misses: int = 0
    online: bool = True


class ContentDeliveryNetwork:
    """Requests go to the online edge with the lowest latency for the client's region; an edge serves from its cache (LRU,
    byte-bounded, entries expire after ``ttl``) and fills from the origin on a miss."""

    def __init__(self, origin: Callable[[str], bytes], ttl: float = 3600.0, clock=time.monotonic): self.origin, self.ttl, self.clock, self.edges, self.origin_fetches = origin, ttl, clock, [], 0
    def add_edge(self, edge: EdgeNode): self.edges.append(edge); return self

    def route(self, client_region: str) -> EdgeNode:
        live = [e for e in self.edges if e.online]
        if not live:
            raise ConnectionError("no edge node is online")
        return min(live, key=lambda e: e.latency_ms.get(client_region, 1e9))

    def get(self, key: str, client_region: str) -> tuple[bytes, dict]:
        e = self.route(client_region)
        now = self.clock()
        if key in e.cache and now - e.cache[key][1] <= self.ttl:
            e.hits += 1; e.cache.move_to_end(key)
            return e.cache[key][0], {"edge": e.name, "cache": "hit", "latency_ms": e.latency_ms.get(client_region)}
        if key in e.cache:
            e.used -= len(e.cache.pop(key)[0])
        e.misses += 1; self.origin_fetches += 1
        data = self.origin(key)
        if len(data) <= e.capacity:
            while e.used + len(data) > e.capacity:
                _, (old, _) = e.cache.popitem(last=False); e.used -= len(old)
            e.cache[key] = (data, now); e.used += len(data)
        return data, {"edge": e.name, "cache": "miss", "latency_ms": e.latency_ms.get(client_region)}

    def invalidate(self, prefix: str = "") -> int:
        n = 0
        for e in self.edges:
            for k in [k for k in e.cache if k.startswith(prefix)]:
                e.used -= len(e.cache.pop(k)[0]); n += 1
        return n

    def prefetch(self, keys: Sequence[str], regions: Sequence[str]):
        for r in regions:
            for k in keys:
                self.get(k, r)

    def statistics(self) -> dict:
        h, m = sum(e.hits for e in self.edges), sum(e.misses for e in self.edges)
        return {"hit_rate": h / (h + m) if h + m else 0.0, "origin_fetches": self.origin_fetches, "edges": {e.name: {"hits": e.hits, "misses": e.misses, "bytes": e.used, "online": e.online} for e in self.edges}}


# ================================================================================================ object store
class ObjectStore:
    """Bucket / key interface of cloud object stores over a directory: put / get / list / delete, object versions,
    multipart uploads assembled on completion, ETags and time-limited signed URLs checked with HMAC."""

    def __init__(self, root, secret: bytes = b"local-secret", versioning: bool = False, clock=time.time):
        self.root, self.secret, self.versioning, self.clock, self._uploads = Path(root), secret, versioning, clock, {}
        self.root.mkdir(parents=True, exist_ok=True)

    def _path(self, bucket, key): return self.root / bucket / base64.urlsafe_b64encode(key.encode()).decode()

    def put(self, bucket: str, key: str, data: bytes, metadata: dict | None = None) -> dict:
        p = self._path(bucket, key)
        p.mkdir(parents=True, exist_ok=True)
        versions = sorted(int(f.stem) for f in p.glob("*.bin"))
        v = (versions[-1] + 1) if versions else 1
        if not self.versioning:
            for old in versions:
                (p / f"{old}.bin").unlink(); (p / f"{old}.json").unlink(missing_ok=True)
        (p / f"{v}.bin").write_bytes(data)
        etag = hashlib.md5(data).hexdigest()                                      # noqa: S324 - an ETag, not a security measure
        (p / f"{v}.json").write_text(json.dumps({"etag": etag, "size": len(data), "metadata": metadata or {}, "modified": self.clock()}))
        return {"etag": etag, "version": v}

    def _latest(self, bucket, key, version=None):
        p = self._path(bucket, key)
        versions = sorted(int(f.stem) for f in p.glob("*.bin")) if p.exists() else []
        if not versions or (version is not None and version not in versions):
            raise KeyError(f"{bucket}/{key}" + (f" version {version}" if version else ""))
        return p, version or versions[-1]

    def get(self, bucket: str, key: str, version: int | None = None, byte_range: tuple[int, int] | None = None) -> bytes:
        p, v = self._latest(bucket, key, version)
        data = (p / f"{v}.bin").read_bytes()
        return data[byte_range[0]:byte_range[1] + 1] if byte_range else data

    def head(self, bucket: str, key: str) -> dict:
        p, v = self._latest(bucket, key)
        return {**json.loads((p / f"{v}.json").read_text()), "version": v}

    def list(self, bucket: str, prefix: str = "") -> list[str]:
        b = self.root / bucket
        keys = [base64.urlsafe_b64decode(d.name.encode()).decode() for d in b.iterdir() if any(d.glob("*.bin"))] if b.exists() else []
        return sorted(k for k in keys if k.startswith(prefix))

    def versions(self, bucket: str, key: str) -> list[int]: return sorted(int(f.stem) for f in self._path(bucket, key).glob("*.bin"))
    def delete(self, bucket: str, key: str): shutil.rmtree(self._path(bucket, key), ignore_errors=True)

    def create_multipart(self, bucket: str, key: str) -> str:
        uid = hashlib.sha1(f"{bucket}/{key}/{len(self._uploads)}/{self.clock()}".encode()).hexdigest()[:16]   # noqa: S324
        self._uploads[uid] = (bucket, key, {})
        return uid

    def upload_part(self, upload_id: str, part_number: int, data: bytes) -> str:
        self._uploads[upload_id][2][part_number] = data
        return hashlib.md5(data).hexdigest()                                      # noqa: S324

    def complete_multipart(self, upload_id: str, parts: Sequence[tuple[int, str]]) -> dict:
        bucket, key, have = self._uploads.pop(upload_id)
        for n, etag in parts:
            if n not in have or hashlib.md5(have[n]).hexdigest() != etag:         # noqa: S324
                self._uploads[upload_id] = (bucket, key, have)
                raise ValueError(f"part {n} is missing or its ETag differs")
        return self.put(bucket, key, b"".join(have[n] for n, _ in sorted(parts)))

    def abort_multipart(self, upload_id: str): self._uploads.pop(upload_id, None)

    def presign(self, bucket: str, key: str, expires_in: float = 600.0, method: str = "GET") -> str:
        exp = int(self.clock() + expires_in)
        sig = hmac.new(self.secret, f"{method}\n{bucket}\n{key}\n{exp}".encode(), hashlib.sha256).hexdigest()
        return f"store://{bucket}/{key}?method={method}&expires={exp}&signature={sig}"

    def open_presigned(self, url: str, method: str = "GET") -> bytes:
        path, _, query = url.removeprefix("store://").partition("?")
        bucket, _, key = path.partition("/")
        q = dict(kv.split("=") for kv in query.split("&"))
        want = hmac.new(self.secret, f"{q['method']}\n{bucket}\n{key}\n{q['expires']}".encode(), hashlib.sha256).hexdigest()
        if not hmac.compare_digest(want, q["signature"]) or q["method"] != method:
            raise PermissionError("signature does not match")
        if self.clock() > int(q["expires"]):
            raise PermissionError("the signed URL has expired")
        return self.get(bucket, key)


# ================================================================================================ syslog
SEVERITY = {"emergency": 0, "alert": 1, "critical": 2, "error": 3, "warning": 4, "notice": 5, "info": 6, "debug": 7}
FACILITY = {"kern": 0, "user": 1, "daemon": 3, "auth": 4, "local0": 16, "local1": 17, "local7": 23}


def format_syslog(message: str, severity: str = "info", facility: str = "local0", app: str = "torsh", hostname: str | None = None, procid: str | int | None = None, msgid: str = "-", structured: dict[str, dict] | None = None, timestamp: float | None = None) -> str:
    """One RFC 5424 record: ``<PRI>1 TIMESTAMP HOST APP PROCID MSGID [SD-ID k="v" ...] MSG`` (structured values escape ``"``, ``\\`` and ``]``)."""
    pri = FACILITY[facility] * 8 + SEVERITY[severity]
    t = time.gmtime(timestamp if timestamp is not None else time.time())
    frac = f"{(timestamp or 0) % 1:.3f}"[1:] if timestamp is not None else ".000"
    ts = time.strftime("%Y-%m-%dT%H:%M:%S", t) + frac + "Z"
    esc = lambda v: str(v).replace("\\", "\\\\").replace('"', '\\"').replace("]", "\\]")
    sd = "".join("[" + sid + "".join(f' {k}="{esc(v)}"' for k, v in kv.items()) + "]" for sid, kv in (structured or {}).items()) or "-"
    return f"<{pri}>1 {ts} {hostname or socket.gethostname() or '-'} {app} {procid if procid is not None else os.getpid()} {msgid} {sd} {message}"


def parse_syslog(record: str) -> dict:
    import re
    m = re.match(r"<(\d+)>1 (\S+) (\S+) (\S+) (\S+) (\S+) (-|(?:\[.*?(?<!\\)\])+) ?(.*)", record, re.S)
    pri = int(m.group(1))
    sd = {}
    if m.group(7) != "-":
        for block in re.findall(r"\[(.*?)(?<!\\)\]", m.group(7)):
            sid, _, rest = block.partition(" ")
            sd[sid] = {k: v.replace('\\"', '"').replace("\\]", "]").replace("\\\\", "\\") for k, v in re.findall(r'(\S+?)="((?:[^"\\]|\\.)*)"', rest)}
    inv = lambda d, v: next(k for k, x in d.items() if x == v)
    return {"facility": inv(FACILITY, pri // 8), "severity": inv(SEVERITY, pri % 8), "timestamp": m.group(2), "hostname": m.group(3), "app": m.group(4), "procid": m.group(5), "msgid": m.group(6), "structured": sd, "message": m.group(8)}


class SyslogSender:
    """Sends records as UDP datagrams (one record per datagram) and drops those below ``min_severity``."""

    def __init__(self, address=("127.0.0.1", 514), min_severity: str = "debug", **defaults): self.addr, self.min, self.defaults, self.sock, self.sent = address, SEVERITY[min_severity], defaults, socket.socket(socket.AF_INET, socket.SOCK_DGRAM), 0
    def send(self, message: str, severity: str = "info", **kw) -> bool:
        if SEVERITY[severity] > self.min:
            return False
        self.sock.sendto(format_syslog(message, severity, **{**self.defaults, **kw}).encode(), self.addr); self.sent += 1
        return True
    def close(self): self.sock.close()


# ================================================================================================ audit storage
class AuditStorage:
    """Append-only audit events in segment files of at most ``segment_bytes``; every record carries the hash of the one
    before it (across segments), an index by actor and action speeds up queries, old segments are removed by retention,
    and ``verify`` replays the chain."""

    def __init__(self, root, segment_bytes: int = 1 << 20, clock=time.time):
        self.root, self.segment_bytes, self.clock = Path(root), segment_bytes, clock
        self.root.mkdir(parents=True, exist_ok=True)
        self.index: dict[tuple[str, str], list[tuple[int, int]]] = {}
        self._seg, self._last_hash, self._count = 0, "0" * 64, 0
        for seg in self._segments():
            for line_no, rec in enumerate(self._read(seg)):
                self._note(rec, seg, line_no); self._last_hash = rec["hash"]; self._count += 1
            self._seg = seg
        self.anchor = self._first_prev()

    def _segments(self): return sorted(int(p.stem.split("-")[1]) for p in self.root.glob("segment-*.jsonl"))
    def _file(self, seg): return self.root / f"segment-{seg:06d}.jsonl"
    def _read(self, seg): return [json.loads(l) for l in self._file(seg).read_text().splitlines() if l]
    def _note(self, rec, seg, line):
        for key in (("actor", rec["actor"]), ("action", rec["action"])):
            self.index.setdefault(key, []).append((seg, line))
    def _first_prev(self):
        segs = self._segments()
        return self._read(segs[0])[0]["prev"] if segs and self._read(segs[0]) else "0" * 64

    def append(self, actor: str, action: str, resource: str, outcome: str = "success", **details) -> dict:
        rec = {"seq": self._count, "time": self.clock(), "actor": actor, "action": action, "resource": resource, "outcome": outcome, "details": details, "prev": self._last_hash}
        rec["hash"] = hashlib.sha256(json.dumps(rec, sort_keys=True).encode()).hexdigest()
        f = self._file(self._seg)
        if f.exists() and f.stat().st_size >= self.segment_bytes:
            self._seg += 1; f = self._file(self._seg)
        line = len(f.read_text().splitlines()) if f.exists() else 0
        with f.open("a") as fh:
            fh.write(json.dumps(rec, sort_keys=True) + "\n")
        self._note(rec, self._seg, line); self._last_hash = rec["hash"]; self._count += 1
        return rec

    def query(self, actor: str | None = None, action: str | None = None, since: float | None = None, outcome: str | None = None) -> list[dict]:
        if actor is not None or action is not None:
            key = ("actor", actor) if actor is not None else ("action", action)
            cache, out = {}, []
            for seg, line in self.index.get(key, []):
                if not self._file(seg).exists():
                    continue
                rows = cache.setdefault(seg, self._read(seg))
                out.append(rows[line])
        else:
            out = [r for seg in self._segments() for r in self._read(seg)]
        return [r for r in out if (actor is None or r["actor"] == actor) and (action is None or r["action"] == action) and (since is None or r["time"] >= since) and (outcome is None or r["outcome"] == outcome)]

    def verify(self) -> dict:
        prev, n = self.anchor, 0
        for seg in self._segments():
            for i, r in enumerate(self._read(seg)):
                body = {k: v for k, v in r.items() if k != "hash"}
                if r["prev"] != prev or hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest() != r["hash"]:
                    return {"valid": False, "segment": seg, "line": i, "records_checked": n}
                prev, n = r["hash"], n + 1
        return {"valid": True, "records_checked": n}

    def apply_retention(self, max_age: float) -> int:
        """Removes whole segments whose newest record is older than ``max_age``; the chain is re-anchored at the first record
        that remains."""
        removed, now = 0, self.clock()
        for seg in self._segments()[:-1]:
            rows = self._read(seg)
            if rows and now - rows[-1]["time"] > max_age:
                self._file(seg).unlink(); removed += 1
            else:
                break
        self.index = {k: [(s, l) for s, l in v if self._file(s).exists()] for k, v in self.index.items()}
        self.anchor = self._first_prev()
        return removed

    def export(self, path, fmt: str = "jsonl") -> int:
        rows = [r for seg in self._segments() for r in self._read(seg)]
        if fmt == "csv":
            import csv
            with open(path, "w", newline="") as f:
                w = csv.writer(f); w.writerow(["seq", "time", "actor", "action", "resource", "outcome"])
                w.writerows([r["seq"], r["time"], r["actor"], r["action"], r["resource"], r["outcome"]] for r in rows)
        else:
            Path(path).write_text("".join(json.dumps(r) + "\n" for r in rows))
        return len(rows)
