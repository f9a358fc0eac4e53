"""Dependency resolution for packages: semantic versions, requirement specifiers (``^1.2``, ``~1.2.3``, ``>=1,<2``, ``*``,
exact), an index of available releases with their own dependencies, and a backtracking resolver that returns one version
per package (highest first) or explains the conflict; plus manifest migration between format versions and a lock file.
Reference: crates/torsh-package/src/ (dependency solver, manifest versions, lock files).
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from functools import total_ordering


@total_ordering
@dataclass(frozen=True)
class Version:
    major: int
    minor: int = 0
    patch: int = 0
    pre: tuple = ()

    @staticmethod
    def parse(s: str) -> "Version":
        m = re.fullmatch(r"v?(\d+)(?:\.(\d+))?(?:\.(\d+))?(?:-([0-9A-Za-z.\-]+))?(?:\+.*)?", s.strip())
        if not m:
            raise ValueError(f"not a semantic version: {s!r}")
        pre = tuple(int(p) if p.isdigit() else p for p in m.group(4).split(".")) if m.group(4) else ()
        return Version(int(m.group(1)), int(m.group(2) or 0), int(m.group(3) or 0), pre)

    def _key(self):
        # a pre-release sorts before its release; numeric identifiers before alphanumeric ones
        pre = tuple((0, p) if isinstance(p, int) else (1, p) for p in self.pre)
        return (self.major, self.minor, self.patch, 0 if self.pre else 1, pre)

    def __lt__(self, o): return self._key() < o._key()
    def __str__(self): return f"{self.major}.{self.minor}.{self.patch}" + ("-" + ".".join(map(str, self.pre)) if self.pre else "")


class Requirement:
    """Comma-separated comparators, all of which must hold."""

    def __init__(self, spec: str = "*"):
        self.spec = spec.strip() or "*"
        self.clauses = []
        for part in self.spec.split(","):
            part = part.strip()
            if part in ("*", ""):
                continue
            m = re.fullmatch(r"(\^|~|>=|<=|>|<|==|=)?\s*(.+)", part)
            op, ver = m.group(1) or "^", m.group(2)                      # a bare version means caret, as in Cargo
            v = Version.parse(ver)
            given = len(ver.lstrip("v").split("-")[0].split("."))
            if op == "^":
                if v.major > 0 or given == 1:
                    hi = Version(v.major + 1)
                elif v.minor > 0 or given == 2:
                    hi = Version(0, v.minor + 1)
                else:
                    hi = Version(0, 0, v.patch + 1)
                self.clauses += [(">=", v), ("<", hi)]
            elif op == "~":
                hi = Version(v.major + 1) if given == 1 else Version(v.major, v.minor + 1)
                self.clauses += [(">=", v), ("<", hi)]
            else:
                self.clauses.append(("==" if op == "=" else op, v))

    def matches(self, v: Version) -> bool:
        if v.pre and not any(c.pre and (c.major, c.minor, c.patch) == (v.major, v.minor, v.patch) for _, c in self.clauses):
            return False                                                  # pre-releases only on explicit request
        ops = {">=": v.__ge__, "<=": v.__le__, ">": v.__gt__, "<": v.__lt__, "==": v.__eq__}
        return all(ops[op](c) for op, c in self.clauses)

    def __repr__(self): return f"Requirement({self.spec!r})"


class ResolutionError(Exception):
    pass


class PackageIndex:
    """name -> {version string: {dependency name: requirement spec}}."""

    def __init__(self, releases: dict | None = None):
        self.releases: dict[str, dict[Version, dict]] = {}
        for name, vers in (releases or {}).items():
            for v, deps in vers.items():
                self.add(name, v, deps)

    def add(self, name: str, version: str, dependencies: dict | None = None):
        self.releases.setdefault(name, {})[Version.parse(version)] = dict(dependencies or {})

    def candidates(self, name: str, req: Requirement) -> list[Version]:
        return sorted((v for v in self.releases.get(name, {}) if req.matches(v)), reverse=True)


def resolve(index: PackageIndex, root_requirements: dict) -> dict:
    """One version per package satisfying every requirement reachable from ``root_requirements`` (highest versions
    preferred, chronological backtracking). Raises :class:`ResolutionError` naming the requirement that cannot be met."""
    last_conflict = [None]

    def solve(pending: list, chosen: dict, reqs: dict):
        if not pending:
            return chosen
        (name, spec, origin), rest = pending[0], pending[1:]
        req = Requirement(spec)
        all_reqs = reqs.get(name, []) + [(req, origin)]
        if name in chosen:
            if req.matches(chosen[name]):
                return solve(rest, chosen, {**reqs, name: all_reqs})
            last_conflict[0] = f"{name} {chosen[name]} (needed by {', '.join(o for _, o in reqs[name])}) does not satisfy {spec!r} needed by {origin}"
            return None
        if name not in index.releases:
            last_conflict[0] = f"unknown package {name!r} needed by {origin}"
            return None
        cands = [v for v in index.candidates(name, req) if all(r.matches(v) for r, _ in all_reqs)]
        if not cands:
            last_conflict[0] = f"no release of {name} satisfies {spec!r} needed by {origin} (available: {', '.join(map(str, sorted(index.releases[name])))})"
        for v in cands:
            deps = [(d, s, f"{name} {v}") for d, s in index.releases[name][v].items()]
            out = solve(deps + rest, {**chosen, name: v}, {**reqs, name: all_reqs})
            if out is not None:
                return out
        return None

    out = solve([(n, s, "the root manifest") for n, s in root_requirements.items()], {}, {})
    if out is None:
        raise ResolutionError(last_conflict[0] or "no solution")
    return {n: str(v) for n, v in sorted(out.items())}


def write_lock(resolution: dict, index: PackageIndex) -> str:
    """Lock file: the chosen versions with the dependencies each was resolved against."""
    return json.dumps({"lock_version": 1, "packages": [
        {"name": n, "version": v, "dependencies": index.releases[n][Version.parse(v)]} for n, v in sorted(resolution.items())]}, indent=2)


def check_lock(lock_text: str, index: PackageIndex, root_requirements: dict) -> list[str]:
    """Problems that make a lock file stale: a locked version missing from the index or violating a requirement."""
    lock = json.loads(lock_text)
    locked = {p["name"]: Version.parse(p["version"]) for p in lock["packages"]}
    problems = []
    for n, s in root_requirements.items():
        if n not in locked:
            problems.append(f"{n} is required but not locked")
        elif not Requirement(s).matches(locked[n]):
            problems.append(f"{n} {locked[n]} violates the root requirement {s!r}")
    for p in lock["packages"]:
        v = Version.parse(p["version"])
        if v not in index.releases.get(p["name"], {}):
            problems.append(f"{p['name']} {v} is no longer in the index")
        for d, s in p["dependencies"].items():
            if d in locked and not Requirement(s).matches(locked[d]):
                problems.append(f"{p['name']} {v} needs {d} {s!r} but {locked[d]} is locked")
    return problems


MANIFEST_FORMAT = 2


def migrate_manifest(manifest: dict) -> dict:
    """Brings a package manifest to the current format: format 1 had ``dependencies`` as a list of ``"name==version"``
    strings or a name -> exact version map and no ``requires_torsh`` / ``files`` digest algorithm fields."""
    m = dict(manifest)
    fmt = int(m.get("format", 1))
    if fmt > MANIFEST_FORMAT:
        raise ValueError(f"manifest format {fmt} is newer than this library understands ({MANIFEST_FORMAT})")
    if fmt < 2:
        deps = m.get("dependencies") or {}
        if isinstance(deps, list):
            deps = dict(re.split(r"\s*==\s*", d, maxsplit=1) if "==" in d else (d, "*") for d in deps)
        m["dependencies"] = {n: (f"=={v}" if re.fullmatch(r"v?\d+(\.\d+){0,2}", str(v)) else str(v)) for n, v in deps.items()}
        m.setdefault("requires_torsh", "*")
        m.setdefault("digest", "sha256")
        m["format"] = 2
    Version.parse(m.get("version", "0.1.0"))
    return m
