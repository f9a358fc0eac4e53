"""Parameter server (``crates/torsh-distributed/src/parameter_server.rs:22-628``): versioned parameters, gradient
push with an optimizer step on the server (SGD with momentum), pull by clients that tells whether the local copy is
stale.  In-process it is a thread-safe object; across processes it is served through :mod:`torsh_b200.parallel.rpc`."""
from __future__ import annotations

import threading
from dataclasses import dataclass

import torch


@dataclass
class ParameterServerConfig:
    learning_rate: float = 0.01
    momentum: float = 0.0
    weight_decay: float = 0.0
    max_staleness: int | None = None   # reject gradients computed on a version older than this many updates
    aggregate: int = 1                 # apply the update after this many pushes (mean of the pushed gradients)


class ParameterServer:
    def __init__(self, config: ParameterServerConfig | None = None):
        self.cfg = config or ParameterServerConfig()
        self.params: dict[str, torch.Tensor] = {}
        self.versions: dict[str, int] = {}
        self._mom: dict[str, torch.Tensor] = {}
        self._pending: dict[str, list[torch.Tensor]] = {}
        self._lock = threading.Lock()
        self.stats = {"pushes": 0, "pulls": 0, "rejected": 0, "updates": 0}

    def register(self, name: str, value: torch.Tensor) -> None:
        with self._lock:
            self.params[name] = value.detach().clone().float()
            self.versions[name] = 0

    def pull(self, name: str, have_version: int = -1):
        """Returns ``(version, tensor or None)``; ``None`` when the caller's copy is current."""
        with self._lock:
            self.stats["pulls"] += 1
            v = self.versions[name]
            return v, (None if have_version == v else self.params[name].clone())

    def push(self, name: str, grad: torch.Tensor, version: int | None = None) -> int:
        with self._lock:
            self.stats["pushes"] += 1
            cur = self.versions[name]
            if self.cfg.max_staleness is not None and version is not None and cur - version > self.cfg.max_staleness:
                self.stats["rejected"] += 1
                return cur
            pend = self._pending.setdefault(name, [])
            pend.append(grad.detach().float())
            if len(pend) < self.cfg.aggregate:
                return cur
            g = torch.stack(pend).mean(0)
            pend.clear()
            p = self.params[name]
            if self.cfg.weight_decay:
                g = g + self.cfg.weight_decay * p
            if self.cfg.momentum:
                m = self._mom.setdefault(name, torch.zeros_like(p))
                m.mul_(self.cfg.momentum).add_(g)
                g = m
            p.add_(g, alpha=-self.cfg.learning_rate)
            self.versions[name] = cur + 1
            self.stats["updates"] += 1
            return cur + 1

    def names(self) -> list[str]:
        return sorted(self.params)

    def serve(self, prefix: str = "ps") -> None:
        """Expose ``register / pull / push / names`` through the RPC layer (call after ``rpc.init_rpc``)."""
        from . import rpc
        rpc.register_function(f"{prefix}.register", lambda n, v: self.register(n, v))
        rpc.register_function(f"{prefix}.pull", lambda n, have=-1: list(self.pull(n, have)))
        rpc.register_function(f"{prefix}.push", lambda n, g, ver=None: self.push(n, g, ver))
        rpc.register_function(f"{prefix}.names", self.names)


class ParameterServerClient:
    """Keeps local copies; ``sync`` pulls what changed, ``push_gradients`` sends ``p.grad`` of a module."""

    def __init__(self, server: ParameterServer | str, prefix: str = "ps"):
        self.server, self.prefix = server, prefix
        self.local: dict[str, torch.Tensor] = {}
        self.versions: dict[str, int] = {}

    def _do(self, op: str, *args):
        if isinstance(self.server, ParameterServer):
            return getattr(self.server, op)(*args)
        from . import rpc
        return rpc.rpc_sync(self.server, f"{self.prefix}.{op}", args)

    def register_module(self, module: torch.nn.Module) -> None:
        for n, p in module.named_parameters():
            self._do("register", n, p.detach().cpu())

    def sync(self, module: torch.nn.Module) -> int:
        changed = 0
        for n, p in module.named_parameters():
            ver, val = self._do("pull", n, self.versions.get(n, -1))
            if val is not None:
                with torch.no_grad():
                    p.copy_(val.to(p.dtype).to(p.device))
                changed += 1
            self.versions[n] = ver
        return changed

    def push_gradients(self, module: torch.nn.Module) -> None:
        for n, p in module.named_parameters():
            if p.grad is not None:
                self._do("push", n, p.grad.detach().cpu(), self.versions.get(n))
