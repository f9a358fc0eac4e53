"""Debug-time checks (roles of ``crates/torsh-tensor/src/nan_inf_detection.rs``, ``crates/torsh-backend/src/
deadlock_prevention.rs:20-224``, ``crates/torsh-core/src/memory_debug.rs``): NaN / Inf scanning of tensors and of every
module output, a lock-order validator with timed acquisition, guard words around symmetric buffers, and a
deterministic-replay check that runs a step twice and compares bit patterns."""
from __future__ import annotations

import threading
import time
from contextlib import contextmanager

import torch


class NonFiniteError(RuntimeError):
    pass


def nan_inf_report(t: torch.Tensor) -> dict:
    f = t.detach().float()
    nan, inf = torch.isnan(f), torch.isinf(f)
    return {"numel": t.numel(), "nan": int(nan.sum()), "pos_inf": int((inf & (f > 0)).sum()), "neg_inf": int((inf & (f < 0)).sum()),
            "first_bad": int((nan | inf).flatten().nonzero()[0]) if (nan | inf).any() else None}


def check_finite(t: torch.Tensor, name: str = "tensor") -> torch.Tensor:
    if not torch.isfinite(t.detach().float()).all():
        raise NonFiniteError(f"{name}: {nan_inf_report(t)}")
    return t


@contextmanager
def detect_non_finite(module: torch.nn.Module):
    """Raise at the first sub-module whose output contains NaN / Inf (forward hooks; removed on exit)."""
    handles = []

    def hook(mod, _inp, out):
        for o in (out if isinstance(out, (tuple, list)) else (out,)):
            if isinstance(o, torch.Tensor) and o.is_floating_point():
                check_finite(o, f"output of {type(mod).__name__}")
    for m in module.modules():
        handles.append(m.register_forward_hook(hook))
    try:
        yield
    finally:
        for h in handles:
            h.remove()


class LockOrderError(RuntimeError):
    pass


class LockOrderValidator:
    """Locks get a rank on creation; a thread may only acquire locks in increasing rank (so no cycle can form)."""

    def __init__(self):
        self._held = threading.local()

    def lock(self, rank: int, name: str = "") -> "SafeLock":
        return SafeLock(self, rank, name or f"lock{rank}")

    def _stack(self) -> list:
        if not hasattr(self._held, "s"):
            self._held.s = []
        return self._held.s


class SafeLock:
    def __init__(self, validator: LockOrderValidator, rank: int, name: str):
        self.v, self.rank, self.name, self._l = validator, rank, name, threading.Lock()

    def acquire(self, timeout: float = 10.0) -> None:
        st = self.v._stack()
        if st and st[-1].rank >= self.rank:
            raise LockOrderError(f"acquiring {self.name} (rank {self.rank}) while holding {st[-1].name} (rank {st[-1].rank})")
        if not self._l.acquire(timeout=timeout):
            raise TimeoutError(f"{self.name}: not acquired within {timeout} s (possible deadlock)")
        st.append(self)

    def release(self) -> None:
        st = self.v._stack()
        if self in st:
            st.remove(self)
        self._l.release()

    def __enter__(self):
        self.acquire(); return self

    def __exit__(self, *a):
        self.release()


GUARD_WORD = 0x5A


def add_guards(buffer: torch.Tensor, guard_elems: int = 64):
    """Returns ``(payload_view, check)`` for a flat buffer whose first and last ``guard_elems`` elements become guard
    zones filled with a byte pattern; ``check()`` raises if a kernel wrote outside the payload."""
    raw = buffer.view(torch.uint8)
    gb = guard_elems * buffer.element_size()
    raw[:gb].fill_(GUARD_WORD); raw[-gb:].fill_(GUARD_WORD)
    payload = buffer[guard_elems: buffer.numel() - guard_elems]

    def check():
        if not (bool((raw[:gb] == GUARD_WORD).all()) and bool((raw[-gb:] == GUARD_WORD).all())):
            raise RuntimeError("guard zone of a buffer was overwritten")
    return payload, check


def deterministic_replay(step_fn, state_fn, restore_fn) -> bool:
    """Run ``step_fn`` twice from the same state and compare the resulting states bit for bit.
    ``state_fn() -> list[Tensor]`` snapshots, ``restore_fn(snapshot)`` restores."""
    snap = [t.detach().clone() for t in state_fn()]
    step_fn()
    a = [t.detach().clone() for t in state_fn()]
    restore_fn(snap)
    step_fn()
    b = state_fn()
    return all(torch.equal(x.view(torch.uint8) if x.is_floating_point() else x, y.view(torch.uint8) if y.is_floating_point() else y)
               for x, y in zip(a, b))


class Stopwatch:
    def __enter__(self):
        self.t0 = time.perf_counter(); return self

    def __exit__(self, *a):
        self.ms = (time.perf_counter() - self.t0) * 1e3
