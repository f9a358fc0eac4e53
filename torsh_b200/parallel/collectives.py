"""Collectives: hand-written NVSwitch kernels on symmetric buffers, NCCL / gloo for everything else.

API names follow ``crates/torsh-distributed/src/collectives.rs:232-1374`` (``all_reduce``, ``all_gather``,
``broadcast``, ``reduce``, ``scatter``, ``barrier``, ``send``/``recv``, ``reduce_scatter``, ``all_to_all``,
``bucket_all_reduce`` ...), where every one of them is a no-op or a local clone. Here the generic
functions move data through ``torch.distributed`` (NCCL on GPUs, gloo on CPU) and
:class:`FusedCollectives` runs the kernels of ``csrc/kernels/collectives_sm100.cu`` on a
:class:`~torsh_b200.parallel.symm.SymmetricBuffer`.
"""
from __future__ import annotations

import ctypes
from enum import Enum

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops._dispatch import call
from .symm import CommContext, SymmetricBuffer


class ReduceOp(Enum):
    """``crates/torsh-distributed/src/backend.rs:15-71``."""
    SUM = "sum"; PRODUCT = "product"; MIN = "min"; MAX = "max"; BAND = "band"; BOR = "bor"; BXOR = "bxor"; MEAN = "mean"

    def to_torch(self):
        return {ReduceOp.SUM: dist.ReduceOp.SUM, ReduceOp.PRODUCT: dist.ReduceOp.PRODUCT, ReduceOp.MIN: dist.ReduceOp.MIN,
                ReduceOp.MAX: dist.ReduceOp.MAX, ReduceOp.BAND: dist.ReduceOp.BAND, ReduceOp.BOR: dist.ReduceOp.BOR,
                ReduceOp.BXOR: dist.ReduceOp.BXOR, ReduceOp.MEAN: dist.ReduceOp.SUM}[self]


def _g(group):
    return group if group is not None else dist.group.WORLD


def all_reduce(t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, group=None) -> torch.Tensor:
    dist.all_reduce(t, op.to_torch(), group=_g(group))
    if op is ReduceOp.MEAN:
        t.div_(dist.get_world_size(_g(group)))
    return t


def all_gather(t: torch.Tensor, group=None) -> list[torch.Tensor]:
    out = [torch.empty_like(t) for _ in range(dist.get_world_size(_g(group)))]
    dist.all_gather(out, t.contiguous(), group=_g(group))
    return out


def all_gather_into_tensor(t: torch.Tensor, group=None) -> torch.Tensor:
    w = dist.get_world_size(_g(group))
    out = torch.empty((w * t.shape[0], *t.shape[1:]), dtype=t.dtype, device=t.device)
    if t.is_cuda:
        dist.all_gather_into_tensor(out, t.contiguous(), group=_g(group))
    else:
        out.copy_(torch.cat(all_gather(t, group), 0))
    return out


def all_gather_varsize(t: torch.Tensor, group=None) -> list[torch.Tensor]:
    """Chunks may differ in length along dim 0."""
    g = _g(group)
    sizes = all_gather(torch.tensor([t.shape[0]], device=t.device), g)
    mx = int(max(s.item() for s in sizes))
    pad = torch.zeros((mx, *t.shape[1:]), dtype=t.dtype, device=t.device)
    pad[: t.shape[0]] = t
    return [p[: int(s.item())] for p, s in zip(all_gather(pad, g), sizes)]


def broadcast(t: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
    dist.broadcast(t, src, group=_g(group))
    return t


def reduce(t: torch.Tensor, dst: int = 0, op: ReduceOp = ReduceOp.SUM, group=None) -> torch.Tensor:
    dist.reduce(t, dst, op.to_torch(), group=_g(group))
    if op is ReduceOp.MEAN and dist.get_rank(_g(group)) == dst:
        t.div_(dist.get_world_size(_g(group)))
    return t


def scatter(out: torch.Tensor, chunks: list[torch.Tensor] | None, src: int = 0, group=None) -> torch.Tensor:
    dist.scatter(out, chunks if dist.get_rank(_g(group)) == src else None, src, group=_g(group))
    return out


def gather(t: torch.Tensor, dst: int = 0, group=None):
    g = _g(group)
    out = [torch.empty_like(t) for _ in range(dist.get_world_size(g))] if dist.get_rank(g) == dst else None
    dist.gather(t, out, dst, group=g)
    return out


def reduce_scatter(t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, group=None) -> torch.Tensor:
    """``t``: ``[world * n, ...]`` → this rank's reduced ``[n, ...]``."""
    g = _g(group)
    w = dist.get_world_size(g)
    out = torch.empty((t.shape[0] // w, *t.shape[1:]), dtype=t.dtype, device=t.device)
    if t.is_cuda:
        dist.reduce_scatter_tensor(out, t.contiguous(), op.to_torch(), group=g)
    else:
        full = t.clone()
        dist.all_reduce(full, op.to_torch(), group=g)
        r = dist.get_rank(g)
        out.copy_(full[r * out.shape[0]:(r + 1) * out.shape[0]])
    if op is ReduceOp.MEAN:
        out.div_(w)
    return out


def all_to_all(chunks: list[torch.Tensor], group=None) -> list[torch.Tensor]:
    g = _g(group)
    out = [torch.empty_like(c) for c in chunks]
    if chunks[0].is_cuda:
        dist.all_to_all(out, [c.contiguous() for c in chunks], group=g)
    else:  # gloo has no all_to_all: one scatter per source rank
        for src in range(dist.get_world_size(g)):
            dist.scatter(out[src], [c.contiguous() for c in chunks] if dist.get_rank(g) == src else None, src, group=g)
    return out


def barrier(group=None):
    dist.barrier(_g(group))


def send(t, dst, tag: int = 0, group=None): dist.send(t, dst, group=_g(group), tag=tag)
def recv(t, src, tag: int = 0, group=None): dist.recv(t, src, group=_g(group), tag=tag)
def isend(t, dst, tag: int = 0, group=None): return dist.isend(t, dst, group=_g(group), tag=tag)
def irecv(t, src, tag: int = 0, group=None): return dist.irecv(t, src, group=_g(group), tag=tag)


def bucket_all_reduce(tensors: list[torch.Tensor], max_bucket_mb: float = 25.0, op: ReduceOp = ReduceOp.SUM, group=None):
    """Greedy grouping up to ``max_bucket_mb`` then one all-reduce per flat bucket
    (grouping arithmetic of ``collectives.rs:1047-1073``)."""
    cap = int(max_bucket_mb * 1024 * 1024)
    bucket, size = [], 0

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        flat = torch.cat([t.reshape(-1) for t in bucket])
        all_reduce(flat, op, group)
        off = 0
        for t in bucket:
            t.copy_(flat[off:off + t.numel()].view_as(t))
            off += t.numel()
        bucket, size = [], 0

    for t in tensors:
        nb = t.numel() * t.element_size()
        if bucket and (size + nb > cap or t.dtype != bucket[0].dtype):
            flush()
        bucket.append(t)
        size += nb
    flush()
    return tensors


def fused_all_reduce(tensors: list[torch.Tensor], threshold_bytes: int = 1 << 20, op: ReduceOp = ReduceOp.SUM, group=None):
    """Tensors smaller than ``threshold_bytes`` travel together in one flat message (``collectives.rs:1121-1141``)."""
    small = [t for t in tensors if t.numel() * t.element_size() < threshold_bytes]
    for t in tensors:
        if t.numel() * t.element_size() >= threshold_bytes:
            all_reduce(t, op, group)
    if small:
        bucket_all_reduce(small, 1e9, op, group)
    return tensors


def ring_all_reduce_host(buffers: list[torch.Tensor]) -> None:
    """Reference algorithm of the host-staged ring (``crates/torsh-backend/src/cuda/multi_gpu.rs:130-217``):
    2(N-1) steps over N equal chunks (remainder spread over the first chunks). In-place sum over a list
    of same-shape host tensors; kept as the CPU oracle for the device kernels."""
    n = len(buffers)
    if n <= 1:
        return
    flat = [b.reshape(-1) for b in buffers]
    ln = flat[0].numel()
    base, rem = divmod(ln, n)
    bounds, s = [], 0
    for i in range(n):
        e = s + base + (1 if i < rem else 0)
        bounds.append((s, e))
        s = e
    for step in range(n - 1):  # reduce-scatter
        sends = [(r, (r - step) % n) for r in range(n)]
        vals = [flat[r][bounds[c][0]:bounds[c][1]].clone() for r, c in sends]
        for (r, c), v in zip(sends, vals):
            flat[(r + 1) % n][bounds[c][0]:bounds[c][1]] += v
    for step in range(n - 1):  # all-gather
        sends = [(r, (r + 1 - step) % n) for r in range(n)]
        vals = [flat[r][bounds[c][0]:bounds[c][1]].clone() for r, c in sends]
        for (r, c), v in zip(sends, vals):
            flat[(r + 1) % n][bounds[c][0]:bounds[c][1]] = v


# ------------------------------------------------------------------------------------ fused kernels
P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float


class FusedCollectives:
    """In-kernel collectives on a :class:`SymmetricBuffer` (P2P loads/stores or NVLS multimem)."""

    def __init__(self, group=None, nblocks: int | None = None, use_nvls: bool | None = None):
        self.ctx = CommContext(group)
        self.rank, self.world, self.nblocks = self.ctx.rank, self.ctx.world, nblocks
        self.use_nvls = use_nvls

    def _blocks(self, nbytes: int) -> int:
        """CTAs for a message: one per 64 KB, at least 8, at most two per SM (enough loads in flight to fill NVLink)."""
        if self.nblocks is not None:
            return self.nblocks
        return max(8, min(296, nbytes // 65536))

    def _nvls(self, buf: SymmetricBuffer) -> bool:
        """In-switch reduction / multicast by default only beyond two ranks: with two, a multicast store also returns
        the sender's own copy and a multimem load also fetches the local half through the switch, so plain peer
        loads / stores move half the bytes over each link."""
        if self.use_nvls is None:
            return buf.has_multicast and self.world > 2
        return self.use_nvls and buf.has_multicast

    def all_reduce_(self, buf: SymmetricBuffer, numel: int | None = None, offset: int = 0, scale: float = 1.0,
                    mode: str | None = None):
        """In-place sum over ranks (× ``scale``) of ``buf.tensor[offset:offset+numel]``.
        ``mode``: ``one_shot`` | ``two_shot`` (NVLS when available, else peer memory); default by size."""
        t = buf.tensor
        n = t.numel() - offset if numel is None else numel
        nbytes = n * t.element_size()
        if mode is None:
            mode = "one_shot" if nbytes <= 256 * 1024 else "two_shot"
        m = 0 if mode == "one_shot" else (1 if self._nvls(buf) else 2)
        st = nv.status_word(t.device)
        call("tb_allreduce", [P, P, P, I, I, P, L, L, I, F, I, I, P, P], buf.ptr_array, self.ctx.flags.ptr_array,
             buf.mc(m == 1), self.rank, self.world, self.ctx.epoch.data_ptr(), offset * t.element_size(), n,
             0 if t.dtype == torch.bfloat16 else 1, float(scale), m, self._blocks(nbytes), st.data_ptr(), nv.stream_ptr())
        return t

    def all_gather_(self, buf: SymmetricBuffer, chunk_numel: int, offset: int = 0):
        """Chunk ``rank`` of ``buf`` (``world`` chunks of ``chunk_numel``) is pushed to every rank."""
        t = buf.tensor
        nvls = self._nvls(buf)
        st = nv.status_word(t.device)
        call("tb_allgather", [P, P, P, I, I, P, L, L, I, I, I, P, P], buf.ptr_array, self.ctx.flags.ptr_array,
             buf.mc(nvls), self.rank, self.world, self.ctx.epoch.data_ptr(), offset * t.element_size(), chunk_numel,
             t.element_size(), int(nvls), self._blocks(chunk_numel * t.element_size()), st.data_ptr(), nv.stream_ptr())
        return t

    def reduce_scatter(self, buf: SymmetricBuffer, chunk_numel: int, out: torch.Tensor | None = None, offset: int = 0,
                       scale: float = 1.0) -> torch.Tensor:
        """``out = scale · Σ_ranks buf[rank·chunk : (rank+1)·chunk]`` (local result)."""
        t = buf.tensor
        if out is None:
            out = torch.empty(chunk_numel, dtype=t.dtype, device=t.device)
        nvls = self._nvls(buf)
        st = nv.status_word(t.device)
        call("tb_reducescatter", [P, P, P, I, I, P, L, L, I, F, I, P, I, P, P], buf.ptr_array,
             self.ctx.flags.ptr_array, buf.mc(nvls), self.rank, self.world, self.ctx.epoch.data_ptr(),
             offset * t.element_size(), chunk_numel, 0 if t.dtype == torch.bfloat16 else 1, float(scale), int(nvls),
             out.data_ptr(), self._blocks(chunk_numel * t.element_size()), st.data_ptr(), nv.stream_ptr())
        return out
