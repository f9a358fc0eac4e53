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


def ring_all_reduce(t: torch.Tensor, op: ReduceOp = ReduceOp.SUM, group=None) -> torch.Tensor:
    """Bandwidth-optimal ring (``collectives.rs``: ``ring_all_reduce``): a reduce-scatter followed by an all-gather.
    On one NVSwitch box NCCL / the fused kernels pick the algorithm; the explicit form exists for API parity."""
    g = _g(group)
    w = dist.get_world_size(g)
    if w == 1:
        return t
    flat = t.reshape(-1)
    pad = (-flat.numel()) % w
    buf = torch.cat([flat, flat.new_zeros(pad)]) if pad else flat.clone()
    shard = reduce_scatter(buf, op, g)
    out = all_gather_into_tensor(shard, g)
    flat.copy_(out[:flat.numel()])
    return t


def hierarchical_all_reduce(t: torch.Tensor, ranks_per_node: int, op: ReduceOp = ReduceOp.SUM, group=None,
                            _groups: dict | None = None) -> torch.Tensor:
    """Two-level all-reduce (``collectives.rs``: ``hierarchical_all_reduce(ranks_per_node)``): reduce inside each node,
    all-reduce among the node leaders, broadcast inside each node. ``GroupManager.create_standard_groups`` builds the
    sub-groups once; they are cached per (group, ranks_per_node)."""
    g = _g(group)
    w, r = dist.get_world_size(g), dist.get_rank(g)
    if ranks_per_node <= 1 or ranks_per_node >= w or w % ranks_per_node:
        return all_reduce(t, op, g)
    gm = GroupManager.for_group(g)
    std = gm.create_standard_groups(ranks_per_node)
    local, leaders = std["local"], std["leaders"]
    leader_rank = (r // ranks_per_node) * ranks_per_node
    mean = op is ReduceOp.MEAN
    top = ReduceOp.SUM if mean else op
    dist.reduce(t, dst=dist.get_global_rank(g, leader_rank), op=top.to_torch(), group=local)
    if r == leader_rank:
        dist.all_reduce(t, op=top.to_torch(), group=leaders)
    dist.broadcast(t, src=dist.get_global_rank(g, leader_rank), group=local)
    if mean:
        t.div_(w)
    return t


def tree_broadcast(t: torch.Tensor, src: int = 0, group=None) -> torch.Tensor:
    """Binomial-tree broadcast with point-to-point messages (``collectives.rs``: ``tree_broadcast``): log2(world)
    rounds; in round k the ranks that already hold the data send to the rank ``2^k`` places further (relative to
    ``src``)."""
    g = _g(group)
    w, r = dist.get_world_size(g), dist.get_rank(g)
    rel = (r - src) % w
    k = 1
    while k < w:
        if rel < k and rel + k < w:
            dist.send(t, dist.get_global_rank(g, (rel + k + src) % w), group=g)
        elif k <= rel < 2 * k:
            dist.recv(t, dist.get_global_rank(g, (rel - k + src) % w), group=g)
        k *= 2
    return t


def pipelined_all_reduce(t: torch.Tensor, chunk_bytes: int = 4 << 20, op: ReduceOp = ReduceOp.SUM, group=None) -> torch.Tensor:
    """All-reduce in chunks issued asynchronously, so chunk i+1 is on the wire while chunk i completes
    (``collectives.rs``: ``pipelined_all_reduce``)."""
    g = _g(group)
    flat = t.reshape(-1)
    per = max(1, chunk_bytes // t.element_size())
    works = [dist.all_reduce(flat[i:i + per], op=op.to_torch(), group=g, async_op=True) for i in range(0, flat.numel(), per)]
    for wk in works:
        wk.wait()
    if op is ReduceOp.MEAN:
        flat.div_(dist.get_world_size(g))
    return t


def double_buffered_all_reduce(tensors: list[torch.Tensor], op: ReduceOp = ReduceOp.SUM, group=None) -> list[torch.Tensor]:
    """Two staging buffers alternate: while buffer A is being reduced, the next tensor is packed into buffer B and the
    previous result is unpacked (``collectives.rs``: ``double_buffered_all_reduce``)."""
    g = _g(group)
    if not tensors:
        return tensors
    cap = max(x.numel() for x in tensors)
    bufs = [tensors[0].new_empty(cap) for _ in range(2)]
    pending = None                       # (work, buffer index, tensor)
    for i, x in enumerate(tensors):
        b = bufs[i % 2][:x.numel()]
        b.copy_(x.reshape(-1))
        wk = dist.all_reduce(b, op=op.to_torch(), group=g, async_op=True)
        if pending is not None:
            pw, pb, px = pending
            pw.wait()
            px.copy_(pb.view_as(px))
        pending = (wk, b, x)
    pw, pb, px = pending
    pw.wait()
    px.copy_(pb.view_as(px))
    if op is ReduceOp.MEAN:
        for x in tensors:
            x.div_(dist.get_world_size(g))
    return tensors


class CommunicationGroup:
    """Global ↔ local rank maps of one sub-group (``collectives.rs:16-229``)."""

    def __init__(self, name: str, ranks: list[int], pg=None):
        self.name, self.ranks, self.pg = name, list(ranks), pg
        self._local = {g: i for i, g in enumerate(self.ranks)}

    def local_rank(self, global_rank: int) -> int | None:
        return self._local.get(global_rank)

    def global_rank(self, local_rank: int) -> int:
        return self.ranks[local_rank]

    def contains(self, global_rank: int) -> bool:
        return global_rank in self._local

    def size(self) -> int:
        return len(self.ranks)


class GroupManager:
    """Creates and caches sub-groups of a process group (``GroupManager::create_standard_groups``): per node a
    ``local`` group, one ``leaders`` group of the first rank of every node, and ``world``. ``dist.new_group`` is
    collective, so every rank creates every group in the same order."""

    _by_group: dict = {}

    def __init__(self, group=None):
        self.group = _g(group)
        self.groups: dict[str, CommunicationGroup] = {}
        self._std: dict[int, dict] = {}

    @classmethod
    def for_group(cls, group=None) -> "GroupManager":
        g = _g(group)
        key = id(g)
        if key not in cls._by_group:
            cls._by_group[key] = cls(g)
        return cls._by_group[key]

    def create_group(self, name: str, ranks: list[int]) -> CommunicationGroup:
        if name in self.groups:
            return self.groups[name]
        pg = dist.new_group([dist.get_global_rank(self.group, r) for r in ranks])
        cg = CommunicationGroup(name, ranks, pg)
        self.groups[name] = cg
        return cg

    def create_standard_groups(self, ranks_per_node: int) -> dict:
        if ranks_per_node in self._std:
            return self._std[ranks_per_node]
        w, r = dist.get_world_size(self.group), dist.get_rank(self.group)
        nodes = w // ranks_per_node
        local = None
        for n in range(nodes):
            cg = self.create_group(f"node{n}/{ranks_per_node}", list(range(n * ranks_per_node, (n + 1) * ranks_per_node)))
            if cg.contains(r):
                local = cg.pg
        leaders = self.create_group(f"leaders/{ranks_per_node}", [n * ranks_per_node for n in range(nodes)])
        self._std[ranks_per_node] = {"local": local, "leaders": leaders.pg, "world": self.group,
                                     "node": r // ranks_per_node, "nodes": nodes}
        return self._std[ranks_per_node]


class CollectiveBatch:
    """Queues collectives and issues them together (``crates/torsh-distributed/src/nccl_ops.rs:519-670``: ``NcclBatch``):
    point-to-point ops go out as one ``batch_isend_irecv`` (one NCCL group call), the others asynchronously; ``execute``
    waits for all of them."""

    def __init__(self, group=None):
        self.group = _g(group)
        self._p2p, self._coll = [], []

    def all_reduce(self, t, op: ReduceOp = ReduceOp.SUM):
        self._coll.append(lambda: dist.all_reduce(t, op=op.to_torch(), group=self.group, async_op=True)); return self

    def broadcast(self, t, src: int = 0):
        self._coll.append(lambda: dist.broadcast(t, src=dist.get_global_rank(self.group, src), group=self.group, async_op=True)); return self

    def all_gather(self, out: torch.Tensor, t: torch.Tensor):
        self._coll.append(lambda: dist.all_gather_into_tensor(out, t, group=self.group, async_op=True)
                          if t.is_cuda else dist.all_gather(list(out.chunk(dist.get_world_size(self.group))), t, group=self.group, async_op=True))
        return self

    def send(self, t, dst: int):
        self._p2p.append(dist.P2POp(dist.isend, t, dist.get_global_rank(self.group, dst), self.group)); return self

    def recv(self, t, src: int):
        self._p2p.append(dist.P2POp(dist.irecv, t, dist.get_global_rank(self.group, src), self.group)); return self

    def __len__(self):
        return len(self._p2p) + len(self._coll)

    def execute(self) -> int:
        works = [f() for f in self._coll]
        if self._p2p:
            works += dist.batch_isend_irecv(self._p2p)
        for wk in works:
            wk.wait()
        n = len(works)
        self._p2p, self._coll = [], []
        return n


NcclBatch = CollectiveBatch


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
