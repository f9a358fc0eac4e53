"""Sparse tensors (``crates/torsh-sparse``): COO / CSR / CSC / BSR / DIA / ELL containers with conversions, SpMV / SpMM,
a sparse linear layer and magnitude pruning into a sparse format.  Storage is plain index / value tensors on any device;
SpMM is an index-add over gathered rows (one pass over the non-zeros)."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class CooTensor:
    rows: torch.Tensor
    cols: torch.Tensor
    values: torch.Tensor
    shape: tuple[int, int]

    @staticmethod
    def from_dense(d: torch.Tensor, threshold: float = 0.0) -> "CooTensor":
        r, c = (d.abs() > threshold).nonzero(as_tuple=True)
        return CooTensor(r, c, d[r, c], tuple(d.shape))

    @property
    def nnz(self): return self.values.numel()
    @property
    def sparsity(self): return 1.0 - self.nnz / (self.shape[0] * self.shape[1])

    def to_dense(self):
        out = torch.zeros(self.shape, dtype=self.values.dtype, device=self.values.device)
        return out.index_put_((self.rows, self.cols), self.values, accumulate=True)

    def coalesce(self) -> "CooTensor":
        key = self.rows * self.shape[1] + self.cols
        uk, inv = key.unique(return_inverse=True)
        v = torch.zeros(uk.numel(), dtype=self.values.dtype, device=self.values.device).index_add_(0, inv, self.values)
        return CooTensor(uk // self.shape[1], uk % self.shape[1], v, self.shape)

    def transpose(self): return CooTensor(self.cols, self.rows, self.values, (self.shape[1], self.shape[0]))

    def matmul(self, b: torch.Tensor) -> torch.Tensor:
        vec = b.dim() == 1
        b2 = b[:, None] if vec else b
        out = torch.zeros(self.shape[0], b2.shape[1], dtype=b2.dtype, device=b2.device)
        out.index_add_(0, self.rows, self.values[:, None].to(b2.dtype) * b2[self.cols])
        return out[:, 0] if vec else out

    def to_csr(self) -> "CsrTensor":
        c = self.coalesce()
        counts = torch.bincount(c.rows, minlength=self.shape[0])
        ptr = torch.zeros(self.shape[0] + 1, dtype=torch.long, device=counts.device)
        ptr[1:] = counts.cumsum(0)
        return CsrTensor(ptr, c.cols, c.values, self.shape)

    def to_csc(self) -> "CscTensor":
        t = self.transpose().to_csr()
        return CscTensor(t.indptr, t.indices, t.values, self.shape)


@dataclass
class CsrTensor:
    indptr: torch.Tensor
    indices: torch.Tensor
    values: torch.Tensor
    shape: tuple[int, int]

    def row_ids(self): return torch.repeat_interleave(torch.arange(self.shape[0], device=self.indptr.device), self.indptr.diff())
    def to_coo(self): return CooTensor(self.row_ids(), self.indices, self.values, self.shape)
    def to_dense(self): return self.to_coo().to_dense()
    def matmul(self, b): return self.to_coo().matmul(b)
    @property
    def nnz(self): return self.values.numel()
    def to_torch(self): return torch.sparse_csr_tensor(self.indptr, self.indices, self.values, self.shape)


@dataclass
class CscTensor:
    indptr: torch.Tensor
    indices: torch.Tensor
    values: torch.Tensor
    shape: tuple[int, int]

    def to_coo(self):
        cols = torch.repeat_interleave(torch.arange(self.shape[1], device=self.indptr.device), self.indptr.diff())
        return CooTensor(self.indices, cols, self.values, self.shape)
    def to_dense(self): return self.to_coo().to_dense()
    def matmul(self, b): return self.to_coo().matmul(b)


@dataclass
class BsrTensor:
    """Block-sparse rows: ``blocks[i]`` is the dense ``bs x bs`` block at block coordinates ``(brow[i], bcol[i])``."""
    brow: torch.Tensor
    bcol: torch.Tensor
    blocks: torch.Tensor
    shape: tuple[int, int]

    @staticmethod
    def from_dense(d: torch.Tensor, bs: int) -> "BsrTensor":
        m, n = d.shape
        t = d.reshape(m // bs, bs, n // bs, bs).permute(0, 2, 1, 3)
        r, c = (t.abs().amax((2, 3)) > 0).nonzero(as_tuple=True)
        return BsrTensor(r, c, t[r, c], (m, n))

    def to_dense(self):
        bs = self.blocks.shape[-1]
        out = torch.zeros(self.shape[0] // bs, self.shape[1] // bs, bs, bs, dtype=self.blocks.dtype, device=self.blocks.device)
        out[self.brow, self.bcol] = self.blocks
        return out.permute(0, 2, 1, 3).reshape(self.shape)

    def matmul(self, b):
        bs = self.blocks.shape[-1]
        bb = b.reshape(self.shape[1] // bs, bs, -1)
        out = torch.zeros(self.shape[0] // bs, bs, bb.shape[-1], dtype=b.dtype, device=b.device)
        out.index_add_(0, self.brow, torch.bmm(self.blocks.to(b.dtype), bb[self.bcol]))
        return out.reshape(self.shape[0], -1)


@dataclass
class DiaTensor:
    offsets: torch.Tensor
    data: torch.Tensor  # [n_diag, n_cols], column-aligned like SciPy
    shape: tuple[int, int]

    @staticmethod
    def from_dense(d):
        m, n = d.shape
        offs = [k for k in range(-m + 1, n) if d.diagonal(k).abs().sum() > 0]
        data = torch.zeros(len(offs), n, dtype=d.dtype)
        for i, k in enumerate(offs):
            dg = d.diagonal(k)
            data[i, max(k, 0): max(k, 0) + dg.numel()] = dg
        return DiaTensor(torch.tensor(offs), data, (m, n))

    def to_dense(self):
        out = torch.zeros(self.shape, dtype=self.data.dtype)
        for i, k in enumerate(self.offsets.tolist()):
            ln = out.diagonal(k).numel()
            out.diagonal(k).copy_(self.data[i, max(k, 0): max(k, 0) + ln])
        return out


@dataclass
class EllTensor:
    cols: torch.Tensor    # [rows, width], -1 = padding
    values: torch.Tensor  # [rows, width]
    shape: tuple[int, int]

    @staticmethod
    def from_dense(d):
        nz = d != 0
        w = int(nz.sum(1).max())
        order = torch.argsort((~nz).to(torch.int8), dim=1, stable=True)[:, :w]
        vals = torch.gather(d, 1, order)
        return EllTensor(torch.where(vals != 0, order, torch.full_like(order, -1)), vals, tuple(d.shape))

    def matmul(self, b):
        vec = b.dim() == 1
        b2 = b[:, None] if vec else b
        g = b2[self.cols.clamp(min=0)] * (self.values * (self.cols >= 0))[..., None].to(b2.dtype)
        return g.sum(1)[:, 0] if vec else g.sum(1)

    def to_dense(self):
        out = torch.zeros(self.shape, dtype=self.values.dtype)
        r = torch.arange(self.shape[0])[:, None].expand_as(self.cols)
        m = self.cols >= 0
        out[r[m], self.cols[m]] = self.values[m]
        return out


class DsrTensor:
    """Dynamic sparse rows (``crates/torsh-sparse``: DSR): one ``{column: value}`` map per row, cheap to update in place
    while a pattern is being built; convert to CSR for arithmetic."""

    def __init__(self, shape: tuple[int, int], dtype=torch.float32):
        self.shape, self.dtype = tuple(shape), dtype
        self.rows: list[dict[int, float]] = [dict() for _ in range(shape[0])]

    @staticmethod
    def from_dense(d: torch.Tensor) -> "DsrTensor":
        out = DsrTensor(tuple(d.shape), d.dtype)
        for r, c in (d != 0).nonzero().tolist():
            out.rows[r][c] = float(d[r, c])
        return out

    def set(self, r: int, c: int, v: float):
        if v == 0:
            self.rows[r].pop(c, None)
        else:
            self.rows[r][c] = float(v)

    def get(self, r: int, c: int) -> float:
        return self.rows[r].get(c, 0.0)

    def nnz(self) -> int:
        return sum(len(r) for r in self.rows)

    def to_dense(self) -> torch.Tensor:
        out = torch.zeros(self.shape, dtype=self.dtype)
        for r, row in enumerate(self.rows):
            for c, v in row.items():
                out[r, c] = v
        return out

    def to_csr(self) -> "CsrTensor":
        return CooTensor.from_dense(self.to_dense()).to_csr()

    def matmul(self, b: torch.Tensor) -> torch.Tensor:
        return self.to_dense().to(b.dtype) @ b


@dataclass
class RleTensor:
    """Run-length encoding of a flattened tensor (``crates/torsh-sparse``: RLE): pairs of (value, run length); compact for
    masks and label maps with long constant runs."""
    values: torch.Tensor
    lengths: torch.Tensor
    shape: tuple

    @staticmethod
    def from_dense(d: torch.Tensor) -> "RleTensor":
        flat = d.reshape(-1)
        if flat.numel() == 0:
            return RleTensor(flat, torch.zeros(0, dtype=torch.int64), tuple(d.shape))
        change = torch.ones(flat.numel(), dtype=torch.bool)
        change[1:] = flat[1:] != flat[:-1]
        starts = change.nonzero()[:, 0]
        lengths = torch.diff(torch.cat([starts, torch.tensor([flat.numel()])]))
        return RleTensor(flat[starts], lengths, tuple(d.shape))

    def to_dense(self) -> torch.Tensor:
        return torch.repeat_interleave(self.values, self.lengths).reshape(self.shape)

    def compression_ratio(self) -> float:
        n = 1
        for s in self.shape:
            n *= s
        return n / max(self.values.numel() * 2, 1)


class CudaSparseTensor:
    """CSR matrix resident on a GPU with its products computed by this package's kernel (`tb_csr_spmm`: one warp per
    row and 128-column tile, fp32 accumulation). Values are fp32; the dense operand and the result are bf16 or fp32.
    The reference's `CudaSparseTensor` (crates/torsh-sparse/src/gpu.rs:13-250) declares the same operations over a
    cuSPARSE wrapper. On a CPU tensor the same class computes through the COO path, so code is portable."""

    def __init__(self, indptr: torch.Tensor, indices: torch.Tensor, values: torch.Tensor, shape: tuple[int, int]):
        self.indptr = indptr.to(torch.int32).contiguous()
        self.indices = indices.to(torch.int32).contiguous()
        self.values = values.float().contiguous()
        self.shape = (int(shape[0]), int(shape[1]))

    @classmethod
    def from_dense(cls, dense: torch.Tensor) -> "CudaSparseTensor":
        d = dense.detach().float()
        nz = d.nonzero()                                   # row-major order: already sorted by (row, column)
        indptr = torch.zeros(d.shape[0] + 1, dtype=torch.int64, device=d.device)
        indptr[1:] = torch.bincount(nz[:, 0], minlength=d.shape[0]).cumsum(0)
        return cls(indptr, nz[:, 1], d[nz[:, 0], nz[:, 1]], tuple(d.shape))

    @classmethod
    def from_coo(cls, coo: "CooTensor") -> "CudaSparseTensor":
        order = torch.argsort(coo.rows * coo.shape[1] + coo.cols)
        rows, cols, vals = coo.rows[order], coo.cols[order], coo.values[order]
        counts = torch.bincount(rows, minlength=coo.shape[0])
        indptr = torch.zeros(coo.shape[0] + 1, dtype=torch.int64, device=rows.device)
        indptr[1:] = counts.cumsum(0)
        return cls(indptr, cols, vals, coo.shape)

    @property
    def nnz(self) -> int:
        return self.values.numel()

    @property
    def device(self):
        return self.values.device

    def to(self, device) -> "CudaSparseTensor":
        return CudaSparseTensor(self.indptr.to(device), self.indices.to(device), self.values.to(device), self.shape)

    def to_dense(self) -> torch.Tensor:
        rows = torch.repeat_interleave(torch.arange(self.shape[0], device=self.device), self.indptr.long().diff())
        out = torch.zeros(self.shape, dtype=torch.float32, device=self.device)
        out.index_put_((rows, self.indices.long()), self.values, accumulate=True)
        return out

    def transpose(self) -> "CudaSparseTensor":
        rows = torch.repeat_interleave(torch.arange(self.shape[0], device=self.device), self.indptr.long().diff())
        return CudaSparseTensor.from_coo(CooTensor(self.indices.long(), rows, self.values, (self.shape[1], self.shape[0])))

    def matmul(self, b: torch.Tensor) -> torch.Tensor:
        """self [M, K] @ b [K, N] (or [K]) -> dense [M, N] in b's dtype."""
        vec = b.dim() == 1
        b2 = (b[:, None] if vec else b).contiguous()
        if b2.shape[0] != self.shape[1]:
            raise ValueError(f"shape mismatch: {self.shape} @ {tuple(b.shape)}")
        if self.values.is_cuda and b2.is_cuda and b2.dtype in (torch.bfloat16, torch.float32):
            from . import _native as nv
            from .ops import _dispatch as dp
            out = torch.empty(self.shape[0], b2.shape[1], dtype=b2.dtype, device=b2.device)
            dp.call("tb_csr_spmm", [dp.P, dp.P, dp.P, dp.P, dp.P, dp.I, dp.I, dp.I, dp.I, dp.P], self.indptr.data_ptr(),
                    self.indices.data_ptr(), self.values.data_ptr(), b2.data_ptr(), out.data_ptr(), self.shape[0], self.shape[1],
                    b2.shape[1], 0 if b2.dtype == torch.bfloat16 else 1, nv.stream_ptr())
        else:
            out = (self.to_dense() @ b2.float()).to(b2.dtype)
        return out[:, 0] if vec else out

    __matmul__ = matmul


class SparseLinear(torch.nn.Module):
    """Linear layer whose weight is held as COO non-zeros (trainable values, fixed pattern)."""

    def __init__(self, dense: torch.nn.Linear, sparsity: float = 0.9):
        super().__init__()
        w = prune_magnitude(dense.weight.detach(), sparsity)
        coo = CooTensor.from_dense(w)
        self.register_buffer("rows", coo.rows)
        self.register_buffer("cols", coo.cols)
        self.values = torch.nn.Parameter(coo.values.clone())
        self.bias = None if dense.bias is None else torch.nn.Parameter(dense.bias.detach().clone())
        self.shape = coo.shape

    def forward(self, x):
        y = CooTensor(self.rows, self.cols, self.values, self.shape).matmul(x.reshape(-1, x.shape[-1]).t()).t()
        y = y.reshape(*x.shape[:-1], self.shape[0])
        return y if self.bias is None else y + self.bias


def prune_magnitude(w: torch.Tensor, sparsity: float) -> torch.Tensor:
    k = int(w.numel() * sparsity)
    if k == 0:
        return w.clone()
    thr = w.abs().flatten().kthvalue(k).values
    return torch.where(w.abs() > thr, w, torch.zeros_like(w))
