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
